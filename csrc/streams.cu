// Several 32-bit residual streams (hyper-connections) and the scaled embedding with sinusoidal positions.
//
//   embed_sinusoid  x[s][t] = wte[tok_t] * scale + pe(p_t) for every stream s;  pe(p)[c] = sin(p f_(c/2)) for even c, cos for odd c,
//                   f_i given as 64-bit inverse frequencies (the angle p f_i is formed and reduced in 64-bit: positions reach far
//                   beyond what a 32-bit product resolves)
//   hyper_residual  write:  x_t <- sum_s mix[s][t] x_s + w_out[t] y      (every stream from the old ones, in place)
//                   read:   u = sum_s w_in[s] x_s ;  out = rms_div(u) * norm_w   (or u itself)
//                   One kernel does the write of one sub-layer and the read of the next: the streams are read once and written
//                   once per sub-layer -- the counterpart of norm_residual / dyt_residual / postnorm_residual for S streams.
//
// Streams are [S][T][W] 32-bit; sums, the norm and its root are 32-bit.
#include "common.cuh"

namespace {

constexpr int HS_MAX = 16;    // streams

template <typename T>
__global__ void __launch_bounds__(256) embed_sinusoid_kernel(const int* __restrict__ tokens, const int* __restrict__ positions,
                                                             const T* __restrict__ wte, const double* __restrict__ inv_freq,
                                                             float* __restrict__ out, int64_t Ttot, int W, int vocab, float scale,
                                                             int S) {
  const int64_t t = blockIdx.x;
  const int tok = min(max(tokens[t], 0), vocab - 1);
  const double p = (double)positions[t];
  const T* row = wte + (int64_t)tok * W;
  for (int c = threadIdx.x; c < W; c += blockDim.x) {
    const double ang = p * inv_freq[c >> 1];
    const float pe = (float)((c & 1) ? cos(ang) : sin(ang));
    const float v = to_f32(row[c]) * scale + pe;
    for (int s = 0; s < S; ++s) out[((int64_t)s * Ttot + t) * W + c] = v;
  }
}

__device__ __forceinline__ float block_sum256(float v, float* red) {
  v = warp_sum(v);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
  if (lane == 0) red[warp] = v;
  __syncthreads();
  float t = 0.f;
  for (int i = 0; i < nw; ++i) t += red[i];
  return t;
}

// one block per token row; VEC = 4: rows are read and written as float4 (W a multiple of 4, 16-byte aligned bases); NS: the
// largest stream count of the instantiation (1, 2, 4, 8 or HS_MAX: the per-thread arrays stay as small as the model's streams)
template <typename T, int VEC, int NS>
__global__ void __launch_bounds__(256) hyper_residual_kernel(float* __restrict__ xs, int64_t Ttot, int W, int S,
                                                             const float* __restrict__ y, int64_t ldy, const float* __restrict__ mix,
                                                             const float* __restrict__ w_out, const float* __restrict__ w_in,
                                                             const float* __restrict__ norm_w, float eps, T* __restrict__ out) {
  extern __shared__ __align__(16) float us[];     // [W] the read-out before its norm
  __shared__ float red[32], cm[HS_MAX * HS_MAX], co[HS_MAX], ci[HS_MAX];
  for (int i = threadIdx.x; i < S * S; i += blockDim.x) cm[i] = y != nullptr ? mix[i] : 0.f;
  if (threadIdx.x < S) {
    co[threadIdx.x] = y != nullptr ? w_out[threadIdx.x] : 0.f;
    ci[threadIdx.x] = w_in != nullptr ? w_in[threadIdx.x] : 0.f;
  }
  __syncthreads();
  const int64_t t = blockIdx.x;
  float ss = 0.f;
  for (int c = threadIdx.x * VEC; c < W; c += blockDim.x * VEC) {
    float x[NS][VEC], yv[VEC];
#pragma unroll
    for (int s = 0; s < NS; ++s) {
      if (s >= S) break;
      const float* p = xs + ((int64_t)s * Ttot + t) * W + c;
      if constexpr (VEC == 4) {
        const float4 v = *reinterpret_cast<const float4*>(p);
        x[s][0] = v.x; x[s][1 % VEC] = v.y; x[s][2 % VEC] = v.z; x[s][3 % VEC] = v.w;
      } else {
        x[s][0] = p[0];
      }
    }
    if (y != nullptr) {
      const float* p = y + t * ldy + c;
      if constexpr (VEC == 4) {
        const float4 v = *reinterpret_cast<const float4*>(p);
        yv[0] = v.x; yv[1 % VEC] = v.y; yv[2 % VEC] = v.z; yv[3 % VEC] = v.w;
      } else {
        yv[0] = p[0];
      }
      float n[NS][VEC];
#pragma unroll
      for (int d = 0; d < NS; ++d) {
        if (d >= S) break;
#pragma unroll
        for (int e = 0; e < VEC; ++e) {
          float acc = 0.f;
#pragma unroll
          for (int s = 0; s < NS; ++s) {
            if (s >= S) break;
            acc = fmaf(cm[s * S + d], x[s][e], acc);
          }
          n[d][e] = fmaf(co[d], yv[e], acc);
        }
      }
#pragma unroll
      for (int d = 0; d < NS; ++d) {
        if (d >= S) break;
        float* p2 = xs + ((int64_t)d * Ttot + t) * W + c;
        if constexpr (VEC == 4) *reinterpret_cast<float4*>(p2) = make_float4(n[d][0], n[d][1 % VEC], n[d][2 % VEC], n[d][3 % VEC]);
        else p2[0] = n[d][0];
#pragma unroll
        for (int e = 0; e < VEC; ++e) x[d][e] = n[d][e];
      }
    }
    if (w_in != nullptr) {
#pragma unroll
      for (int e = 0; e < VEC; ++e) {
        float acc = 0.f;
#pragma unroll
        for (int s = 0; s < NS; ++s) {
          if (s >= S) break;
          acc = fmaf(ci[s], x[s][e], acc);
        }
        us[c + e] = acc;
        ss = fmaf(acc, acc, ss);
      }
    }
  }
  if (w_in == nullptr) return;
  float r = 1.f;
  if (norm_w != nullptr) r = rsqrtf(block_sum256(ss, red) / W + eps);
  // every thread re-reads only the columns it wrote itself
  for (int c = threadIdx.x * VEC; c < W; c += blockDim.x * VEC) {
    float v[VEC];
#pragma unroll
    for (int e = 0; e < VEC; ++e) v[e] = norm_w != nullptr ? us[c + e] * r * norm_w[c + e] : us[c + e];
    if constexpr (VEC == 4) {
      if constexpr (sizeof(T) == 4) {
        *reinterpret_cast<float4*>(out + t * W + c) = make_float4(v[0], v[1 % VEC], v[2 % VEC], v[3 % VEC]);
      } else {
        __align__(8) T tmp[4] = {from_f32<T>(v[0]), from_f32<T>(v[1 % VEC]), from_f32<T>(v[2 % VEC]), from_f32<T>(v[3 % VEC])};
        *reinterpret_cast<uint2*>(out + t * W + c) = *reinterpret_cast<const uint2*>(tmp);
      }
    } else {
      out[t * W + c] = from_f32<T>(v[0]);
    }
  }
}

}  // namespace

LLMSS_API int llmss_embed_sinusoid(const int* tokens, const int* positions, const void* wte, const double* inv_freq, float* out, int T_,
                                   int W, int vocab, float scale, int streams, int dtype, cudaStream_t stream) {
  LLMSS_REQUIRE(streams >= 1 && W > 0 && vocab > 0, "embed_sinusoid: bad sizes");
  if (T_ <= 0) return 0;
  LLMSS_BY_DTYPE(dtype, (embed_sinusoid_kernel<T><<<T_, W >= 1024 ? 256 : 128, 0, stream>>>(tokens, positions, (const T*)wte, inv_freq, out,
                                                                                             (int64_t)T_, W, vocab, scale, streams)));
  LLMSS_CHECK_CUDA(cudaGetLastError());
  return 0;
}

LLMSS_API int llmss_hyper_residual(float* xs, int T_, int W, int streams, const float* y, int64_t ldy, const float* mix,
                                   const float* w_out, const float* w_in, const float* norm_w, float eps, void* out, int out_dtype,
                                   cudaStream_t stream) {
  LLMSS_REQUIRE(streams >= 1 && streams <= HS_MAX, "hyper_residual: %d streams (at most %d)", streams, HS_MAX);
  LLMSS_REQUIRE((y == nullptr) == (mix == nullptr) && (y == nullptr) == (w_out == nullptr), "hyper_residual: y, mix and w_out go together");
  LLMSS_REQUIRE(w_in != nullptr || norm_w == nullptr, "hyper_residual: a norm needs a read-out");
  LLMSS_REQUIRE(w_in == nullptr || out != nullptr, "hyper_residual: a read-out needs an output");
  if (T_ <= 0 || (y == nullptr && w_in == nullptr)) return 0;
  const size_t smem = w_in != nullptr ? sizeof(float) * (size_t)W : 0;
  LLMSS_REQUIRE(smem <= 200 * 1024, "hyper_residual: width %d exceeds shared memory", W);
  const bool vec = W % 4 == 0 && ((uintptr_t)xs & 15) == 0 && (y == nullptr || (((uintptr_t)y & 15) == 0 && ldy % 4 == 0));
  const int threads = W >= 1024 ? 256 : 128;
#define LLMSS_HR(TT, V, N)                                                                                          \
  do {                                                                                                              \
    static PerDeviceSmem gsm;                                                                                       \
    if (smem > 48 * 1024) LLMSS_CHECK_CUDA(gsm.ensure(hyper_residual_kernel<TT, V, N>, (int)smem));                 \
    hyper_residual_kernel<TT, V, N><<<T_, threads, smem, stream>>>(xs, (int64_t)T_, W, streams, y, ldy, mix, w_out, \
                                                                   w_in, norm_w, eps, (TT*)out);                    \
  } while (0)
#define LLMSS_HR_N(TT, V)                      \
  do {                                         \
    if (streams <= 1) LLMSS_HR(TT, V, 1);      \
    else if (streams <= 2) LLMSS_HR(TT, V, 2); \
    else if (streams <= 4) LLMSS_HR(TT, V, 4); \
    else if (streams <= 8) LLMSS_HR(TT, V, 8); \
    else LLMSS_HR(TT, V, HS_MAX);              \
  } while (0)
  if (vec) LLMSS_BY_DTYPE(out_dtype, LLMSS_HR_N(T, 4));
  else LLMSS_BY_DTYPE(out_dtype, LLMSS_HR_N(T, 1));
#undef LLMSS_HR_N
#undef LLMSS_HR
  LLMSS_CHECK_CUDA(cudaGetLastError());
  return 0;
}

// 32-bit residual stream: layer-scaled branch sum + Dynamic Tanh, 32-bit embedding, cast + concat.
//
// Dynamic Tanh is a statistics-free norm: y = tanh(alpha * x) * w + b with a learned scalar alpha, so the
// kernel is a pure element-wise pass (no reduction).  dyt_residual is to it what norm_residual is to
// LayerNorm / RMSNorm: it first folds the outputs of the previous layer's branches into the residual,
//     r' = r + s1 * a + s2 * b          (s1, s2: per-feature layer scales; a, b: 32-bit branch outputs)
// keeps r' in 32-bit and emits the normed activation in the compute type for the next GEMM.
// T is the compute / weight type (half, bf16 or float).
#include "common.cuh"

namespace {

template <typename T>
__global__ void __launch_bounds__(256) dyt_residual_kernel(const float* res_in, float* res_out, const float* a,
                                                           const T* __restrict__ s1, const float* b,
                                                           const T* __restrict__ s2, const T* __restrict__ w,
                                                           const T* __restrict__ bias, T* __restrict__ out, float alpha,
                                                           int H, int64_t ldr, int64_t lda, int64_t ldb, int64_t ldo) {
  const int64_t row = blockIdx.x;
  for (int c = threadIdx.x; c < H; c += blockDim.x) {
    float v = res_in[row * ldr + c];
    if (a != nullptr) v += (s1 != nullptr ? to_f32(s1[c]) : 1.f) * a[row * lda + c];
    if (b != nullptr) v += (s2 != nullptr ? to_f32(s2[c]) : 1.f) * b[row * ldb + c];
    if (res_out != nullptr) res_out[row * ldr + c] = v;
    if (out != nullptr) {
      float y = tanhf(alpha * v) * to_f32(w[c]);
      if (bias != nullptr) y += to_f32(bias[c]);
      out[row * ldo + c] = from_f32<T>(y);
    }
  }
}

template <typename T>
__global__ void __launch_bounds__(128) embed_f32_kernel(const int* __restrict__ tokens, const int* __restrict__ positions,
                                                        const T* __restrict__ wte, const T* __restrict__ wpe,
                                                        float* __restrict__ out, int H, int vocab, int max_pos,
                                                        int pos_offset, int64_t ldo, float scale) {
  const int t = blockIdx.x;
  const int tok = min(max(tokens[t], 0), vocab - 1);
  const T* src = wte + (int64_t)tok * H;
  const T* psrc = nullptr;
  if (wpe != nullptr) psrc = wpe + (int64_t)min(max(positions[t] + pos_offset, 0), max_pos - 1) * H;
  for (int c = threadIdx.x; c < H; c += blockDim.x) {
    float v = to_f32(src[c]) * scale;
    if (psrc != nullptr) v += to_f32(psrc[c]);
    out[(int64_t)t * ldo + c] = v;
  }
}

template <typename T>
__global__ void __launch_bounds__(256) cast_concat_kernel(const float* __restrict__ a, const float* __restrict__ b,
                                                          T* __restrict__ out, int Ha, int Hb, int64_t lda, int64_t ldb,
                                                          int64_t ldo) {
  const int64_t row = blockIdx.x;
  for (int c = threadIdx.x; c < Ha + Hb; c += blockDim.x) {
    const float v = c < Ha ? a[row * lda + c] : b[row * ldb + (c - Ha)];
    out[row * ldo + c] = from_f32<T>(v);
  }
}

}  // namespace

LLMSS_API int llmss_dyt_residual(const float* res_in, float* res_out, const float* a, const void* s1, const float* b,
                                 const void* s2, const void* w, const void* bias, void* out, float alpha, int M, int H,
                                 int64_t ldr, int64_t lda, int64_t ldb, int64_t ldo, int dtype, cudaStream_t stream) {
  if (M == 0) return 0;
  LLMSS_BY_DTYPE(dtype, (dyt_residual_kernel<T><<<M, 256, 0, stream>>>(res_in, res_out, a, (const T*)s1, b, (const T*)s2,
                                                                       (const T*)w, (const T*)bias, (T*)out, alpha, H, ldr,
                                                                       lda, ldb, ldo)));
  LLMSS_CHECK_CUDA(cudaGetLastError());
  return 0;
}

// out[t] = wte[tok_t] * scale (+ wpe[pos_t]) in 32-bit
LLMSS_API int llmss_embed_scaled_f32(const int* tokens, const int* positions, const void* wte, const void* wpe, float* out, int T_,
                                     int H, int vocab, int max_pos, int pos_offset, int64_t ldo, float scale, int dtype,
                                     cudaStream_t stream) {
  if (T_ == 0) return 0;
  LLMSS_BY_DTYPE(dtype, (embed_f32_kernel<T><<<T_, 128, 0, stream>>>(tokens, positions, (const T*)wte, (const T*)wpe, out, H,
                                                                    vocab, max_pos, pos_offset, ldo, scale)));
  LLMSS_CHECK_CUDA(cudaGetLastError());
  return 0;
}

LLMSS_API int llmss_embed_f32(const int* tokens, const int* positions, const void* wte, const void* wpe, float* out, int T_,
                              int H, int vocab, int max_pos, int pos_offset, int64_t ldo, int dtype, cudaStream_t stream) {
  return llmss_embed_scaled_f32(tokens, positions, wte, wpe, out, T_, H, vocab, max_pos, pos_offset, ldo, 1.f, dtype, stream);
}

LLMSS_API int llmss_cast_concat(const float* a, const float* b, void* out, int M, int Ha, int Hb, int64_t lda, int64_t ldb,
                                int64_t ldo, int dtype, cudaStream_t stream) {
  if (M == 0) return 0;
  LLMSS_BY_DTYPE(dtype, (cast_concat_kernel<T><<<M, 256, 0, stream>>>(a, b, (T*)out, Ha, Hb, lda, ldb, ldo)));
  LLMSS_CHECK_CUDA(cudaGetLastError());
  return 0;
}

// Rotation by a frequency table, and the element-wise / per-row steps around it.
//
//   rope_norm_kv_write : grouped-query attention whose values are the projected keys.  q and k are rotated (pairs (2i, 2i+1) or
//                        (i, i + n)), optionally every head is divided by its root mean square, the prepared keys go to the K
//                        pages, the raw key projection to the V pages, the queries out in the compute type.
//   latent_rope_prep   : latent attention with a rotated key part, first stage: RMS norm of the query latent (-> GEMM operand),
//                        RMS norm of the key / value latent and rotation of the shared key part (-> one cache row), sigmoid of
//                        the gate columns.
//   latent_query_rope  : second stage: per head, the unrotated query part (-> operand of the absorption) and the rotated part
//                        (-> its columns of the absorbed-query buffer).
//   hgrn_gates         : q = silu(q), k = 1 - f, ln f with f = lower + (1 - lower) sigmoid(f_raw).
//   sandwich_residual  : r = resid + rms_div(y) * w_post; optional store as a layer output and depth-weighted average of the
//                        outputs so far; h = rms_div(r) * w_next.  One CTA per token.
//   softcap            : z <- cap * tanh(z / cap).
//
// Every rotation takes its frequencies as a 64-bit table [n] (n pairs: the first 2 n channels rotate, the rest pass) and a
// magnitude that multiplies cos and sin, so linear interpolation, YaRN or any other schedule is a different table.  The angle
// position * frequency is formed and reduced to [-pi, pi] in 64-bit once per token and pair.  Everything else is 32-bit.
#include "common.cuh"

namespace {

constexpr int kMaxPairs = 256;      // rotated pairs per head (512 rotated channels)

// cos / sin of this token's angles into shared memory.  The angle position * frequency and its reduction to [-pi, pi] are
// 64-bit (one multiply, one rounding, one fused multiply-add); cosine and sine of the reduced angle are 32-bit.
__device__ __forceinline__ void token_angles(const double* __restrict__ freq, int n, int pos, float mag, float* cs, float* sn) {
  constexpr double kTwoPi = 6.283185307179586476925286766559;
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    const double a = (double)pos * freq[i];
    const float r = (float)fma(-rint(a * (1.0 / kTwoPi)), kTwoPi, a);
    float s, c;
    sincosf(r, &s, &c);
    cs[i] = c * mag;
    sn[i] = s * mag;
  }
}

// channel c of a head after rotation; x points at the head's first channel
__device__ __forceinline__ float rotated(const float* __restrict__ x, int c, int n, bool interleaved, const float* cs, const float* sn) {
  if (c >= 2 * n) return x[c];
  if (interleaved) {
    const int i = c >> 1;
    return (c & 1) ? fmaf(x[c], cs[i], x[c - 1] * sn[i]) : fmaf(x[c], cs[i], -x[c + 1] * sn[i]);
  }
  return c < n ? fmaf(x[c], cs[c], -x[c + n] * sn[c]) : fmaf(x[c], cs[c - n], x[c - n] * sn[c - n]);
}

// grid T, block 256; the token's row is staged in shared memory (16-byte loads where the row allows), then the warps walk
// its hq + hkv heads.  STAGE = false: rows too long for shared memory are read in place.
template <typename T, bool STAGE>
__global__ void __launch_bounds__(256) rope_norm_kv_write_kernel(const float* __restrict__ qk, int64_t ld, int hq, int hkv, int d,
                                                                 const double* __restrict__ freq, int n, float mag, int interleaved,
                                                                 int unit_norm, float eps, const int* __restrict__ positions,
                                                                 const int* __restrict__ slots, T* __restrict__ k_cache,
                                                                 T* __restrict__ v_cache, int bs, T* __restrict__ q_out) {
  __shared__ float cs[kMaxPairs], sn[kMaxPairs];
  extern __shared__ __align__(16) float rowbuf[];
  const int64_t t = blockIdx.x;
  token_angles(freq, n, positions[t], mag, cs, sn);
  const float* src = qk + t * ld;
  if constexpr (STAGE) {
    const int cols = (hq + hkv) * d;
    if ((cols & 3) == 0 && (ld & 3) == 0 && (((uintptr_t)qk) & 15) == 0) {
      for (int c = threadIdx.x * 4; c < cols; c += 1024) *reinterpret_cast<float4*>(rowbuf + c) = *reinterpret_cast<const float4*>(src + c);
    } else {
      for (int c = threadIdx.x; c < cols; c += 256) rowbuf[c] = src[c];
    }
    src = rowbuf;
  }
  __syncthreads();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int slot = slots[t];
  if constexpr (STAGE) {
    // A lane owns whole pairs: it rotates them in place in the staged row (one pass, both outputs of a pair at once) and sums
    // the squares; the second pass scales and stores in channel order.  The projected keys leave for the V pages first.
    for (int hh = warp; hh < hq + hkv; hh += 8) {
      float* x = rowbuf + (int64_t)hh * d;
      const bool is_k = hh >= hq;
      const int64_t base = is_k && slot >= 0 ? (((int64_t)(slot / bs) * hkv + (hh - hq)) * bs + slot % bs) * d : 0;
      if (is_k && slot >= 0)
        for (int c = lane; c < d; c += 32) v_cache[base + c] = from_f32<T>(x[c]);
      __syncwarp();
      float ss = 0.f;
      for (int i = lane; i < n; i += 32) {
        const int iu = interleaved ? 2 * i : i, iv = interleaved ? 2 * i + 1 : i + n;
        const float u = x[iu], v = x[iv], c = cs[i], sgn = sn[i];
        const float ou = fmaf(u, c, -v * sgn), ov = fmaf(v, c, u * sgn);
        x[iu] = ou;
        x[iv] = ov;
        ss = fmaf(ou, ou, fmaf(ov, ov, ss));
      }
      if (unit_norm)
        for (int c = 2 * n + lane; c < d; c += 32) ss = fmaf(x[c], x[c], ss);
      const float rstd = unit_norm ? rsqrtf(warp_sum(ss) / (float)d + eps) : 1.f;
      __syncwarp();
      if (!is_k) {
        T* o = q_out + t * (int64_t)hq * d + (int64_t)hh * d;
        for (int c = lane; c < d; c += 32) o[c] = from_f32<T>(x[c] * rstd);
      } else if (slot >= 0) {
        for (int c = lane; c < d; c += 32) k_cache[base + c] = from_f32<T>(x[c] * rstd);
      }
    }
    return;
  }
  for (int hh = warp; hh < hq + hkv; hh += 8) {
    const float* x = src + (int64_t)hh * d;
    float rstd = 1.f;
    if (unit_norm) {
      float ss = 0.f;
      for (int c = lane; c < d; c += 32) { const float r = rotated(x, c, n, interleaved, cs, sn); ss = fmaf(r, r, ss); }
      rstd = rsqrtf(warp_sum(ss) / (float)d + eps);
    }
    if (hh < hq) {
      T* o = q_out + t * (int64_t)hq * d + (int64_t)hh * d;
      for (int c = lane; c < d; c += 32) o[c] = from_f32<T>(rotated(x, c, n, interleaved, cs, sn) * rstd);
    } else if (slot >= 0) {
      const int g = hh - hq;
      const int64_t base = (((int64_t)(slot / bs) * hkv + g) * bs + slot % bs) * d;
      for (int c = lane; c < d; c += 32) {
        k_cache[base + c] = from_f32<T>(rotated(x, c, n, interleaved, cs, sn) * rstd);
        v_cache[base + c] = from_f32<T>(x[c]);
      }
    }
  }
}

__device__ __forceinline__ float block_sum_256(float v, float* red) {
  v = warp_sum(v);
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
  __syncthreads();
  if (l == 0) red[w] = v;
  __syncthreads();
  return warp_sum(l < 8 ? red[l] : 0.f);
}

// grid T, block 256
template <typename T>
__global__ void __launch_bounds__(256) latent_rope_prep_kernel(const float* __restrict__ y, int64_t ldy, int q_off, int q_rank, int c_off,
                                                               int R, int rot, int g_off, int n_gate, const float* __restrict__ qn_w,
                                                               const float* __restrict__ cn_w, float eps, const double* __restrict__ freq,
                                                               int n, float mag, const int* __restrict__ positions,
                                                               const int* __restrict__ slots, T* __restrict__ cache, int width,
                                                               T* __restrict__ cq_out, float* __restrict__ gate) {
  __shared__ float cs[kMaxPairs], sn[kMaxPairs], red[8];
  const int64_t t = blockIdx.x;
  const float* row = y + t * ldy;
  token_angles(freq, n, positions[t], mag, cs, sn);
  if (q_rank > 0) {
    float ss = 0.f;
    for (int i = threadIdx.x; i < q_rank; i += 256) ss = fmaf(row[q_off + i], row[q_off + i], ss);
    const float rstd = rsqrtf(block_sum_256(ss, red) / (float)q_rank + eps);
    for (int i = threadIdx.x; i < q_rank; i += 256) cq_out[t * q_rank + i] = from_f32<T>(row[q_off + i] * rstd * qn_w[i]);
  }
  float ss = 0.f;
  for (int i = threadIdx.x; i < R; i += 256) ss = fmaf(row[c_off + i], row[c_off + i], ss);
  const float rstd = rsqrtf(block_sum_256(ss, red) / (float)R + eps);      // (its barriers also publish cs / sn)
  const int slot = slots[t];
  if (slot >= 0) {
    T* dst = cache + (int64_t)slot * width;
    for (int i = threadIdx.x; i < R; i += 256) dst[i] = from_f32<T>(row[c_off + i] * rstd * cn_w[i]);
    const float* kr = row + c_off + R;
    for (int c = threadIdx.x; c < rot; c += 256) dst[R + c] = from_f32<T>(rotated(kr, c, n, true, cs, sn));
    for (int c = R + rot + threadIdx.x; c < width; c += 256) dst[c] = from_f32<T>(0.f);
  }
  for (int i = threadIdx.x; i < n_gate; i += 256) gate[t * n_gate + i] = 1.f / (1.f + expf(-row[g_off + i]));
}

// grid T, block 256; q [T, H * (d + rot)] 32-bit
template <typename T, typename TA>
__global__ void __launch_bounds__(256) latent_query_rope_kernel(const float* __restrict__ q, int64_t ldq, int H, int d, int rot, int R,
                                                                int width, const double* __restrict__ freq, int n, float mag,
                                                                const int* __restrict__ positions, T* __restrict__ q_nope,
                                                                TA* __restrict__ q_abs) {
  __shared__ float cs[kMaxPairs], sn[kMaxPairs];
  const int64_t t = blockIdx.x;
  token_angles(freq, n, positions[t], mag, cs, sn);
  __syncthreads();
  const float* row = q + t * ldq;
  for (int i = threadIdx.x; i < H * d; i += 256) {
    const int h = i / d, c = i - h * d;
    q_nope[t * (int64_t)H * d + i] = from_f32<T>(row[(int64_t)h * (d + rot) + c]);
  }
  const int tail = width - R;          // rotated part, then zero padding
  for (int i = threadIdx.x; i < H * tail; i += 256) {
    const int h = i / tail, c = i - h * tail;
    const float v = c < rot ? rotated(row + (int64_t)h * (d + rot) + d, c, n, true, cs, sn) : 0.f;
    q_abs[t * (int64_t)H * width + (int64_t)h * width + R + c] = from_f32<TA>(v);
  }
}

__global__ void __launch_bounds__(256) hgrn_gates_kernel(const float* __restrict__ y, int64_t ldy, int nqk, const float* __restrict__ lower,
                                                         float* __restrict__ q, float* __restrict__ k, float* __restrict__ lnf,
                                                         int64_t total) {
  const int64_t i = (int64_t)blockIdx.x * 256 + threadIdx.x;
  if (i >= total) return;
  const int64_t t = i / nqk;
  const int c = (int)(i - t * nqk);
  const float qr = y[t * ldy + c], z = y[t * ldy + nqk + c], lo = lower[c];
  const float sg = 1.f / (1.f + expf(-z));
  q[i] = qr / (1.f + expf(-qr));
  k[i] = (1.f - lo) * (1.f / (1.f + expf(z)));       // 1 - f without cancellation
  lnf[i] = logf(lo + (1.f - lo) * sg);
}

__global__ void __launch_bounds__(256) softcap_kernel(float* __restrict__ z, int64_t ldz, int cols, float cap, int64_t total) {
  const int64_t i = (int64_t)blockIdx.x * 256 + threadIdx.x;
  if (i >= total) return;
  float* p = z + (i / cols) * ldz + (i % cols);
  *p = cap * tanhf(*p / cap);
}

// ------------------------------------------------------------------------------------------------ sandwich_residual
struct SwArgs {
  const float* resid; int64_t ldr;     // [T, W]
  const float* y; int64_t ldy;         // sub-layer output [T, W] or null
  const float* w_post;                 // [W] (with y)
  float* hist; int64_t plane;          // layer outputs [n, T, W] (plane = T * W) or null
  int index;                           // r is stored as output `index`
  const float* depth_w;                // [index + 1] or null: r <- sum_j depth_w[j] * hist[j]
  const float* w_next;                 // [W] or null
  float* out_r;                        // [T, W] new residual
  void* out_h;                         // [T, W] normed, TO
  int W; float eps;
};

constexpr int kSwRegs = 4;             // columns kept in registers per thread and pass: W <= 256 * VEC * kSwRegs, else re-read

template <int VEC> __device__ __forceinline__ void ldv(const float* p, float (&v)[VEC]) {
  if constexpr (VEC == 4) {
    const float4 x = *reinterpret_cast<const float4*>(p);
    v[0] = x.x; v[1] = x.y; v[2] = x.z; v[3] = x.w;
  } else v[0] = p[0];
}
template <int VEC> __device__ __forceinline__ void stv(float* p, const float (&v)[VEC]) {
  if constexpr (VEC == 4) *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
  else p[0] = v[0];
}

// columns c .. c + VEC - 1 of row t: the new residual (stored as a layer output and averaged, if asked)
template <int VEC>
__device__ __forceinline__ void sandwich_columns(const SwArgs& a, int64_t t, int c, float rstd_y, float (&r)[VEC]) {
  ldv<VEC>(a.resid + t * a.ldr + c, r);
  if (a.y != nullptr) {
    float yv[VEC], wv[VEC];
    ldv<VEC>(a.y + t * a.ldy + c, yv);
    ldv<VEC>(a.w_post + c, wv);
#pragma unroll
    for (int e = 0; e < VEC; ++e) r[e] = fmaf(yv[e] * rstd_y, wv[e], r[e]);
  }
  if (a.hist != nullptr) {
    stv<VEC>(a.hist + (int64_t)a.index * a.plane + t * (int64_t)a.W + c, r);
    if (a.depth_w != nullptr) {
      const float wi = a.depth_w[a.index];
#pragma unroll
      for (int e = 0; e < VEC; ++e) r[e] *= wi;
      for (int j = 0; j < a.index; ++j) {
        const float wj = a.depth_w[j];
        float v[VEC];
        ldv<VEC>(a.hist + (int64_t)j * a.plane + t * (int64_t)a.W + c, v);
#pragma unroll
        for (int e = 0; e < VEC; ++e) r[e] = fmaf(wj, v[e], r[e]);
      }
    }
  }
  stv<VEC>(a.out_r + t * (int64_t)a.W + c, r);
}

template <typename TO, int VEC>
__device__ __forceinline__ void sandwich_emit(const SwArgs& a, int64_t t, int c, float rstd, const float (&r)[VEC]) {
  TO* ho = reinterpret_cast<TO*>(a.out_h) + t * (int64_t)a.W + c;
  float wv[VEC];
  ldv<VEC>(a.w_next + c, wv);
  if constexpr (VEC == 4) {
    struct alignas(4 * sizeof(TO)) V4 { TO v[4]; };
    V4 o;
#pragma unroll
    for (int e = 0; e < 4; ++e) o.v[e] = from_f32<TO>(r[e] * rstd * wv[e]);
    *reinterpret_cast<V4*>(ho) = o;
  } else ho[0] = from_f32<TO>(r[0] * rstd * wv[0]);
}

template <typename TO, int VEC>
__global__ void __launch_bounds__(256, 5) sandwich_residual_kernel(SwArgs a) {
  __shared__ float red[8];
  const int64_t t = blockIdx.x;
  const int W = a.W;
  constexpr int STEP = 256 * VEC;
  float rstd_y = 0.f;
  if (a.y != nullptr) {
    const float* yr = a.y + t * a.ldy;
    float ss = 0.f;
    for (int c = threadIdx.x * VEC; c < W; c += STEP) {
      float v[VEC];
      ldv<VEC>(yr + c, v);
#pragma unroll
      for (int e = 0; e < VEC; ++e) ss = fmaf(v[e], v[e], ss);
    }
    rstd_y = rsqrtf(block_sum_256(ss, red) / (float)W + a.eps);
  }
  float keep[kSwRegs][VEC];
  float ss = 0.f;
#pragma unroll
  for (int it = 0; it < kSwRegs; ++it) {
    const int c = threadIdx.x * VEC + it * STEP;
    if (c < W) {
      sandwich_columns<VEC>(a, t, c, rstd_y, keep[it]);
#pragma unroll
      for (int e = 0; e < VEC; ++e) ss = fmaf(keep[it][e], keep[it][e], ss);
    }
  }
  for (int c = threadIdx.x * VEC + kSwRegs * STEP; c < W; c += STEP) {
    float r[VEC];
    sandwich_columns<VEC>(a, t, c, rstd_y, r);
#pragma unroll
    for (int e = 0; e < VEC; ++e) ss = fmaf(r[e], r[e], ss);
  }
  if (a.w_next == nullptr) return;
  const float rstd = rsqrtf(block_sum_256(ss, red) / (float)W + a.eps);
#pragma unroll
  for (int it = 0; it < kSwRegs; ++it) {
    const int c = threadIdx.x * VEC + it * STEP;
    if (c < W) sandwich_emit<TO, VEC>(a, t, c, rstd, keep[it]);
  }
  for (int c = threadIdx.x * VEC + kSwRegs * STEP; c < W; c += STEP) {     // beyond the registers: this thread's own stores
    float r[VEC];
    ldv<VEC>(a.out_r + t * (int64_t)W + c, r);
    sandwich_emit<TO, VEC>(a, t, c, rstd, r);
  }
}

template <typename TO>
int sandwich_launch(const SwArgs& a, int T_, bool vec, cudaStream_t stream) {
  if (vec) sandwich_residual_kernel<TO, 4><<<T_, 256, 0, stream>>>(a);
  else sandwich_residual_kernel<TO, 1><<<T_, 256, 0, stream>>>(a);
  LLMSS_CHECK_CUDA(cudaGetLastError());
  return 0;
}

}  // namespace

LLMSS_API int llmss_rope_norm_kv_write(const float* qk, int64_t ld, int hq, int hkv, int d, const double* freq, int n_pairs, float mag,
                                       int interleaved, int unit_norm, float eps, const int* positions, const int* slots,
                                       void* k_cache, void* v_cache, int block_size, void* q_out, int T_, int dtype,
                                       cudaStream_t stream) {
  LLMSS_REQUIRE(hq > 0 && hkv > 0 && d > 0, "rope_norm_kv_write: bad sizes");
  LLMSS_REQUIRE(n_pairs >= 0 && n_pairs <= kMaxPairs && 2 * n_pairs <= d, "rope_norm_kv_write: %d rotated pairs for head size %d (at most %d)",
                n_pairs, d, kMaxPairs);
  if (T_ <= 0) return 0;
  const size_t row_bytes = sizeof(float) * (size_t)(hq + hkv) * d;
  if (row_bytes <= 40 * 1024) {      // within the default dynamic shared memory: the row is staged
    LLMSS_BY_DTYPE(dtype, (rope_norm_kv_write_kernel<T, true><<<T_, 256, row_bytes, stream>>>(
                              qk, ld, hq, hkv, d, freq, n_pairs, mag, interleaved, unit_norm, eps, positions, slots, (T*)k_cache,
                              (T*)v_cache, block_size, (T*)q_out)));
  } else {
    LLMSS_BY_DTYPE(dtype, (rope_norm_kv_write_kernel<T, false><<<T_, 256, 0, stream>>>(
                              qk, ld, hq, hkv, d, freq, n_pairs, mag, interleaved, unit_norm, eps, positions, slots, (T*)k_cache,
                              (T*)v_cache, block_size, (T*)q_out)));
  }
  LLMSS_CHECK_CUDA(cudaGetLastError());
  return 0;
}

LLMSS_API int llmss_latent_rope_prep(const float* y, int64_t ldy, int q_off, int q_rank, int c_off, int rank, int rot, int g_off,
                                     int n_gate, const float* qn_w, const float* cn_w, float eps, const double* freq, int n_pairs,
                                     float mag, const int* positions, const int* slots, void* cache, int width, void* cq_out,
                                     float* gate, int T_, int dtype, cudaStream_t stream) {
  LLMSS_REQUIRE(rank > 0 && rot >= 0 && width >= rank + rot, "latent_rope_prep: cache row %d for rank %d + %d rotated", width, rank, rot);
  LLMSS_REQUIRE(n_pairs >= 0 && n_pairs <= kMaxPairs && 2 * n_pairs <= rot, "latent_rope_prep: %d rotated pairs for %d channels", n_pairs, rot);
  if (T_ <= 0) return 0;
  LLMSS_BY_DTYPE(dtype, (latent_rope_prep_kernel<T><<<T_, 256, 0, stream>>>(y, ldy, q_off, q_rank, c_off, rank, rot, g_off, n_gate, qn_w, cn_w,
                                                                           eps, freq, n_pairs, mag, positions, slots, (T*)cache, width,
                                                                           (T*)cq_out, gate)));
  LLMSS_CHECK_CUDA(cudaGetLastError());
  return 0;
}

// abs_f32: the absorbed-query buffer is 32-bit (generic attention kernel), else it has the compute type
LLMSS_API int llmss_latent_query_rope(const float* q, int64_t ldq, int H, int d, int rot, int rank, int width, const double* freq,
                                      int n_pairs, float mag, const int* positions, void* q_nope, void* q_abs, int abs_f32, int T_,
                                      int dtype, cudaStream_t stream) {
  LLMSS_REQUIRE(H > 0 && d > 0 && width >= rank + rot, "latent_query_rope: bad sizes");
  LLMSS_REQUIRE(n_pairs >= 0 && n_pairs <= kMaxPairs && 2 * n_pairs <= rot, "latent_query_rope: %d rotated pairs for %d channels", n_pairs, rot);
  if (T_ <= 0) return 0;
  if (abs_f32 || dtype == LLMSS_F32) {
    LLMSS_BY_DTYPE(dtype, (latent_query_rope_kernel<T, float><<<T_, 256, 0, stream>>>(q, ldq, H, d, rot, rank, width, freq, n_pairs, mag,
                                                                                     positions, (T*)q_nope, (float*)q_abs)));
  } else {
    LLMSS_BY_DTYPE(dtype, (latent_query_rope_kernel<T, T><<<T_, 256, 0, stream>>>(q, ldq, H, d, rot, rank, width, freq, n_pairs, mag,
                                                                                 positions, (T*)q_nope, (T*)q_abs)));
  }
  LLMSS_CHECK_CUDA(cudaGetLastError());
  return 0;
}

LLMSS_API int llmss_hgrn_gates(const float* y, int64_t ldy, int n_qk, const float* lower, float* q, float* k, float* logf, int T_,
                               cudaStream_t stream) {
  if (T_ <= 0 || n_qk <= 0) return 0;
  const int64_t total = (int64_t)T_ * n_qk;
  hgrn_gates_kernel<<<(unsigned)((total + 255) / 256), 256, 0, stream>>>(y, ldy, n_qk, lower, q, k, logf, total);
  LLMSS_CHECK_CUDA(cudaGetLastError());
  return 0;
}

LLMSS_API int llmss_softcap(float* z, int64_t ldz, int rows, int cols, float cap, cudaStream_t stream) {
  LLMSS_REQUIRE(cap > 0.f, "softcap: cap %f", cap);
  if (rows <= 0 || cols <= 0) return 0;
  const int64_t total = (int64_t)rows * cols;
  softcap_kernel<<<(unsigned)((total + 255) / 256), 256, 0, stream>>>(z, ldz, cols, cap, total);
  LLMSS_CHECK_CUDA(cudaGetLastError());
  return 0;
}

// hist: [n, T, W] contiguous planes (or null); out_r [T, W] contiguous; out_h [T, W] contiguous in out_dtype (or null with w_next)
LLMSS_API int llmss_sandwich_residual(const float* resid, int64_t ldr, const float* y, int64_t ldy, const float* w_post, float* hist,
                                      int index, const float* depth_w, const float* w_next, float* out_r, void* out_h, int T_, int W,
                                      float eps, int out_dtype, cudaStream_t stream) {
  LLMSS_REQUIRE(W > 0 && (y == nullptr || w_post != nullptr) && (w_next == nullptr || out_h != nullptr), "sandwich_residual: bad arguments");
  LLMSS_REQUIRE(depth_w == nullptr || hist != nullptr, "sandwich_residual: averaging needs the layer outputs");
  if (T_ <= 0) return 0;
  SwArgs a{resid, ldr, y, ldy, w_post, hist, (int64_t)T_ * W, index, depth_w, w_next, out_r, out_h, W, eps};
  const bool vec = W % 4 == 0 && ldr % 4 == 0 && ldy % 4 == 0 &&
                   ((((uintptr_t)resid) | ((uintptr_t)y) | ((uintptr_t)hist) | ((uintptr_t)out_r) | ((uintptr_t)out_h) |
                     ((uintptr_t)w_post) | ((uintptr_t)w_next)) & 15) == 0;
  LLMSS_BY_DTYPE(out_dtype, return (sandwich_launch<T>(a, T_, vec, stream)));
}

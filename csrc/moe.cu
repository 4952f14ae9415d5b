// Routed mixture of experts: grouped top-k router and the per-token expert products.
//
//   moe_route : scores s = softmax(z) or sigmoid(z) over all E experts (32-bit); experts are chosen by s plus an optional
//               per-expert correction, weighted by s itself; the experts form `groups` equal groups of neighbours, a
//               group scores as its best expert (or as the sum of its few best), only experts of the `keep` best groups
//               are eligible; the `top` eligible experts with the largest choice scores are chosen; weights = s_chosen
//               (/ (sum + 1e-20) if renormalised) * route_scale.  Ties go to the lower index.  One warp per token.
//   moe_up    : a[t, k, :] = act(W_up[e_k] h_t)            one warp per output feature, weights read row-wise
//   moe_down  : y[t, :]    = sum_k w_k W_down[e_k] a[t, k] 32-bit output; the experts' down matrices lie side by side
//               in one [W, E * F] tensor (row stride ldd), which is also the dense form's GEMM operand
// The two expert kernels gather the chosen experts' weight rows per token: the form for decode and short
// portions, where every token touches its own few experts and the pass is bound by those weight bytes.
// Long prompts use the dense form instead (all experts through the tensor-core GEMM, unchosen ones weighted 0).
#include "common.cuh"

namespace {

constexpr int kMaxPerLane = 8;   // experts per lane: E <= 256

constexpr int kMaxGroupTop = 4;  // a group scores as the sum of at most this many of its best experts

// score_kind 0: s = softmax(z); 1: s = sigmoid(z).  Experts are chosen by c = s + correction (correction may be null); the
// weights are the chosen experts' s.  A group scores as the sum of its `group_top` largest c (1: its best expert).
// renorm: weights / (their sum + 1e-20).  Experts outside the kept groups are never chosen, whatever the sign of c.
__global__ void __launch_bounds__(128) moe_route_kernel(const float* __restrict__ z, int64_t ldz, int E, int top, int groups,
                                                        int keep, float route_scale, int score_kind,
                                                        const float* __restrict__ correction, int group_top, int renorm,
                                                        int* __restrict__ ids, float* __restrict__ wts,
                                                        float* __restrict__ dense, int T) {
  __shared__ float cs_all[4][32 * kMaxPerLane];
  const int t = blockIdx.x * 4 + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (t >= T) return;
  float* cs = cs_all[threadIdx.x >> 5];
  const float* zr = z + (int64_t)t * ldz;
  float s[kMaxPerLane], c[kMaxPerLane];
  bool ok[kMaxPerLane];
  float mx = -INFINITY;
#pragma unroll
  for (int i = 0; i < kMaxPerLane; ++i) {
    const int e = lane + i * 32;
    s[i] = e < E ? zr[e] : -INFINITY;
    mx = fmaxf(mx, s[i]);
  }
  if (score_kind == 0) {
    mx = warp_max(mx);
    float sum = 0.f;
#pragma unroll
    for (int i = 0; i < kMaxPerLane; ++i) {
      const int e = lane + i * 32;
      s[i] = e < E ? expf(s[i] - mx) : 0.f;
      sum += s[i];
    }
    sum = warp_sum(sum);
#pragma unroll
    for (int i = 0; i < kMaxPerLane; ++i) s[i] /= sum;
  } else {
#pragma unroll
    for (int i = 0; i < kMaxPerLane; ++i) s[i] = lane + i * 32 < E ? 1.f / (1.f + expf(-s[i])) : 0.f;
  }
#pragma unroll
  for (int i = 0; i < kMaxPerLane; ++i) {
    const int e = lane + i * 32;
    c[i] = e < E ? s[i] + (correction != nullptr ? correction[e] : 0.f) : -INFINITY;
    ok[i] = false;
    if (e < E) cs[e] = c[i];
  }
  __syncwarp();
  // group scores: lane l owns groups l, l + 32, ...
  const int gsz = E / groups;
  float gs[kMaxPerLane];
#pragma unroll
  for (int j = 0; j < kMaxPerLane; ++j) {
    const int g = lane + j * 32;
    gs[j] = -INFINITY;
    if (g >= groups) continue;
    float best[kMaxGroupTop];
#pragma unroll
    for (int n = 0; n < kMaxGroupTop; ++n) best[n] = -INFINITY;
    for (int e = g * gsz; e < (g + 1) * gsz; ++e) {
      float v = cs[e];
#pragma unroll
      for (int n = 0; n < kMaxGroupTop; ++n)
        if (n < group_top && v > best[n]) { const float o = best[n]; best[n] = v; v = o; }
    }
    float sum = 0.f;
#pragma unroll
    for (int n = 0; n < kMaxGroupTop; ++n)
      if (n < group_top && n < gsz) sum += best[n];
    gs[j] = sum;
  }
  // best `keep` groups: repeatedly take the group with the largest score (ties: the lower group)
  unsigned long long taken_lo = 0ull, taken_hi = 0ull, taken_2 = 0ull, taken_3 = 0ull;   // up to 256 groups
  for (int n = 0; n < keep; ++n) {
    float bv = -INFINITY;
    int bg = 0x7fffffff;
#pragma unroll
    for (int j = 0; j < kMaxPerLane; ++j) {
      const int g = lane + j * 32;
      if (g >= groups) continue;
      const unsigned long long word = g < 64 ? taken_lo : g < 128 ? taken_hi : g < 192 ? taken_2 : taken_3;
      if ((word >> (g & 63)) & 1ull) continue;
      if (gs[j] > bv || (gs[j] == bv && g < bg) || bg == 0x7fffffff) { bv = gs[j]; bg = g; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
      const int og = __shfl_xor_sync(0xffffffffu, bg, o);
      if (og != 0x7fffffff && (bg == 0x7fffffff || ov > bv || (ov == bv && og < bg))) { bv = ov; bg = og; }
    }
    if (bg < 64) taken_lo |= 1ull << bg; else if (bg < 128) taken_hi |= 1ull << (bg - 64);
    else if (bg < 192) taken_2 |= 1ull << (bg - 128); else if (bg < 256) taken_3 |= 1ull << (bg - 192);
  }
#pragma unroll
  for (int i = 0; i < kMaxPerLane; ++i) {
    const int e = lane + i * 32;
    if (e >= E) continue;
    const int g = e / gsz;
    const unsigned long long word = g < 64 ? taken_lo : g < 128 ? taken_hi : g < 192 ? taken_2 : taken_3;
    ok[i] = (word >> (g & 63)) & 1ull;
  }
  // top experts among the eligible ones, by choice score; the weight is the plain score
  float wsum = 0.f;
  float myw = 0.f;      // lane n keeps the n-th pick (top <= 32)
  int myid = 0;
  bool mine = false;
  for (int n = 0; n < top; ++n) {
    float bv = -INFINITY, bs = 0.f;
    int be = 0x7fffffff;
#pragma unroll
    for (int i = 0; i < kMaxPerLane; ++i) {
      const int e = lane + i * 32;
      if (e < E && ok[i] && (be == 0x7fffffff || c[i] > bv || (c[i] == bv && e < be))) { bv = c[i]; be = e; bs = s[i]; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
      const float os = __shfl_xor_sync(0xffffffffu, bs, o);
      const int oe = __shfl_xor_sync(0xffffffffu, be, o);
      if (oe != 0x7fffffff && (be == 0x7fffffff || ov > bv || (ov == bv && oe < be))) { bv = ov; be = oe; bs = os; }
    }
    if (be < E) {
      if ((be & 31) == lane) ok[be >> 5] = false;
      wsum += bs;
      if (lane == n) { myw = bs; myid = be; mine = true; }
    } else if (lane == n) { myw = 0.f; myid = 0; }
  }
  const float inv = renorm ? route_scale / (wsum + 1e-20f) : route_scale;
  if (lane < top) {
    ids[(int64_t)t * top + lane] = myid;
    wts[(int64_t)t * top + lane] = myw * inv;
  }
  if (dense != nullptr) {   // [T, E] routing weights, 0 for experts that were not chosen
    for (int e = lane; e < E; e += 32) dense[(int64_t)t * E + e] = 0.f;
    __syncwarp();
    if (lane < top && mine) dense[(int64_t)t * E + myid] = myw * inv;
  }
}

// grid (T, top, ceil(F / 8)); 8 warps, one output feature each
template <typename T>
__global__ void __launch_bounds__(256) moe_up_kernel(const T* __restrict__ h, int64_t ldh, const int* __restrict__ ids,
                                                     const T* __restrict__ w_up, T* __restrict__ act_out, int W, int F,
                                                     int top, int act, int gated) {
  extern __shared__ float hs[];
  const int64_t t = blockIdx.x;
  const int k = blockIdx.y;
  for (int c = threadIdx.x; c < W; c += 256) hs[c] = to_f32(h[t * ldh + c]);
  __syncthreads();
  const int f = blockIdx.z * 8 + (threadIdx.x >> 5);
  if (f >= F) return;
  const int lane = threadIdx.x & 31;
  const int e = ids[t * top + k];
  if (gated) {   // rows interleave (gate_f, up_f): hidden = act(gate) * up
    const T* wg = w_up + ((int64_t)e * 2 * F + 2 * f) * W;
    const T* wu = wg + W;
    float g = 0.f, u = 0.f;
    for (int c = lane; c < W; c += 32) { g = fmaf(to_f32(wg[c]), hs[c], g); u = fmaf(to_f32(wu[c]), hs[c], u); }
    g = warp_sum(g); u = warp_sum(u);
    if (lane == 0) act_out[(t * top + k) * F + f] = from_f32<T>(act_exact(g, act) * u);
    return;
  }
  const T* wr = w_up + ((int64_t)e * F + f) * W;
  float s = 0.f;
  for (int c = lane; c < W; c += 32) s = fmaf(to_f32(wr[c]), hs[c], s);
  s = warp_sum(s);
  if (lane == 0) act_out[(t * top + k) * F + f] = from_f32<T>(act_apply(s, act));
}

// grid (T, ceil(W / 8)); 8 warps, one output feature each, summed over the chosen experts in 32-bit
template <typename T>
__global__ void __launch_bounds__(256) moe_down_kernel(const T* __restrict__ act_in, const int* __restrict__ ids,
                                                       const float* __restrict__ wts, const T* __restrict__ w_down, int64_t ldd,
                                                       float* __restrict__ out, int64_t ldo, int W, int F, int top) {
  extern __shared__ float as[];   // [top][F]
  const int64_t t = blockIdx.x;
  for (int c = threadIdx.x; c < top * F; c += 256) as[c] = to_f32(act_in[t * top * F + c]);
  __syncthreads();
  const int n = blockIdx.y * 8 + (threadIdx.x >> 5);
  if (n >= W) return;
  const int lane = threadIdx.x & 31;
  float y = 0.f;
  for (int k = 0; k < top; ++k) {
    const int e = ids[t * top + k];
    const T* wr = w_down + (int64_t)n * ldd + (int64_t)e * F;   // row n of expert e inside [W, E * F]
    float s = 0.f;
    for (int c = lane; c < F; c += 32) s = fmaf(to_f32(wr[c]), as[k * F + c], s);
    y += wts[t * top + k] * warp_sum(s);
  }
  if (lane == 0) out[t * ldo + n] = y;
}

// a[t, e * F + f] *= dense[t, e]   (dense form: weight each expert's block before the shared down projection)
template <typename T>
__global__ void __launch_bounds__(256) moe_scale_kernel(T* __restrict__ a, int64_t lda, const float* __restrict__ dense, int E,
                                                        int F) {
  const int64_t t = blockIdx.x;
  for (int c = threadIdx.x; c < E * F; c += 256) {
    const float w = dense[t * E + c / F];
    a[t * lda + c] = from_f32<T>(to_f32(a[t * lda + c]) * w);
  }
}


// ---- grouped form for long prompts: (token, chosen expert) pairs sorted by expert, so that every expert multiplies one
// contiguous block of rows.  count -> (host: offsets) -> permute (ordered compaction, one CTA per expert: the order inside an
// expert's block is the pair order, so the result does not depend on scheduling) -> gather rows -> per-expert GEMMs ->
// combine (sum over a token's experts in its own order, 32-bit).
__global__ void __launch_bounds__(256) moe_count_kernel(const int* __restrict__ ids, int P, int* __restrict__ counts) {
  __shared__ int red[8];
  const int e = blockIdx.x;
  int c = 0;
  for (int p = threadIdx.x; p < P; p += 256) c += (ids[p] == e);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) c += __shfl_xor_sync(0xffffffffu, c, o);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = c;
  __syncthreads();
  if (threadIdx.x == 0) {
    int t = 0;
    for (int i = 0; i < 8; ++i) t += red[i];
    counts[e] = t;
  }
}

__global__ void __launch_bounds__(256) moe_permute_kernel(const int* __restrict__ ids, int P, const int* __restrict__ offsets,
                                                          int* __restrict__ perm, int* __restrict__ inv) {
  __shared__ int wsum[8];
  __shared__ int running;
  const int e = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (threadIdx.x == 0) running = offsets[e];
  __syncthreads();
  for (int p0 = 0; p0 < P; p0 += 256) {
    const int p = p0 + threadIdx.x;
    const bool mine = p < P && ids[p] == e;
    const unsigned m = __ballot_sync(0xffffffffu, mine);
    if (lane == 0) wsum[warp] = __popc(m);
    __syncthreads();
    int before = running;
    for (int w = 0; w < warp; ++w) before += wsum[w];
    if (mine) {
      const int pos = before + __popc(m & ((1u << lane) - 1u));
      perm[pos] = p;
      inv[p] = pos;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      int t = 0;
      for (int w = 0; w < 8; ++w) t += wsum[w];
      running += t;
    }
    __syncthreads();
  }
}

template <typename T>
__global__ void __launch_bounds__(256) moe_gather_rows_kernel(const T* __restrict__ h, int64_t ldh, const int* __restrict__ perm,
                                                              int top, T* __restrict__ xs, int W) {
  const int64_t i = blockIdx.x;
  const T* src = h + (int64_t)(perm[i] / top) * ldh;
  for (int c = threadIdx.x; c < W; c += 256) xs[i * W + c] = src[c];
}

__global__ void __launch_bounds__(256) moe_combine_kernel(const float* __restrict__ y, const int* __restrict__ inv,
                                                          const float* __restrict__ wts, float* __restrict__ out, int64_t ldo,
                                                          int W, int top) {
  const int64_t t = blockIdx.x;
  for (int c = threadIdx.x; c < W; c += 256) {
    float v = 0.f;
    for (int k = 0; k < top; ++k) v += wts[t * top + k] * y[(int64_t)inv[t * top + k] * W + c];
    out[t * ldo + c] = v;
  }
}

template <typename T>
int launch_experts(const void* h, int64_t ldh, const int* ids, const float* wts, const void* w_up, const void* w_down,
                   int64_t ldd, void* act_scratch, float* out, int64_t ldo, int T_, int W, int F, int top, int act, int gated,
                   cudaStream_t stream) {
  const size_t sm_up = (size_t)W * 4, sm_dn = (size_t)top * F * 4;
  static PerDeviceSmem g1, g2;
  LLMSS_CHECK_CUDA(g1.ensure(moe_up_kernel<T>, (int)sm_up));
  LLMSS_CHECK_CUDA(g2.ensure(moe_down_kernel<T>, (int)sm_dn));
  moe_up_kernel<T><<<dim3(T_, top, (F + 7) / 8), 256, sm_up, stream>>>((const T*)h, ldh, ids, (const T*)w_up, (T*)act_scratch, W, F, top, act, gated);
  moe_down_kernel<T><<<dim3(T_, (W + 7) / 8), 256, sm_dn, stream>>>((const T*)act_scratch, ids, wts, (const T*)w_down, ldd, out, ldo, W, F, top);
  LLMSS_CHECK_CUDA(cudaGetLastError());
  return 0;
}

}  // namespace

LLMSS_API int llmss_moe_route_ex(const float* z, int64_t ldz, int T_, int E, int top, int groups, int keep, float route_scale,
                                 int score_kind, const float* correction, int group_top, int renorm, int* ids, float* wts,
                                 float* dense, cudaStream_t stream) {
  LLMSS_REQUIRE(E > 0 && E <= 32 * kMaxPerLane, "moe_route: %d experts (at most %d)", E, 32 * kMaxPerLane);
  LLMSS_REQUIRE(top > 0 && top <= 32 && top <= E, "moe_route: top=%d must be in 1..min(32, experts)", top);
  LLMSS_REQUIRE(groups > 0 && E % groups == 0 && keep > 0 && keep <= groups, "moe_route: bad groups %d / keep %d for %d experts",
                groups, keep, E);
  LLMSS_REQUIRE(score_kind == 0 || score_kind == 1, "moe_route: score kind %d (0 softmax, 1 sigmoid)", score_kind);
  LLMSS_REQUIRE(group_top >= 1 && group_top <= kMaxGroupTop, "moe_route: a group sums its %d best (1..%d)", group_top, kMaxGroupTop);
  if (T_ == 0) return 0;
  moe_route_kernel<<<(T_ + 3) / 4, 128, 0, stream>>>(z, ldz, E, top, groups, keep, route_scale, score_kind, correction, group_top,
                                                     renorm, ids, wts, dense, T_);
  LLMSS_CHECK_CUDA(cudaGetLastError());
  return 0;
}

LLMSS_API int llmss_moe_route(const float* z, int64_t ldz, int T_, int E, int top, int groups, int keep, float route_scale,
                              int* ids, float* wts, float* dense, cudaStream_t stream) {
  return llmss_moe_route_ex(z, ldz, T_, E, top, groups, keep, route_scale, 0, nullptr, 1, 1, ids, wts, dense, stream);
}

LLMSS_API int llmss_moe_experts(const void* h, int64_t ldh, const int* ids, const float* wts, const void* w_up,
                                const void* w_down, int64_t ldd, void* act_scratch, float* out, int64_t ldo, int T_, int W, int F, int top,
                                int act, int gated, int dtype, cudaStream_t stream) {
  LLMSS_REQUIRE(T_ <= 0x7fffffff / 1 && top <= 65535 && (F + 7) / 8 <= 65535 && (W + 7) / 8 <= 65535, "moe_experts: grid too large");
  LLMSS_REQUIRE((size_t)W * 4 <= 200 * 1024 && (size_t)top * F * 4 <= 200 * 1024, "moe_experts: width %d / top * ff %d exceed shared memory", W, top * F);
  if (T_ == 0) return 0;
  LLMSS_BY_DTYPE(dtype, return (launch_experts<T>(h, ldh, ids, wts, w_up, w_down, ldd, act_scratch, out, ldo, T_, W, F, top, act, gated, stream)));
}

LLMSS_API int llmss_moe_scale(void* a, int64_t lda, const float* dense, int T_, int E, int F, int dtype, cudaStream_t stream) {
  if (T_ == 0) return 0;
  LLMSS_BY_DTYPE(dtype, (moe_scale_kernel<T><<<T_, 256, 0, stream>>>((T*)a, lda, dense, E, F)));
  LLMSS_CHECK_CUDA(cudaGetLastError());
  return 0;
}

LLMSS_API int llmss_moe_count(const int* ids, int P, int E, int* counts, cudaStream_t stream) {
  if (E <= 0) return 0;
  moe_count_kernel<<<E, 256, 0, stream>>>(ids, P, counts);
  LLMSS_CHECK_CUDA(cudaGetLastError());
  return 0;
}

// offsets[e] = first row of expert e's block; perm[row] = pair index (token * top + k); inv[pair] = row
LLMSS_API int llmss_moe_permute(const int* ids, int P, int E, const int* offsets, int* perm, int* inv, cudaStream_t stream) {
  if (E <= 0 || P <= 0) return 0;
  moe_permute_kernel<<<E, 256, 0, stream>>>(ids, P, offsets, perm, inv);
  LLMSS_CHECK_CUDA(cudaGetLastError());
  return 0;
}

LLMSS_API int llmss_moe_gather_rows(const void* h, int64_t ldh, const int* perm, int top, void* xs, int P, int W, int dtype,
                                    cudaStream_t stream) {
  if (P <= 0) return 0;
  LLMSS_BY_DTYPE(dtype, (moe_gather_rows_kernel<T><<<P, 256, 0, stream>>>((const T*)h, ldh, perm, top, (T*)xs, W)));
  LLMSS_CHECK_CUDA(cudaGetLastError());
  return 0;
}

LLMSS_API int llmss_moe_combine(const float* y, const int* inv, const float* wts, float* out, int64_t ldo, int T_, int W, int top,
                                cudaStream_t stream) {
  if (T_ <= 0) return 0;
  moe_combine_kernel<<<T_, 256, 0, stream>>>(y, inv, wts, out, ldo, W, top);
  LLMSS_CHECK_CUDA(cudaGetLastError());
  return 0;
}

// Gated delta rule over a packed batch (same batch convention as recurrent.cu: cu_q / seq_lens / state slots).
//
//   per head and token:  S <- g_t S ;  u = beta_t (v_t - S^T k_t) ;  S <- S + k_t u^T ;  o_t = S^T q_t
//
// Every value column of the state is a recurrence of its own (S^T k, the write and the read-out only couple the rows of one
// column), so thread (j, r) keeps rows [r * KPT, r * KPT + KPT) of column j in registers and the R threads of a column meet
// in two warp-shuffle sums per token.  One block = one (sequence, head, slice of value columns); the block that reads a
// slot's old state is the block that writes its new one.  Tokens are staged 16 at a time through shared memory: q and k in
// strips of KPT + 4 floats (the strips a warp reads together lie in different banks, every read a 16-byte one; strips beyond
// dk hold zeros), copied asynchronously one stage ahead, made unit vectors there (x / sqrt(sum x^2 + eps), q times its scale), decays exp(log g) and write
// strengths (sigmoid taken here if asked) beside them.  The state lies in memory column-major per head ([dv][dk]).
// KPT is the key size itself up to 64 (R = 1): the lanes of a warp then differ only in their value column, every staged q / k
// read is one address for the whole warp (a shared-memory broadcast), and no shuffle is needed; larger keys split over R lanes.
//
// A batch of single tokens (decode) runs the row-split form instead (delta_step_kernel): one warp per value column, lanes over
// the key rows, so that every state access is one contiguous column (512 bytes at dk = 128) -- a decode step is bound by
// reading and writing the states once.
// Everything is 32-bit with full-precision exponentials.
#include "common.cuh"

namespace {

constexpr int DTCH = 16;

struct DeltaArgs {
  const float* q; int64_t ldq;
  const float* k; int64_t ldk;
  const float* v; int64_t ldv;
  const float* log_decay; int64_t ldg;   // [T, H]
  const float* beta; int64_t ldb;        // [T, H]
  float* out;                            // [T, H * dv]
  float* state;                          // [slots, H, dv, dk]
  const int* cu_q; const int* seq_lens; const int* slots;
  int H, rep, dk, dv, dvt, R;
  float unit_eps, q_scale;
  int unit, beta_sigmoid;
  int vec16;       // q / k / v rows, the key size and the value slices allow 16-byte copies
};

__device__ __forceinline__ void cp_async_4(float* dst, const float* src) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(smem_u32(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_16(float* dst, const float* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

// Stages of 16 tokens are double-buffered: the asynchronous copies of stage s + 1 (global -> shared, no registers) run behind the
// arithmetic of stage s, so the dependent chain of a long portion never waits for memory.
template <int KPT>
__global__ void __launch_bounds__(256) delta_scan_kernel(DeltaArgs a) {
  constexpr int STRIP = KPT + 4;
  extern __shared__ __align__(16) float sm[];
  const int b = blockIdx.x;
  const int q0 = a.cu_q[b], ql = a.cu_q[b + 1] - q0, ctx = a.seq_lens[b] - ql, slot = a.slots[b];
  if (slot < 0 || ctx < 0 || ql <= 0) return;
  const int h = blockIdx.y, hk = h / a.rep;
  const int j0 = blockIdx.z * a.dvt, nj = min(a.dvt, a.dv - j0);
  const int dk = a.dk, R = a.R, row = R * STRIP, nthr = blockDim.x;
  const int jl = threadIdx.x / R, r = threadIdx.x % R;
  const bool live = jl < nj;
  const int j = j0 + jl, i0 = r * KPT;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = nthr >> 5;
  const int stage_floats = 2 * DTCH * row + DTCH * a.dvt + 2 * DTCH;     // q, k [DTCH][row]; v [DTCH][dvt]; decays, strengths [DTCH]
  float S[KPT];
  float* sp = a.state + (((int64_t)slot * a.H + h) * a.dv + (live ? j : 0)) * dk;
  const bool vec = (dk & 3) == 0;        // every column of the state starts on a 16-byte boundary
#pragma unroll
  for (int ii = 0; ii < KPT; ii += 4) {
    float4 t4 = make_float4(0.f, 0.f, 0.f, 0.f);
    if (live && ctx > 0) {
      if (vec && i0 + ii + 4 <= dk) t4 = *reinterpret_cast<const float4*>(sp + i0 + ii);
      else {
        if (i0 + ii < dk) t4.x = sp[i0 + ii];
        if (i0 + ii + 1 < dk) t4.y = sp[i0 + ii + 1];
        if (i0 + ii + 2 < dk) t4.z = sp[i0 + ii + 2];
        if (i0 + ii + 3 < dk) t4.w = sp[i0 + ii + 3];
      }
    }
    S[ii] = t4.x; S[ii + 1] = t4.y; S[ii + 2] = t4.z; S[ii + 3] = t4.w;
  }
  // the strips' padding (beyond dk, and between strips) is read by the arithmetic and never copied into: zero it once
  for (int idx = threadIdx.x; idx < 2 * stage_floats; idx += nthr) sm[idx] = 0.f;
  __syncthreads();
  auto issue = [&](int t0, float* B) {
    const int nt = min(DTCH, ql - t0);
    float* qs = B;
    float* ks = B + DTCH * row;
    float* vs = ks + DTCH * row;
    float* gs = vs + DTCH * a.dvt;
    if (a.vec16) {
      const int n4 = dk >> 2;
      for (int idx = threadIdx.x; idx < nt * n4; idx += nthr) {
        const int tt = idx / n4, c = (idx - tt * n4) << 2;
        const int dst = tt * row + (c / KPT) * STRIP + c % KPT;
        const int64_t t = q0 + t0 + tt;
        cp_async_16(qs + dst, a.q + t * a.ldq + (int64_t)hk * dk + c);
        cp_async_16(ks + dst, a.k + t * a.ldk + (int64_t)hk * dk + c);
      }
      const int v4 = nj >> 2;       // vec16: dv and the slice width are multiples of 4
      for (int idx = threadIdx.x; idx < nt * v4; idx += nthr) {
        const int tt = idx / v4, c = (idx - tt * v4) << 2;
        cp_async_16(vs + tt * a.dvt + c, a.v + (int64_t)(q0 + t0 + tt) * a.ldv + (int64_t)h * a.dv + j0 + c);
      }
    } else {
      for (int idx = threadIdx.x; idx < nt * dk; idx += nthr) {
        const int tt = idx / dk, c = idx - tt * dk;
        const int dst = tt * row + (c / KPT) * STRIP + c % KPT;
        const int64_t t = q0 + t0 + tt;
        cp_async_4(qs + dst, a.q + t * a.ldq + (int64_t)hk * dk + c);
        cp_async_4(ks + dst, a.k + t * a.ldk + (int64_t)hk * dk + c);
      }
      for (int idx = threadIdx.x; idx < nt * nj; idx += nthr) {
        const int tt = idx / nj, c = idx - tt * nj;
        cp_async_4(vs + tt * a.dvt + c, a.v + (int64_t)(q0 + t0 + tt) * a.ldv + (int64_t)h * a.dv + j0 + c);
      }
    }
    if (threadIdx.x < nt) {
      const int64_t t = q0 + t0 + threadIdx.x;
      cp_async_4(gs + threadIdx.x, a.log_decay + t * a.ldg + h);
      cp_async_4(gs + DTCH + threadIdx.x, a.beta + t * a.ldb + h);
    }
    cp_async_commit();
  };
  issue(0, sm);
  int cur = 0;
  for (int t0 = 0; t0 < ql; t0 += DTCH, cur ^= 1) {
    const int nt = min(DTCH, ql - t0);
    float* qs = sm + cur * stage_floats;
    float* ks = qs + DTCH * row;
    float* vs = ks + DTCH * row;
    float* gs = vs + DTCH * a.dvt;
    float* bs = gs + DTCH;
    if (t0 + DTCH < ql) {
      issue(t0 + DTCH, sm + (cur ^ 1) * stage_floats);
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();
    if (threadIdx.x < nt) {
      gs[threadIdx.x] = expf(gs[threadIdx.x]);
      if (a.beta_sigmoid) bs[threadIdx.x] = 1.f / (1.f + expf(-bs[threadIdx.x]));
    }
    if (a.unit || a.q_scale != 1.f) {
      for (int tt = warp; tt < nt; tt += nwarp) {
        float sq = 0.f, sk = 0.f;
        for (int w = lane; w < row; w += 32) {
          sq = fmaf(qs[tt * row + w], qs[tt * row + w], sq);
          sk = fmaf(ks[tt * row + w], ks[tt * row + w], sk);
        }
        sq = warp_sum(sq);
        sk = warp_sum(sk);
        const float rq = (a.unit ? rsqrtf(sq + a.unit_eps) : 1.f) * a.q_scale, rk = a.unit ? rsqrtf(sk + a.unit_eps) : 1.f;
        for (int w = lane; w < row; w += 32) {
          qs[tt * row + w] *= rq;
          ks[tt * row + w] *= rk;
        }
      }
    }
    __syncthreads();
    for (int tt = 0; tt < nt; ++tt) {
      const float g = gs[tt], be = bs[tt];
      const float* kr = ks + tt * row + r * STRIP;
      const float* qr = qs + tt * row + r * STRIP;
      float d0 = 0.f, d1 = 0.f, d2 = 0.f, d3 = 0.f;
#pragma unroll
      for (int ii = 0; ii < KPT; ii += 4) {
        const float4 k4 = *reinterpret_cast<const float4*>(kr + ii);
        d0 = fmaf(S[ii], k4.x, d0); d1 = fmaf(S[ii + 1], k4.y, d1); d2 = fmaf(S[ii + 2], k4.z, d2); d3 = fmaf(S[ii + 3], k4.w, d3);
      }
      float d = (d0 + d1) + (d2 + d3);
      for (int o = R >> 1; o > 0; o >>= 1) d += __shfl_xor_sync(0xffffffffu, d, o);
      const float u = be * (vs[tt * a.dvt + jl] - g * d);
      float e0 = 0.f, e1 = 0.f, e2 = 0.f, e3 = 0.f;
#pragma unroll
      for (int ii = 0; ii < KPT; ii += 4) {
        const float4 k4 = *reinterpret_cast<const float4*>(kr + ii);
        const float4 q4 = *reinterpret_cast<const float4*>(qr + ii);
        S[ii] = fmaf(g, S[ii], k4.x * u); S[ii + 1] = fmaf(g, S[ii + 1], k4.y * u);
        S[ii + 2] = fmaf(g, S[ii + 2], k4.z * u); S[ii + 3] = fmaf(g, S[ii + 3], k4.w * u);
        e0 = fmaf(S[ii], q4.x, e0); e1 = fmaf(S[ii + 1], q4.y, e1); e2 = fmaf(S[ii + 2], q4.z, e2); e3 = fmaf(S[ii + 3], q4.w, e3);
      }
      float o = (e0 + e1) + (e2 + e3);
      for (int s = R >> 1; s > 0; s >>= 1) o += __shfl_xor_sync(0xffffffffu, o, s);
      if (live && r == 0) a.out[(int64_t)(q0 + t0 + tt) * a.H * a.dv + (int64_t)h * a.dv + j] = o;
    }
    __syncthreads();      // this buffer is copied into again at the start of the next round
  }
  if (live) {
#pragma unroll
    for (int ii = 0; ii < KPT; ii += 4) {
      if (vec && i0 + ii + 4 <= dk) *reinterpret_cast<float4*>(sp + i0 + ii) = make_float4(S[ii], S[ii + 1], S[ii + 2], S[ii + 3]);
      else {
        if (i0 + ii < dk) sp[i0 + ii] = S[ii];
        if (i0 + ii + 1 < dk) sp[i0 + ii + 1] = S[ii + 1];
        if (i0 + ii + 2 < dk) sp[i0 + ii + 2] = S[ii + 2];
        if (i0 + ii + 3 < dk) sp[i0 + ii + 3] = S[ii + 3];
      }
    }
  }
}

// Single tokens: grid (B, H, column groups), 8 warps per block; warp w takes columns j0 + w, j0 + w + 8, ... four at a time.
// Lane l holds rows l, l + 32, ... (KL of them) of q, k and of the column in flight.
constexpr int STEP_WARPS = 8, STEP_COLS = 4;
template <int KL>
__global__ void __launch_bounds__(STEP_WARPS * 32) delta_step_kernel(DeltaArgs a, int cols_per_block) {
  const int b = blockIdx.x;
  const int q0 = a.cu_q[b], ql = a.cu_q[b + 1] - q0, ctx = a.seq_lens[b] - ql, slot = a.slots[b];
  if (slot < 0 || ctx < 0 || ql != 1) return;
  const int h = blockIdx.y, hk = h / a.rep, dk = a.dk, dv = a.dv;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int64_t t = q0;
  float qv[KL], kv[KL];
  float sq = 0.f, sk = 0.f;
#pragma unroll
  for (int m = 0; m < KL; ++m) {
    const int i = lane + 32 * m;
    qv[m] = i < dk ? a.q[t * a.ldq + (int64_t)hk * dk + i] : 0.f;
    kv[m] = i < dk ? a.k[t * a.ldk + (int64_t)hk * dk + i] : 0.f;
    sq = fmaf(qv[m], qv[m], sq);
    sk = fmaf(kv[m], kv[m], sk);
  }
  if (a.unit || a.q_scale != 1.f) {
    sq = warp_sum(sq);
    sk = warp_sum(sk);
    const float rq = (a.unit ? rsqrtf(sq + a.unit_eps) : 1.f) * a.q_scale, rk = a.unit ? rsqrtf(sk + a.unit_eps) : 1.f;
#pragma unroll
    for (int m = 0; m < KL; ++m) { qv[m] *= rq; kv[m] *= rk; }
  }
  const float g = expf(a.log_decay[t * a.ldg + h]);
  const float braw = a.beta[t * a.ldb + h];
  const float be = a.beta_sigmoid ? 1.f / (1.f + expf(-braw)) : braw;
  float* sp = a.state + ((int64_t)slot * a.H + h) * dv * dk;
  const float* vp = a.v + t * a.ldv + (int64_t)h * dv;
  float* op = a.out + t * a.H * dv + (int64_t)h * dv;
  const int j0 = blockIdx.z * cols_per_block, j1 = min(dv, j0 + cols_per_block);
  for (int jb = j0 + warp; jb < j1; jb += STEP_WARPS * STEP_COLS) {
    float S[STEP_COLS][KL], d[STEP_COLS], e[STEP_COLS];
#pragma unroll
    for (int c = 0; c < STEP_COLS; ++c) {
      const int j = jb + c * STEP_WARPS;
      d[c] = 0.f;
#pragma unroll
      for (int m = 0; m < KL; ++m) {
        const int i = lane + 32 * m;
        S[c][m] = (j < j1 && ctx > 0 && i < dk) ? sp[(int64_t)j * dk + i] : 0.f;
        d[c] = fmaf(S[c][m], kv[m], d[c]);
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1)
#pragma unroll
      for (int c = 0; c < STEP_COLS; ++c) d[c] += __shfl_xor_sync(0xffffffffu, d[c], o);
#pragma unroll
    for (int c = 0; c < STEP_COLS; ++c) {
      const int j = jb + c * STEP_WARPS;
      const float u = be * ((j < j1 ? vp[j] : 0.f) - g * d[c]);
      e[c] = 0.f;
#pragma unroll
      for (int m = 0; m < KL; ++m) {
        S[c][m] = fmaf(g, S[c][m], kv[m] * u);
        e[c] = fmaf(S[c][m], qv[m], e[c]);
        const int i = lane + 32 * m;
        if (j < j1 && i < dk) sp[(int64_t)j * dk + i] = S[c][m];
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1)
#pragma unroll
      for (int c = 0; c < STEP_COLS; ++c) e[c] += __shfl_xor_sync(0xffffffffu, e[c], o);
#pragma unroll
    for (int c = 0; c < STEP_COLS; ++c) {
      const int j = jb + c * STEP_WARPS;
      if (lane == 0 && j < j1) op[j] = e[c];
    }
  }
}

}  // namespace

// q, k [T, qk_heads * dk] (value head h reads q / k head h / (heads / qk_heads)); v [T, heads * dv]; log_decay, beta [T, heads];
// out [T, heads * dv]; state [slots, heads, dv, dk].  unit_eps >= 0: q and k become x / sqrt(sum x^2 + unit_eps) per head first.
LLMSS_API int llmss_delta_scan(const float* q, int64_t ldq, const float* k, int64_t ldk, const float* v, int64_t ldv,
                               const float* log_decay, int64_t ldg, const float* beta, int64_t ldb, float* out, float* state,
                               const int* cu_q, const int* seq_lens, const int* slots, int B, int max_q, int heads, int qk_heads, int dk,
                               int dv, float unit_eps, float q_scale, int beta_sigmoid, cudaStream_t stream) {
  LLMSS_REQUIRE(heads > 0 && qk_heads > 0 && heads % qk_heads == 0, "delta_scan: %d value heads over %d query/key heads", heads, qk_heads);
  LLMSS_REQUIRE(dk > 0 && dk <= 1024 && dv > 0, "delta_scan: key size %d (at most 1024), value size %d", dk, dv);
  if (B <= 0) return 0;
  DeltaArgs a;
  a.q = q; a.ldq = ldq; a.k = k; a.ldk = ldk; a.v = v; a.ldv = ldv; a.log_decay = log_decay; a.ldg = ldg; a.beta = beta; a.ldb = ldb;
  a.out = out; a.state = state; a.cu_q = cu_q; a.seq_lens = seq_lens; a.slots = slots;
  a.H = heads; a.rep = heads / qk_heads; a.dk = dk; a.dv = dv;
  a.unit = unit_eps >= 0.f ? 1 : 0; a.unit_eps = unit_eps >= 0.f ? unit_eps : 0.f; a.q_scale = q_scale; a.beta_sigmoid = beta_sigmoid;
  if (max_q <= 1 && dk <= 256) {
    // every sequence brings one token: one warp per value column, lanes over the key rows
    a.R = 1; a.dvt = 0;
    const int per_pass = STEP_WARPS * STEP_COLS;
    int groups = 1;
    while ((int64_t)B * heads * groups < 1024 && groups * per_pass < dv) groups *= 2;
    int cols = (dv + groups - 1) / groups;
    cols = ((cols + per_pass - 1) / per_pass) * per_pass;
    const dim3 sgrid(B, heads, (dv + cols - 1) / cols);
    LLMSS_REQUIRE(sgrid.y <= 65535 && sgrid.z <= 65535, "delta_scan: grid too large");
    const int kl = (dk + 31) / 32;
    if (kl <= 1) delta_step_kernel<1><<<sgrid, STEP_WARPS * 32, 0, stream>>>(a, cols);
    else if (kl <= 2) delta_step_kernel<2><<<sgrid, STEP_WARPS * 32, 0, stream>>>(a, cols);
    else if (kl <= 4) delta_step_kernel<4><<<sgrid, STEP_WARPS * 32, 0, stream>>>(a, cols);
    else delta_step_kernel<8><<<sgrid, STEP_WARPS * 32, 0, stream>>>(a, cols);
    LLMSS_CHECK_CUDA(cudaGetLastError());
    return 0;
  }
  // key rows per thread: the key size itself up to 64 (a column per thread), 64 beyond (R lanes per column)
  static const int kpt_max = [] { const char* e = getenv("LLMSS_DELTA_KPT"); const int v = e ? atoi(e) : 64; return v == 32 || v == 128 ? v : 64; }();
  int kpt = dk <= 8 ? 8 : (dk <= 16 ? 16 : (dk <= 32 ? 32 : (dk <= 64 ? 64 : 128)));
  if (kpt > kpt_max) kpt = kpt_max;
  int R = 1;
  while (R * kpt < dk) R *= 2;
  a.R = R;
  int threads = ((dv * R + 31) / 32) * 32;
  threads = threads > 256 ? 256 : threads;
  a.dvt = threads / R;
  const dim3 grid(B, heads, (dv + a.dvt - 1) / a.dvt);
  LLMSS_REQUIRE(grid.y <= 65535 && grid.z <= 65535, "delta_scan: grid too large");
  a.vec16 = (dk % 4 == 0 && dv % 4 == 0 && a.dvt % 4 == 0 && ldq % 4 == 0 && ldk % 4 == 0 && ldv % 4 == 0 &&
             (((uintptr_t)q | (uintptr_t)k | (uintptr_t)v) & 15) == 0) ? 1 : 0;
  const size_t smem = 2 * sizeof(float) * ((size_t)2 * DTCH * R * (kpt + 4) + (size_t)DTCH * a.dvt + 2 * DTCH);
#define LLMSS_DS(K)                                                                     \
  do {                                                                                  \
    static PerDeviceSmem gsm;                                                           \
    if (smem > 48 * 1024) LLMSS_CHECK_CUDA(gsm.ensure(delta_scan_kernel<K>, (int)smem)); \
    delta_scan_kernel<K><<<grid, threads, smem, stream>>>(a);                           \
  } while (0)
  if (kpt == 8) LLMSS_DS(8);
  else if (kpt == 16) LLMSS_DS(16);
  else if (kpt == 32) LLMSS_DS(32);
  else if (kpt == 64) LLMSS_DS(64);
  else LLMSS_DS(128);
#undef LLMSS_DS
  LLMSS_CHECK_CUDA(cudaGetLastError());
  return 0;
}

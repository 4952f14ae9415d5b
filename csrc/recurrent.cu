// Kernels of recurrent token mixers over a packed batch, and of the post-normed 32-bit residual stream.
//
// Batch convention (all kernels): sequence b owns rows cu_q[b] .. cu_q[b+1] of the packed batch, holds seq_lens[b] tokens
// including them, and keeps what it carries from step to step in row state_slots[b] of each state tensor.  A sequence
// whose first row is its position 0 starts from zeros whatever the slot holds (slots change hands uncleared); a slot < 0
// is an inert row of a padded batch and is skipped.  State rows are read and written by ONE block per (sequence, slice):
// the block that reads a slot's old state is the block that writes its new one, so a step needs no ordering between
// blocks even when a portion is many rows long.
//
//   embed_bigram      x = wte[tok] + table[(prev * mul_prev + tok * mul_cur) mod buckets]   (row `buckets` for a first token)
//   postnorm_residual r' = r + rms_div(y) * (1 + w)     (optionally y = mean of two normed branches)  -> (cast(r'), r')
//   token_shift       mix_s = x + (x_prev - x) * mu_s   for S mixing vectors at once
//   causal_conv       y_t = act(sum_j w[:, j] u_(t - taps + 1 + j) + b)  per channel, tails kept per sequence
//   unary / ssm_dt    tanh, -exp;  dt = softplus(raw + bias), log decay = -exp(A_log) dt
//   linear_scan       S_t = diag(a_t) S_(t-1) + k_t (c_t v_t)^T ;  o_t = S_t^T q_t   or   (S_(t-1) + diag(u) k_t v_t^T)^T q_t
//   gated_rmsnorm     y = o (+ D x); gate before or after; rms_div in equal groups; times weight
//
// Everything here computes in 32-bit: states, decays, exponentials, norms and the residual sum.
#include "common.cuh"

namespace {

__device__ __forceinline__ float block_sum(float v, float* red) {   // red: >= 32 floats of shared memory
  v = warp_sum(v);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
  __syncthreads();
  if (lane == 0) red[warp] = v;
  __syncthreads();
  float t = 0.f;
  for (int i = 0; i < nw; ++i) t += red[i];
  return t;
}

struct Seq {
  int q0, ql, ctx, slot;
};
__device__ __forceinline__ Seq seq_of(const int* cu_q, const int* seq_lens, const int* slots, int b) {
  Seq s;
  s.q0 = cu_q[b];
  s.ql = cu_q[b + 1] - s.q0;
  s.ctx = seq_lens[b] - s.ql;
  s.slot = slots[b];
  if (s.slot < 0 || s.ctx < 0) s.ql = 0;
  return s;
}

// ------------------------------------------------------------------------------------------------ embed_bigram
// grid (B, row lanes); block (b, 0) owns row 0 of the sequence and with it the slot's previous-token entry
template <typename T>
__global__ void __launch_bounds__(128) embed_bigram_kernel(const int* __restrict__ tokens, const T* __restrict__ wte,
                                                           const T* __restrict__ table, float* __restrict__ out, int W, int vocab,
                                                           long long mul_prev, long long mul_cur, int buckets,
                                                           const int* __restrict__ cu_q, const int* __restrict__ seq_lens,
                                                           const int* __restrict__ slots, int* __restrict__ prev_state) {
  const Seq s = seq_of(cu_q, seq_lens, slots, blockIdx.x);
  for (int j = blockIdx.y; j < s.ql; j += gridDim.y) {
    const int t = s.q0 + j;
    const int tok = min(max(tokens[t], 0), vocab - 1);
    int row;
    if (j == 0 && s.ctx == 0) row = buckets;
    else {
      const long long prev = j > 0 ? tokens[t - 1] : prev_state[s.slot];
      row = (int)((prev * mul_prev + (long long)tok * mul_cur) % buckets);
      if (row < 0) row += buckets;
    }
    const T* a = wte + (int64_t)tok * W;
    const T* b = table + (int64_t)row * W;
    for (int c = threadIdx.x; c < W; c += blockDim.x) out[(int64_t)t * W + c] = to_f32(a[c]) + to_f32(b[c]);
  }
  if (blockIdx.y == 0 && s.ql > 0) {
    __syncthreads();   // row 0 has read the old entry
    if (threadIdx.x == 0) prev_state[s.slot] = tokens[s.q0 + s.ql - 1];
  }
}

// ------------------------------------------------------------------------------------------------ postnorm_residual
template <typename T>
__global__ void __launch_bounds__(256) postnorm_kernel(const float* __restrict__ y, int64_t ldy, const float* __restrict__ y2,
                                                       int64_t ldy2, const float* __restrict__ w_a, const float* __restrict__ w_b,
                                                       const float* __restrict__ weight, const float* __restrict__ resid,
                                                       int64_t ldr, float* __restrict__ new_resid, T* __restrict__ out, int W,
                                                       float eps, int one_plus) {
  __shared__ float red[32];
  const int64_t t = blockIdx.x;
  const float* yr = y + t * ldy;
  const float* y2r = y2 != nullptr ? y2 + t * ldy2 : nullptr;
  float ra = 0.f, rb = 0.f;
  if (y2r != nullptr) {
    float sa = 0.f, sb = 0.f;
    for (int c = threadIdx.x; c < W; c += blockDim.x) { sa = fmaf(yr[c], yr[c], sa); sb = fmaf(y2r[c], y2r[c], sb); }
    ra = rsqrtf(block_sum(sa, red) / W + eps);
    rb = rsqrtf(block_sum(sb, red) / W + eps);
  }
  float ss = 0.f;
  for (int c = threadIdx.x; c < W; c += blockDim.x) {
    const float v = y2r != nullptr ? 0.5f * (yr[c] * ra * w_a[c] + y2r[c] * rb * w_b[c]) : yr[c];
    ss = fmaf(v, v, ss);
  }
  const float r = rsqrtf(block_sum(ss, red) / W + eps);
  for (int c = threadIdx.x; c < W; c += blockDim.x) {
    const float v = y2r != nullptr ? 0.5f * (yr[c] * ra * w_a[c] + y2r[c] * rb * w_b[c]) : yr[c];
    float n = v * r * (one_plus ? 1.f + weight[c] : weight[c]);
    if (resid != nullptr) {
      n += resid[t * ldr + c];
      new_resid[t * W + c] = n;
    }
    out[t * W + c] = from_f32<T>(n);
  }
}

// ------------------------------------------------------------------------------------------------ token_shift
// VEC = 4: four columns per thread, 16-byte loads and 8- / 16-byte stores (W, ldx multiples of 4, 16-byte aligned bases)
template <typename T, int VEC>
__global__ void __launch_bounds__(128) token_shift_kernel(const float* __restrict__ x, int64_t ldx, const float* __restrict__ mu,
                                                          int S, T* __restrict__ out, int64_t Ttot, int W,
                                                          const int* __restrict__ cu_q, const int* __restrict__ seq_lens,
                                                          const int* __restrict__ slots, float* __restrict__ prev_state) {
  const Seq s = seq_of(cu_q, seq_lens, slots, blockIdx.x);
  for (int j = blockIdx.y; j < s.ql; j += gridDim.y) {
    const int64_t t = s.q0 + j;
    for (int c = (blockIdx.z * blockDim.x + threadIdx.x) * VEC; c < W; c += gridDim.z * blockDim.x * VEC) {
      float cur[VEC], d[VEC];
      if constexpr (VEC == 4) {
        const float4 a = *reinterpret_cast<const float4*>(x + t * ldx + c);
        const float4 p = j > 0 ? *reinterpret_cast<const float4*>(x + (t - 1) * ldx + c)
                               : (s.ctx > 0 ? *reinterpret_cast<const float4*>(prev_state + (int64_t)s.slot * W + c)
                                            : make_float4(0.f, 0.f, 0.f, 0.f));
        cur[0] = a.x; cur[1 % VEC] = a.y; cur[2 % VEC] = a.z; cur[3 % VEC] = a.w;
        d[0] = p.x - a.x; d[1 % VEC] = p.y - a.y; d[2 % VEC] = p.z - a.z; d[3 % VEC] = p.w - a.w;
      } else {
        cur[0] = x[t * ldx + c];
        const float prev = j > 0 ? x[(t - 1) * ldx + c] : (s.ctx > 0 ? prev_state[(int64_t)s.slot * W + c] : 0.f);
        d[0] = prev - cur[0];
      }
      for (int k = 0; k < S; ++k) {
        T* o = out + ((int64_t)k * Ttot + t) * W + c;
        const float* m = mu + (int64_t)k * W + c;
        if constexpr (VEC == 4) {
          const float4 m4 = *reinterpret_cast<const float4*>(m);
          const float v0 = fmaf(d[0], m4.x, cur[0]), v1 = fmaf(d[1 % VEC], m4.y, cur[1 % VEC]), v2 = fmaf(d[2 % VEC], m4.z, cur[2 % VEC]),
                      v3 = fmaf(d[3 % VEC], m4.w, cur[3 % VEC]);
          if constexpr (sizeof(T) == 4) {
            *reinterpret_cast<float4*>(o) = make_float4(v0, v1, v2, v3);
          } else {
            __align__(8) T tmp[4] = {from_f32<T>(v0), from_f32<T>(v1), from_f32<T>(v2), from_f32<T>(v3)};
            *reinterpret_cast<uint2*>(o) = *reinterpret_cast<const uint2*>(tmp);
          }
        } else {
          o[0] = from_f32<T>(fmaf(d[0], m[0], cur[0]));
        }
      }
      // the thread that read columns c .. of the old row is the one that replaces them
      if (j == 0 && blockIdx.y == 0) {
        const float* last = x + (int64_t)(s.q0 + s.ql - 1) * ldx + c;
        float* st = prev_state + (int64_t)s.slot * W + c;
        if constexpr (VEC == 4) *reinterpret_cast<float4*>(st) = *reinterpret_cast<const float4*>(last);
        else st[0] = last[0];
      }
    }
  }
}

// ------------------------------------------------------------------------------------------------ causal_conv
constexpr int kConvChunk = 64, kMaxTapsAny = 16;

// grid (B, ceil(C / 128), token chunks); thread = channel; chunk 0 of a sequence reads and replaces the slot's tail.
// kMaxTaps bounds the register window (instantiated for 4, 8 and 16 taps).
template <int kMaxTaps, typename TO>
__global__ void __launch_bounds__(128) causal_conv_kernel(const float* __restrict__ u, int64_t ldu, const float* __restrict__ w,
                                                          const float* __restrict__ bias, TO* __restrict__ out, int C, int taps,
                                                          int act, const int* __restrict__ cu_q, const int* __restrict__ seq_lens,
                                                          const int* __restrict__ slots, float* __restrict__ state) {
  const Seq s = seq_of(cu_q, seq_lens, slots, blockIdx.x);
  const int c = blockIdx.y * 128 + threadIdx.x;
  if (c >= C) return;
  const int hist = taps - 1;
  float wt[kMaxTaps], win[kMaxTaps], old[kMaxTaps];
#pragma unroll
  for (int i = 0; i < kMaxTaps; ++i) { wt[i] = i < taps ? w[(int64_t)c * taps + i] : 0.f; old[i] = 0.f; }
  const float bv = bias != nullptr ? bias[c] : 0.f;
  float* st = state != nullptr && s.slot >= 0 ? state + ((int64_t)s.slot * hist) * C + c : nullptr;
  for (int z = blockIdx.z; z * kConvChunk < s.ql; z += gridDim.z) {
    const int j0 = z * kConvChunk, j1 = min(s.ql, j0 + kConvChunk);
    if (z == 0 && st != nullptr && s.ctx > 0) {
#pragma unroll
      for (int i = 0; i < kMaxTaps; ++i) if (i < hist) old[i] = st[(int64_t)i * C];
    }
    // window = inputs j0 - hist .. j0 - 1 (win[i] is input j0 - hist + i); only chunk 0 reaches before the step's first row
#pragma unroll
    for (int i = 0; i < kMaxTaps; ++i) {
      const int jj = j0 - hist + i;
      win[i] = i >= hist ? 0.f : (jj >= 0 ? u[(int64_t)(s.q0 + jj) * ldu + c] : old[i]);
    }
#pragma unroll 8
    for (int j = j0; j < j1; ++j) {
      const float cur = u[(int64_t)(s.q0 + j) * ldu + c];
      float acc = bv;
#pragma unroll
      for (int i = 0; i < kMaxTaps; ++i) if (i < taps) acc = fmaf(wt[i], i < hist ? win[i] : cur, acc);
#pragma unroll
      for (int i = 0; i < kMaxTaps - 1; ++i) win[i] = i + 1 < hist ? win[i + 1] : cur;
      out[(int64_t)(s.q0 + j) * C + c] = from_f32<TO>(act_exact(acc, act));
    }
    if (z == 0 && st != nullptr) {
      // new tail: inputs ql - hist .. ql - 1; those before this step's first row come from the old tail
#pragma unroll
      for (int i = 0; i < kMaxTaps; ++i) {
        if (i >= hist) continue;
        const int jj = s.ql - hist + i;
        float v;
        if (jj >= 0) v = u[(int64_t)(s.q0 + jj) * ldu + c];
        else {
          v = 0.f;
#pragma unroll
          for (int k = 0; k < kMaxTaps; ++k) if (k == i + s.ql) v = old[k];
        }
        st[(int64_t)i * C] = v;
      }
    }
  }
}

// The same with four neighbouring channels per thread: 16-byte loads and stores (C and ldu multiples of 4, 16-byte aligned
// bases); grid (B, ceil(C / 512), token chunks of CH tokens: shorter chunks than the scalar form, for enough blocks).
template <typename TO> __device__ __forceinline__ void store4(TO* p, float a, float b, float c, float d) {
  struct alignas(4 * sizeof(TO)) V4 { TO v[4]; };
  V4 o;
  o.v[0] = from_f32<TO>(a); o.v[1] = from_f32<TO>(b); o.v[2] = from_f32<TO>(c); o.v[3] = from_f32<TO>(d);
  *reinterpret_cast<V4*>(p) = o;
}

template <int kMaxTaps, int CH, typename TO>
__global__ void __launch_bounds__(128) causal_conv4_kernel(const float* __restrict__ u, int64_t ldu, const float* __restrict__ w,
                                                           const float* __restrict__ bias, TO* __restrict__ out, int C, int taps,
                                                           int act, const int* __restrict__ cu_q, const int* __restrict__ seq_lens,
                                                           const int* __restrict__ slots, float* __restrict__ state) {
  const Seq s = seq_of(cu_q, seq_lens, slots, blockIdx.x);
  const int c = (blockIdx.y * 128 + threadIdx.x) * 4;
  if (c >= C) return;
  const int hist = taps - 1;
  float wt[kMaxTaps][4];
  float4 win[kMaxTaps], old[kMaxTaps];
  const float4 zero = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
  for (int i = 0; i < kMaxTaps; ++i) {
#pragma unroll
    for (int e = 0; e < 4; ++e) wt[i][e] = i < taps ? w[(int64_t)(c + e) * taps + i] : 0.f;
    old[i] = zero;
  }
  const float4 bv = bias != nullptr ? *reinterpret_cast<const float4*>(bias + c) : zero;
  float* st = state != nullptr && s.slot >= 0 ? state + ((int64_t)s.slot * hist) * C + c : nullptr;
  for (int z = blockIdx.z; z * CH < s.ql; z += gridDim.z) {
    const int j0 = z * CH, j1 = min(s.ql, j0 + CH);
    if (z == 0 && st != nullptr && s.ctx > 0) {
#pragma unroll
      for (int i = 0; i < kMaxTaps; ++i) if (i < hist) old[i] = *reinterpret_cast<const float4*>(st + (int64_t)i * C);
    }
#pragma unroll
    for (int i = 0; i < kMaxTaps; ++i) {
      const int jj = j0 - hist + i;
      win[i] = i >= hist ? zero : (jj >= 0 ? *reinterpret_cast<const float4*>(u + (int64_t)(s.q0 + jj) * ldu + c) : old[i]);
    }
    const float* up = u + (int64_t)(s.q0 + j0) * ldu + c;
    TO* op = out + (int64_t)(s.q0 + j0) * C + c;
#pragma unroll 4
    for (int j = j0; j < j1; ++j, up += ldu, op += C) {
      const float4 cur = *reinterpret_cast<const float4*>(up);
      float4 acc = bv;
#pragma unroll
      for (int i = 0; i < kMaxTaps; ++i) {
        if (i < taps) {
          const float4 v = i < hist ? win[i] : cur;
          acc.x = fmaf(wt[i][0], v.x, acc.x); acc.y = fmaf(wt[i][1], v.y, acc.y);
          acc.z = fmaf(wt[i][2], v.z, acc.z); acc.w = fmaf(wt[i][3], v.w, acc.w);
        }
      }
#pragma unroll
      for (int i = 0; i < kMaxTaps - 1; ++i) win[i] = i + 1 < hist ? win[i + 1] : cur;
      store4<TO>(op, act_exact(acc.x, act), act_exact(acc.y, act), act_exact(acc.z, act), act_exact(acc.w, act));
    }
    if (z == 0 && st != nullptr) {
      // new tail: inputs ql - hist .. ql - 1; those before this step's first row come from the old tail
#pragma unroll
      for (int i = 0; i < kMaxTaps; ++i) {
        if (i >= hist) continue;
        const int jj = s.ql - hist + i;
        float4 v = zero;
        if (jj >= 0) v = *reinterpret_cast<const float4*>(u + (int64_t)(s.q0 + jj) * ldu + c);
        else {
#pragma unroll
          for (int k = 0; k < kMaxTaps; ++k) if (k == i + s.ql) v = old[k];
        }
        *reinterpret_cast<float4*>(st + (int64_t)i * C) = v;
      }
    }
  }
}

// ------------------------------------------------------------------------------------------------ elementwise
template <typename TO>
__global__ void __launch_bounds__(256) unary_kernel(const float* __restrict__ x, int64_t ldx, TO* __restrict__ out, int64_t n,
                                                    int cols, int op) {
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
    const float v = x[(i / cols) * ldx + i % cols];
    out[i] = from_f32<TO>(op == 0 ? tanhf(v) : -expf(v));
  }
}

__global__ void __launch_bounds__(256) ssm_dt_kernel(const float* __restrict__ raw, int64_t ldr, const float* __restrict__ dt_bias,
                                                     const float* __restrict__ a_log, float* __restrict__ dt,
                                                     float* __restrict__ logdecay, int64_t n, int H) {
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
    const int h = (int)(i % H);
    const float v = raw[(i / H) * ldr + h] + dt_bias[h];
    const float d = v > 30.f ? v : log1pf(expf(v));
    dt[i] = d;
    logdecay[i] = -expf(a_log[h]) * d;
  }
}

// ------------------------------------------------------------------------------------------------ linear_scan
// One block per (sequence, head, slice of value channels).  Thread (j, r) keeps rows [r * 16, r * 16 + 16) of column j
// of the state in registers (thread index = j * R + r, R a power of two, so the R partial dot products of an output meet
// in one warp shuffle).  Tokens are staged 16 at a time through shared memory -- q, k, per-channel decays (exponentials
// taken while staging), scaled values -- in 16-float strips 20 floats apart, so that the strips a warp reads together lie
// in different banks and every read is a 16-byte one; strips beyond dk hold zeros, which leaves the inner loop without
// bounds checks.  The state lies in memory column-major per head ([dv][dk]: a thread's 16 rows are contiguous).
//
// A recurrence is a dependent chain per token, so one block per (sequence, head) leaves a prompt round of a few long
// sequences bound by latency.  Long portions therefore run in two passes over chunks of `chunk` tokens, every chunk a block:
//   pass 1 (MODE 1)  every chunk but a sequence's last runs from a ZERO state and leaves its summary in scratch: the state
//                    it ends with and the product of its decays (per key row); chunk 0 also copies the sequence's old state;
//   pass 2 (MODE 2)  chunk c rebuilds its true start state from the old state and the summaries of chunks 0 .. c - 1
//                    (S <- D_c' S + S_c'), runs its tokens and writes the outputs; the last chunk writes the new state.
// Pass 2 never reads the state tensor and pass 1 never writes it, so the passes need no ordering inside themselves.
// MODE 0 is the single pass (decode steps, short portions).
constexpr int TCH = 16, SCAN_THREADS = 256;
struct ScanArgs {
  const float* q; int64_t ldq;
  const float* k; int64_t ldk;
  const float* v; int64_t ldv;
  const float* decay; int64_t ldd;     // kind 0: [H] decays; 1: [T, H] log decays; 2: [T, H * dk] log decays
  const float* bonus;                  // [H, dk] or null
  const float* vscale; int64_t ldvs;   // [T, H] or null
  float* out;                          // [T, H * dv]
  float* state;                        // [slots, H, dv, dk]
  const int* cu_q; const int* seq_lens; const int* slots;
  int H, rep, dk, dv, dvt, R;
  // chunked passes: scratch = [B][H][dv][dk] copies of the old states, then [B][nch][H][dv][dk] chunk states, then
  // [B][nch][H][dk] decay products
  float* old_copy; float* chunk_state; float* chunk_decay;
  int chunk, nch, nslices;
};

__device__ __forceinline__ float4 ld4(const float* p, int i, int n, bool vec) {   // p[i .. i+3], zeros beyond n
  if (vec && i + 4 <= n) return *reinterpret_cast<const float4*>(p + i);
  return make_float4(i < n ? p[i] : 0.f, i + 1 < n ? p[i + 1] : 0.f, i + 2 < n ? p[i + 2] : 0.f, i + 3 < n ? p[i + 3] : 0.f);
}
__device__ __forceinline__ void st4(float* p, int i, int n, bool vec, float a, float b, float c, float d) {
  if (vec && i + 4 <= n) { *reinterpret_cast<float4*>(p + i) = make_float4(a, b, c, d); return; }
  if (i < n) p[i] = a;
  if (i + 1 < n) p[i + 1] = b;
  if (i + 2 < n) p[i + 2] = c;
  if (i + 3 < n) p[i + 3] = d;
}

// KPT = key rows per thread.  64 where the key size allows: a warp's lanes then differ only in their value column, the
// staged q / k / decay reads are the same address for the whole warp (shared memory serves them as broadcasts), and every
// loaded value feeds a multiply-add in each lane -- with 16 rows the kernel was bound by shared-memory wavefronts.
template <bool READ_BEFORE, int KIND, int MODE, int KPT>
__global__ void __launch_bounds__(SCAN_THREADS) linear_scan_kernel(ScanArgs a) {
  constexpr int STRIP = KPT + 4;        // floats between staged strips: different banks for the strips of one warp
  extern __shared__ __align__(16) float sm[];
  const Seq s = seq_of(a.cu_q, a.seq_lens, a.slots, blockIdx.x);
  if (s.ql == 0) return;
  const int h = blockIdx.y;
  const int slice = MODE == 0 ? blockIdx.z : blockIdx.z % a.nslices, ch = MODE == 0 ? 0 : blockIdx.z / a.nslices;
  const int j0 = slice * a.dvt;
  const int t_lo = MODE == 0 ? 0 : ch * a.chunk, t_hi = MODE == 0 ? s.ql : min(s.ql, t_lo + a.chunk);
  if (t_lo >= s.ql) return;
  const bool last_chunk = MODE == 0 || t_hi == s.ql;
  const int nj = min(a.dvt, a.dv - j0);
  const int dk = a.dk, R = a.R, row = R * STRIP;      // floats per staged token
  const int jl = threadIdx.x / R, r = threadIdx.x % R;
  const bool live = jl < nj;
  const int j = j0 + jl, i0 = r * KPT;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = blockDim.x >> 5;
  float* qs = sm;                       // [TCH][row]
  float* ks = qs + TCH * row;           // [TCH][row]
  float* as = ks + TCH * row;           // [TCH][row] (kind 2) or [TCH] (kind 1)
  float* us = as + (KIND == 2 ? TCH * row : TCH);            // [TCH][row] bonus * k (READ_BEFORE)
  float* vs = us + (READ_BEFORE ? TCH * row : 0);            // [TCH][dvt]
  float S[KPT], dp[KIND == 2 && MODE == 1 ? KPT : 1];
  float dps = 1.f;                      // decay product of a chunk when it is one number per head
  const int64_t col = live ? j : 0;
  float* sp = a.state + (((int64_t)s.slot * a.H + h) * a.dv + col) * dk;
  const bool vec = (dk & 3) == 0;       // every row of a state column and of a summary is 16-byte aligned
  const int64_t bh = (int64_t)blockIdx.x * a.H + h;
  auto load_col = [&](const float* p, bool on) {
#pragma unroll
    for (int g = 0; g < KPT; g += 4) {
      const float4 t = on ? ld4(p, i0 + g, dk, vec) : make_float4(0.f, 0.f, 0.f, 0.f);
      S[g] = t.x; S[g + 1] = t.y; S[g + 2] = t.z; S[g + 3] = t.w;
    }
  };
  auto store_col = [&](float* p) {
#pragma unroll
    for (int g = 0; g < KPT; g += 4) st4(p, i0 + g, dk, vec, S[g], S[g + 1], S[g + 2], S[g + 3]);
  };
  if (MODE == 0) {
    load_col(sp, live && s.ctx > 0);
  } else if (MODE == 1) {
    if (ch == 0 && live) {               // the old state, for pass 2 (which must not read the state tensor)
      load_col(sp, s.ctx > 0);
      store_col(a.old_copy + (bh * a.dv + col) * dk);
    }
    if (last_chunk) return;              // nobody needs the last chunk's summary
#pragma unroll
    for (int ii = 0; ii < KPT; ++ii) S[ii] = 0.f;
    if (KIND == 2) {
#pragma unroll
      for (int ii = 0; ii < (KIND == 2 && MODE == 1 ? KPT : 1); ++ii) dp[ii] = 1.f;
    }
  } else {
    load_col(a.old_copy + (bh * a.dv + col) * dk, live);
    for (int c = 0; c < ch; ++c) {
      const int64_t cb = ((int64_t)blockIdx.x * a.nch + c) * a.H + h;
      const float* cs = a.chunk_state + (cb * a.dv + col) * dk;
      const float* cd = a.chunk_decay + cb * dk;
#pragma unroll
      for (int g = 0; g < KPT; g += 4) {
        const float4 sl = live ? ld4(cs, i0 + g, dk, vec) : make_float4(0.f, 0.f, 0.f, 0.f);
        const float4 d4 = ld4(cd, i0 + g, dk, vec);
        S[g] = fmaf(d4.x, S[g], sl.x); S[g + 1] = fmaf(d4.y, S[g + 1], sl.y);
        S[g + 2] = fmaf(d4.z, S[g + 2], sl.z); S[g + 3] = fmaf(d4.w, S[g + 3], sl.w);
      }
    }
  }
  const float a_const = KIND == 0 ? a.decay[h] : 0.f;
  const int hq = h / a.rep;
  const float* bon = (READ_BEFORE && a.bonus != nullptr) ? a.bonus + (int64_t)h * dk : nullptr;
  if (MODE == 0 && s.ql == 1) {
    // a decode step: one token, nothing to share through shared memory -- every thread fetches its rows of q, k and the
    // decays itself (the threads of a column group read the same lines), so these loads and the state's are in flight together
    const int64_t t = s.q0;
    const float* qp = a.q + t * a.ldq + (int64_t)hq * dk;
    const float* kp = a.k + t * a.ldk + (int64_t)hq * dk;
    const float* dpp = KIND == 2 ? a.decay + t * a.ldd + (int64_t)h * dk : nullptr;
    const bool vq = vec && ((reinterpret_cast<uintptr_t>(qp) | reinterpret_cast<uintptr_t>(kp) | reinterpret_cast<uintptr_t>(dpp) |
                             reinterpret_cast<uintptr_t>(bon)) & 15) == 0;
    const float at = KIND == 1 ? expf(a.decay[t * a.ldd + h]) : a_const;
    float vj = live ? a.v[t * a.ldv + (int64_t)h * a.dv + j] : 0.f;
    if (a.vscale != nullptr) vj *= a.vscale[t * a.ldvs + h];
    float acc0 = 0.f, acc1 = 0.f;
#pragma unroll
    for (int g = 0; g < KPT; g += 4) {
      const float4 q4 = ld4(qp, i0 + g, dk, vq), k4 = ld4(kp, i0 + g, dk, vq);
      float4 d4 = make_float4(at, at, at, at), u4 = make_float4(0.f, 0.f, 0.f, 0.f);
      if (KIND == 2) { d4 = ld4(dpp, i0 + g, dk, vq); d4 = make_float4(expf(d4.x), expf(d4.y), expf(d4.z), expf(d4.w)); }
      if (READ_BEFORE && bon != nullptr) u4 = ld4(bon, i0 + g, dk, vq);
      const float qq[4] = {q4.x, q4.y, q4.z, q4.w}, kk[4] = {k4.x, k4.y, k4.z, k4.w}, dd[4] = {d4.x, d4.y, d4.z, d4.w},
                  uu[4] = {u4.x, u4.y, u4.z, u4.w};
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float x = kk[e] * vj;
        float& acc = (e & 1) ? acc1 : acc0;
        if (READ_BEFORE) {
          acc = fmaf(qq[e], fmaf(uu[e], x, S[g + e]), acc);
          S[g + e] = fmaf(dd[e], S[g + e], x);
        } else {
          S[g + e] = fmaf(dd[e], S[g + e], x);
          acc = fmaf(qq[e], S[g + e], acc);
        }
      }
    }
    float acc = acc0 + acc1;
    for (int o = 1; o < R; o <<= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
    if (live) {
      if (r == 0) a.out[t * a.H * a.dv + (int64_t)h * a.dv + j] = acc;
      store_col(sp);
    }
    return;
  }
  for (int c0 = t_lo; c0 < t_hi; c0 += TCH) {
    const int nt = min(TCH, t_hi - c0);
    __syncthreads();
    for (int tt = warp; tt < nt; tt += nwarp) {
      const int64_t t = s.q0 + c0 + tt;
      for (int i = lane; i < R * KPT; i += 32) {
        const int p = tt * row + (i / KPT) * STRIP + (i % KPT);
        const bool in = i < dk;
        const float kx = in ? a.k[t * a.ldk + (int64_t)hq * dk + i] : 0.f;
        if (MODE != 1) qs[p] = in ? a.q[t * a.ldq + (int64_t)hq * dk + i] : 0.f;
        ks[p] = kx;
        if (KIND == 2) as[p] = in ? expf(a.decay[t * a.ldd + (int64_t)h * dk + i]) : 0.f;
        if (READ_BEFORE && MODE != 1) us[p] = (in && bon != nullptr) ? bon[i] * kx : 0.f;
      }
      const float sc = a.vscale != nullptr ? a.vscale[t * a.ldvs + h] : 1.f;
      for (int jj = lane; jj < nj; jj += 32) vs[tt * a.dvt + jj] = a.v[t * a.ldv + (int64_t)h * a.dv + j0 + jj] * sc;
      if (KIND == 1 && lane == 0) as[tt] = expf(a.decay[t * a.ldd + h]);
    }
    __syncthreads();
#pragma unroll 1
    for (int tt = 0; tt < nt; ++tt) {
      const float vj = live ? vs[tt * a.dvt + jl] : 0.f;
      const float at = KIND == 1 ? as[tt] : a_const;
      const float4* q4 = reinterpret_cast<const float4*>(qs + tt * row + r * STRIP);
      const float4* k4 = reinterpret_cast<const float4*>(ks + tt * row + r * STRIP);
      const float4* a4 = reinterpret_cast<const float4*>(as + tt * row + r * STRIP);
      const float4* u4 = reinterpret_cast<const float4*>(us + tt * row + r * STRIP);
      float acc[4] = {0.f, 0.f, 0.f, 0.f};
      if (KIND != 2 && MODE == 1) dps *= at;
#pragma unroll
      for (int g = 0; g < KPT / 4; ++g) {
        const float4 kv4 = k4[g];
        float4 qv = make_float4(0.f, 0.f, 0.f, 0.f), dv4 = make_float4(at, at, at, at), uv = make_float4(0.f, 0.f, 0.f, 0.f);
        if (MODE != 1) qv = q4[g];
        if (KIND == 2) dv4 = a4[g];
        if (READ_BEFORE && MODE != 1) uv = u4[g];
        const float qq[4] = {qv.x, qv.y, qv.z, qv.w}, kk[4] = {kv4.x, kv4.y, kv4.z, kv4.w}, dd[4] = {dv4.x, dv4.y, dv4.z, dv4.w},
                    uu[4] = {uv.x, uv.y, uv.z, uv.w};
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int ii = g * 4 + e;
          const float kv = kk[e] * vj;
          if (MODE == 1) {
            S[ii] = fmaf(dd[e], S[ii], kv);
            if (KIND == 2) dp[KIND == 2 && MODE == 1 ? ii : 0] *= dd[e];
          } else if (READ_BEFORE) {
            acc[e] = fmaf(qq[e], fmaf(uu[e], vj, S[ii]), acc[e]);     // uu = bonus * k
            S[ii] = fmaf(dd[e], S[ii], kv);
          } else {
            S[ii] = fmaf(dd[e], S[ii], kv);
            acc[e] = fmaf(qq[e], S[ii], acc[e]);
          }
        }
      }
      if (MODE != 1) {
        float o = (acc[0] + acc[1]) + (acc[2] + acc[3]);
        for (int w = 1; w < R; w <<= 1) o += __shfl_xor_sync(0xffffffffu, o, w);
        if (live && r == 0) a.out[(int64_t)(s.q0 + c0 + tt) * a.H * a.dv + (int64_t)h * a.dv + j] = o;
      }
    }
  }
  if (MODE == 1) {
    const int64_t cb = ((int64_t)blockIdx.x * a.nch + ch) * a.H + h;
    if (live) store_col(a.chunk_state + (cb * a.dv + col) * dk);
    if (slice == 0 && jl == 0) {
      float* cd = a.chunk_decay + cb * dk;
#pragma unroll
      for (int g = 0; g < KPT; g += 4) {
        if (KIND == 2) st4(cd, i0 + g, dk, vec, dp[KIND == 2 && MODE == 1 ? g : 0], dp[KIND == 2 && MODE == 1 ? g + 1 : 0],
                           dp[KIND == 2 && MODE == 1 ? g + 2 : 0], dp[KIND == 2 && MODE == 1 ? g + 3 : 0]);
        else st4(cd, i0 + g, dk, vec, dps, dps, dps, dps);
      }
    }
  } else if (live && last_chunk) {
    store_col(sp);
  }
}

// The same recurrence with a two-dimensional register tile: a thread owns 8 key rows x 8 value columns of the state, so the
// 8 + 8 (+ 8 + 8) staged values it reads per token feed 64 state elements (the column-per-thread form above reads one
// staged value per element and is bound by shared-memory wavefronts).  RG row groups of 8 (8 for key sizes up to 64, 16 up
// to 128) are adjacent lanes; an output column is finished by a reduce-scatter over those lanes (4 + 2 + 1 shuffles leave
// lane g with column g), so a warp's stores are 32 consecutive outputs.  Same passes (MODE) and state layout as above.
constexpr int TSTR = 12;    // floats between the staged 8-row groups of a token: the 8 groups a quarter warp reads lie in different banks

template <bool READ_BEFORE, int KIND, int MODE, int RG>
__global__ void __launch_bounds__(128) linear_scan_tile_kernel(ScanArgs a) {
  extern __shared__ __align__(16) float sm[];
  const Seq s = seq_of(a.cu_q, a.seq_lens, a.slots, blockIdx.x);
  if (s.ql == 0) return;
  const int h = blockIdx.y;
  const int slice = MODE == 0 ? blockIdx.z : blockIdx.z % a.nslices, ch = MODE == 0 ? 0 : blockIdx.z / a.nslices;
  const int j0 = slice * a.dvt;
  const int t_lo = MODE == 0 ? 0 : ch * a.chunk, t_hi = MODE == 0 ? s.ql : min(s.ql, t_lo + a.chunk);
  if (t_lo >= s.ql) return;
  const bool last_chunk = MODE == 0 || t_hi == s.ql;
  const int nj = min(a.dvt, a.dv - j0);          // value columns of this block
  const int dk = a.dk;
  constexpr int row = RG * TSTR;                 // floats per staged token
  const int cg = threadIdx.x / RG, rg = threadIdx.x % RG;
  const int i0 = rg * 8, c0 = cg * 8;            // first key row / first column (inside the slice) of this thread
  float* qs = sm;
  float* ks = qs + TCH * row;
  float* as = ks + TCH * row;                                   // [TCH][row] (kind 2) or [TCH] (kind 1)
  float* us = as + (KIND == 2 ? TCH * row : TCH);               // bonus * k (READ_BEFORE)
  float* vs = us + (READ_BEFORE ? TCH * row : 0);               // [TCH][dvt]
  float S[8][8], dp[8];
  float dps = 1.f;
  const bool vec = (dk & 3) == 0;
  const int64_t bh = (int64_t)blockIdx.x * a.H + h;
  float* sp = a.state + ((int64_t)s.slot * a.H + h) * a.dv * dk;           // this head's [dv][dk]
  auto load_tile = [&](const float* base, bool on) {
#pragma unroll
    for (int c = 0; c < 8; ++c) {
      const bool ok = on && c0 + c < nj;
      const float* p = base + (int64_t)(j0 + c0 + c) * dk;
      const float4 x = ok ? ld4(p, i0, dk, vec) : make_float4(0.f, 0.f, 0.f, 0.f);
      const float4 y = ok ? ld4(p, i0 + 4, dk, vec) : make_float4(0.f, 0.f, 0.f, 0.f);
      S[0][c] = x.x; S[1][c] = x.y; S[2][c] = x.z; S[3][c] = x.w; S[4][c] = y.x; S[5][c] = y.y; S[6][c] = y.z; S[7][c] = y.w;
    }
  };
  auto store_tile = [&](float* base) {
#pragma unroll
    for (int c = 0; c < 8; ++c) {
      if (c0 + c >= nj) continue;
      float* p = base + (int64_t)(j0 + c0 + c) * dk;
      st4(p, i0, dk, vec, S[0][c], S[1][c], S[2][c], S[3][c]);
      st4(p, i0 + 4, dk, vec, S[4][c], S[5][c], S[6][c], S[7][c]);
    }
  };
  if (MODE == 0) {
    load_tile(sp, s.ctx > 0);
  } else if (MODE == 1) {
    if (ch == 0) {
      load_tile(sp, s.ctx > 0);
      store_tile(a.old_copy + bh * a.dv * dk);
    }
    if (last_chunk) return;
#pragma unroll
    for (int r = 0; r < 8; ++r) {
      dp[r] = 1.f;
#pragma unroll
      for (int c = 0; c < 8; ++c) S[r][c] = 0.f;
    }
  } else {
    load_tile(a.old_copy + bh * a.dv * dk, true);
    for (int cc = 0; cc < ch; ++cc) {
      const int64_t cb = ((int64_t)blockIdx.x * a.nch + cc) * a.H + h;
      const float* cs = a.chunk_state + cb * a.dv * dk;
      const float* cd = a.chunk_decay + cb * dk;
      const float4 d0 = ld4(cd, i0, dk, vec), d1 = ld4(cd, i0 + 4, dk, vec);
      const float d[8] = {d0.x, d0.y, d0.z, d0.w, d1.x, d1.y, d1.z, d1.w};
#pragma unroll
      for (int c = 0; c < 8; ++c) {
        if (c0 + c >= nj) continue;
        const float* p = cs + (int64_t)(j0 + c0 + c) * dk;
        const float4 x = ld4(p, i0, dk, vec), y = ld4(p, i0 + 4, dk, vec);
        const float sl[8] = {x.x, x.y, x.z, x.w, y.x, y.y, y.z, y.w};
#pragma unroll
        for (int r = 0; r < 8; ++r) S[r][c] = fmaf(d[r], S[r][c], sl[r]);
      }
    }
  }
  const float a_const = KIND == 0 ? a.decay[h] : 0.f;
  const int hq = h / a.rep;
  const float* bon = (READ_BEFORE && a.bonus != nullptr) ? a.bonus + (int64_t)h * dk : nullptr;
  // one token: q / k / decay / bonus * k rows and the scaled value columns of this thread in registers -> outputs
  auto step = [&](const float (&qq)[8], const float (&kk)[8], const float (&dd)[8], const float (&uk)[8], const float (&vv)[8],
                  int64_t t) {
    float acc[8];
    float quk = 0.f;
#pragma unroll
    for (int c = 0; c < 8; ++c) acc[c] = 0.f;
    if (READ_BEFORE && MODE != 1) {
#pragma unroll
      for (int r = 0; r < 8; ++r) quk = fmaf(qq[r], uk[r], quk);
    }
#pragma unroll
    for (int r = 0; r < 8; ++r) {
#pragma unroll
      for (int c = 0; c < 8; ++c) {
        if (MODE == 1) {
          S[r][c] = fmaf(dd[r], S[r][c], kk[r] * vv[c]);
        } else if (READ_BEFORE) {
          acc[c] = fmaf(qq[r], S[r][c], acc[c]);
          S[r][c] = fmaf(dd[r], S[r][c], kk[r] * vv[c]);
        } else {
          S[r][c] = fmaf(dd[r], S[r][c], kk[r] * vv[c]);
          acc[c] = fmaf(qq[r], S[r][c], acc[c]);
        }
      }
      if (MODE == 1 && KIND == 2) dp[r] *= dd[r];
    }
    if (MODE == 1) return;
    if (READ_BEFORE) {
#pragma unroll
      for (int c = 0; c < 8; ++c) acc[c] = fmaf(vv[c], quk, acc[c]);       // the current token's bonus term
    }
    if (RG == 16) {
#pragma unroll
      for (int c = 0; c < 8; ++c) acc[c] += __shfl_xor_sync(0xffffffffu, acc[c], 8);
    }
    // reduce-scatter over the 8 lanes of a column group: lane g ends with column g
    float b4[4], b2[2];
    const bool hi4 = rg & 4, hi2 = rg & 2, hi1 = rg & 1;
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      const float give = hi4 ? acc[c] : acc[c + 4];
      b4[c] = (hi4 ? acc[c + 4] : acc[c]) + __shfl_xor_sync(0xffffffffu, give, 4);
    }
#pragma unroll
    for (int c = 0; c < 2; ++c) {
      const float give = hi2 ? b4[c] : b4[c + 2];
      b2[c] = (hi2 ? b4[c + 2] : b4[c]) + __shfl_xor_sync(0xffffffffu, give, 2);
    }
    const float give = hi1 ? b2[0] : b2[1];
    const float o = (hi1 ? b2[1] : b2[0]) + __shfl_xor_sync(0xffffffffu, give, 1);
    const int c = rg & 7;
    if ((RG == 8 || rg < 8) && c0 + c < nj) a.out[t * a.H * a.dv + (int64_t)h * a.dv + j0 + c0 + c] = o;
  };
  if (MODE == 0 && s.ql == 1) {   // a decode step: straight from global memory, no staging, no barrier
    const int64_t t = s.q0;
    const float* qp = a.q + t * a.ldq + (int64_t)hq * dk;
    const float* kp = a.k + t * a.ldk + (int64_t)hq * dk;
    const float* dpp = KIND == 2 ? a.decay + t * a.ldd + (int64_t)h * dk : nullptr;
    const float* vp = a.v + t * a.ldv + (int64_t)h * a.dv + j0;
    const bool vq = vec && ((reinterpret_cast<uintptr_t>(qp) | reinterpret_cast<uintptr_t>(kp) | reinterpret_cast<uintptr_t>(dpp) |
                             reinterpret_cast<uintptr_t>(bon)) & 15) == 0;
    const bool vv4 = (reinterpret_cast<uintptr_t>(vp) & 15) == 0;
    const float at = KIND == 1 ? expf(a.decay[t * a.ldd + h]) : a_const;
    const float sc = a.vscale != nullptr ? a.vscale[t * a.ldvs + h] : 1.f;
    float qq[8], kk[8], dd[8], uk[8], vv[8];
    const float4 q0 = ld4(qp, i0, dk, vq), q1 = ld4(qp, i0 + 4, dk, vq), k0 = ld4(kp, i0, dk, vq), k1 = ld4(kp, i0 + 4, dk, vq);
    const float4 v0 = ld4(vp, c0, nj, vv4), v1 = ld4(vp, c0 + 4, nj, vv4);
    const float qa[8] = {q0.x, q0.y, q0.z, q0.w, q1.x, q1.y, q1.z, q1.w}, ka[8] = {k0.x, k0.y, k0.z, k0.w, k1.x, k1.y, k1.z, k1.w};
    const float va[8] = {v0.x, v0.y, v0.z, v0.w, v1.x, v1.y, v1.z, v1.w};
    float da[8] = {at, at, at, at, at, at, at, at}, ua[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    if (KIND == 2) {
      const float4 x = ld4(dpp, i0, dk, vq), y = ld4(dpp, i0 + 4, dk, vq);
      da[0] = expf(x.x); da[1] = expf(x.y); da[2] = expf(x.z); da[3] = expf(x.w);
      da[4] = i0 + 4 < dk ? expf(y.x) : 0.f; da[5] = expf(y.y); da[6] = expf(y.z); da[7] = expf(y.w);
    }
    if (READ_BEFORE && bon != nullptr) {
      const float4 x = ld4(bon, i0, dk, vq), y = ld4(bon, i0 + 4, dk, vq);
      ua[0] = x.x; ua[1] = x.y; ua[2] = x.z; ua[3] = x.w; ua[4] = y.x; ua[5] = y.y; ua[6] = y.z; ua[7] = y.w;
    }
#pragma unroll
    for (int r = 0; r < 8; ++r) { qq[r] = qa[r]; kk[r] = ka[r]; dd[r] = da[r]; uk[r] = ua[r] * ka[r]; vv[r] = va[r] * sc; }
    step(qq, kk, dd, uk, vv, t);
    store_tile(sp);
    return;
  }
  const float* qbase = a.q + (int64_t)hq * dk;
  const float* kbase = a.k + (int64_t)hq * dk;
  const float* dbase = KIND == 2 ? a.decay + (int64_t)h * dk : nullptr;
  const float* vbase = a.v + (int64_t)h * a.dv + j0;
  // whole 16-byte vectors of q / k / decay / bonus rows: the row count, the row strides and the bases allow it
  const bool in_vec = vec && ((a.ldq | a.ldk | (KIND == 2 ? a.ldd : 0)) & 3) == 0 &&
                      ((reinterpret_cast<uintptr_t>(qbase) | reinterpret_cast<uintptr_t>(kbase) | reinterpret_cast<uintptr_t>(dbase) |
                        reinterpret_cast<uintptr_t>(bon)) & 15) == 0;
  // Register prefetch: the next stage's rows are fetched (16-byte loads, up to four per array and thread) before the current
  // stage's tokens are computed and written to shared memory after them, so their latency hides behind the arithmetic.
  const int nthr = blockDim.x;
  const bool v_vec = (a.dvt & 3) == 0 && nj == a.dvt && (a.ldv & 3) == 0 && (reinterpret_cast<uintptr_t>(vbase) & 15) == 0;
  const bool pf = in_vec && v_vec && nthr * 4 >= TCH * RG * 2 && nthr * 16 >= TCH * a.dvt;
  float4 rq[4], rk[4], rd[4], rv[4];
  float rdec = 0.f;
  auto fetch = [&](int t0n, int ntn) {
    const float4 z = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int idx = threadIdx.x + u * nthr;
      rq[u] = rk[u] = rd[u] = rv[u] = z;
      if (idx < ntn * (RG * 2)) {
        const int tt = idx / (RG * 2), i = (idx % (RG * 2)) * 4;
        const int64_t t = s.q0 + t0n + tt;
        if (i < dk) {
          rk[u] = *reinterpret_cast<const float4*>(kbase + t * a.ldk + i);
          if (MODE != 1) rq[u] = *reinterpret_cast<const float4*>(qbase + t * a.ldq + i);
          if (KIND == 2) rd[u] = *reinterpret_cast<const float4*>(dbase + t * a.ldd + i);
        }
      }
      if (idx < ntn * (a.dvt >> 2)) {
        const int tt = idx / (a.dvt >> 2), jj = (idx % (a.dvt >> 2)) * 4;
        const int64_t t = s.q0 + t0n + tt;
        const float sc = a.vscale != nullptr ? a.vscale[t * a.ldvs + h] : 1.f;
        const float4 x = *reinterpret_cast<const float4*>(vbase + t * a.ldv + jj);
        rv[u] = make_float4(x.x * sc, x.y * sc, x.z * sc, x.w * sc);
      }
    }
    if (KIND == 1 && threadIdx.x < ntn) rdec = a.decay[(int64_t)(s.q0 + t0n + threadIdx.x) * a.ldd + h];
  };
  auto commit = [&](int ntn) {
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int idx = threadIdx.x + u * nthr;
      if (idx < ntn * (RG * 2)) {
        const int tt = idx / (RG * 2), i = (idx % (RG * 2)) * 4;
        const int p = tt * row + (i >> 3) * TSTR + (i & 7);
        const bool in = i < dk;
        if (MODE != 1) *reinterpret_cast<float4*>(qs + p) = rq[u];
        *reinterpret_cast<float4*>(ks + p) = rk[u];
        if (KIND == 2) *reinterpret_cast<float4*>(as + p) = in ? make_float4(expf(rd[u].x), expf(rd[u].y), expf(rd[u].z), expf(rd[u].w))
                                                               : make_float4(0.f, 0.f, 0.f, 0.f);
        if (READ_BEFORE && MODE != 1) {
          const float4 b4 = (in && bon != nullptr) ? *reinterpret_cast<const float4*>(bon + i) : make_float4(0.f, 0.f, 0.f, 0.f);
          *reinterpret_cast<float4*>(us + p) = make_float4(b4.x * rk[u].x, b4.y * rk[u].y, b4.z * rk[u].z, b4.w * rk[u].w);
        }
      }
      if (idx < ntn * (a.dvt >> 2)) *reinterpret_cast<float4*>(vs + idx * 4) = rv[u];
    }
    if (KIND == 1 && threadIdx.x < ntn) as[threadIdx.x] = expf(rdec);
  };
  if (pf) fetch(t_lo, min(TCH, t_hi - t_lo));
  for (int t0 = t_lo; t0 < t_hi; t0 += TCH) {
    const int nt = min(TCH, t_hi - t0);
    __syncthreads();
    if (pf) {
      commit(nt);
      __syncthreads();
      if (t0 + TCH < t_hi) fetch(t0 + TCH, min(TCH, t_hi - t0 - TCH));
    } else {
    // flattened over (token, row) so that a thread's loads are independent and many are in flight at once; 16-byte loads
    // where the rows allow
    if (in_vec) {
#pragma unroll 4
      for (int idx = threadIdx.x; idx < nt * (RG * 2); idx += blockDim.x) {
        const int tt = idx / (RG * 2), i = (idx % (RG * 2)) * 4;
        const int p = tt * row + (i >> 3) * TSTR + (i & 7);
        const float4 z = make_float4(0.f, 0.f, 0.f, 0.f);
        const bool in = i < dk;                    // dk is a multiple of 4 here: whole vectors
        const int64_t t = s.q0 + t0 + tt;
        const float4 k4 = in ? *reinterpret_cast<const float4*>(kbase + t * a.ldk + i) : z;
        if (MODE != 1) *reinterpret_cast<float4*>(qs + p) = in ? *reinterpret_cast<const float4*>(qbase + t * a.ldq + i) : z;
        *reinterpret_cast<float4*>(ks + p) = k4;
        if (KIND == 2) {
          const float4 d4 = in ? *reinterpret_cast<const float4*>(dbase + t * a.ldd + i) : z;
          *reinterpret_cast<float4*>(as + p) = in ? make_float4(expf(d4.x), expf(d4.y), expf(d4.z), expf(d4.w)) : z;
        }
        if (READ_BEFORE && MODE != 1) {
          const float4 b4 = (in && bon != nullptr) ? *reinterpret_cast<const float4*>(bon + i) : z;
          *reinterpret_cast<float4*>(us + p) = make_float4(b4.x * k4.x, b4.y * k4.y, b4.z * k4.z, b4.w * k4.w);
        }
      }
    } else {
#pragma unroll 4
      for (int idx = threadIdx.x; idx < nt * (RG * 8); idx += blockDim.x) {
        const int tt = idx / (RG * 8), i = idx % (RG * 8);
        const int64_t t = s.q0 + t0 + tt;
        const int p = tt * row + (i >> 3) * TSTR + (i & 7);
        const bool in = i < dk;
        const float kx = in ? kbase[t * a.ldk + i] : 0.f;
        if (MODE != 1) qs[p] = in ? qbase[t * a.ldq + i] : 0.f;
        ks[p] = kx;
        if (KIND == 2) as[p] = in ? expf(dbase[t * a.ldd + i]) : 0.f;
        if (READ_BEFORE && MODE != 1) us[p] = (in && bon != nullptr) ? bon[i] * kx : 0.f;
      }
    }
#pragma unroll 4
    for (int idx = threadIdx.x; idx < nt * a.dvt; idx += blockDim.x) {
      const int tt = idx / a.dvt, jj = idx % a.dvt;
      const int64_t t = s.q0 + t0 + tt;
      const float sc = a.vscale != nullptr ? a.vscale[t * a.ldvs + h] : 1.f;
      vs[idx] = jj < nj ? vbase[t * a.ldv + jj] * sc : 0.f;
    }
    if (KIND == 1 && threadIdx.x < nt) as[threadIdx.x] = expf(a.decay[(int64_t)(s.q0 + t0 + threadIdx.x) * a.ldd + h]);
    __syncthreads();
    }
#pragma unroll 1
    for (int tt = 0; tt < nt; ++tt) {
      const float at = KIND == 1 ? as[tt] : a_const;
      if (KIND != 2 && MODE == 1) dps *= at;
      float qq[8], kk[8], dd[8], uk[8], vv[8];
      const int p = tt * row + rg * TSTR;
#pragma unroll
      for (int g = 0; g < 2; ++g) {
        const float4 k4 = *reinterpret_cast<const float4*>(ks + p + 4 * g);
        const float4 v4 = *reinterpret_cast<const float4*>(vs + tt * a.dvt + c0 + 4 * g);
        float4 q4 = make_float4(0.f, 0.f, 0.f, 0.f), d4 = make_float4(at, at, at, at), u4 = make_float4(0.f, 0.f, 0.f, 0.f);
        if (MODE != 1) q4 = *reinterpret_cast<const float4*>(qs + p + 4 * g);
        if (KIND == 2) d4 = *reinterpret_cast<const float4*>(as + p + 4 * g);
        if (READ_BEFORE && MODE != 1) u4 = *reinterpret_cast<const float4*>(us + p + 4 * g);
        kk[4 * g] = k4.x; kk[4 * g + 1] = k4.y; kk[4 * g + 2] = k4.z; kk[4 * g + 3] = k4.w;
        vv[4 * g] = v4.x; vv[4 * g + 1] = v4.y; vv[4 * g + 2] = v4.z; vv[4 * g + 3] = v4.w;
        qq[4 * g] = q4.x; qq[4 * g + 1] = q4.y; qq[4 * g + 2] = q4.z; qq[4 * g + 3] = q4.w;
        dd[4 * g] = d4.x; dd[4 * g + 1] = d4.y; dd[4 * g + 2] = d4.z; dd[4 * g + 3] = d4.w;
        uk[4 * g] = u4.x; uk[4 * g + 1] = u4.y; uk[4 * g + 2] = u4.z; uk[4 * g + 3] = u4.w;
      }
      step(qq, kk, dd, uk, vv, s.q0 + t0 + tt);
    }
  }
  if (MODE == 1) {
    const int64_t cb = ((int64_t)blockIdx.x * a.nch + ch) * a.H + h;
    store_tile(a.chunk_state + cb * a.dv * dk);
    if (slice == 0 && cg == 0) {
      float* cd = a.chunk_decay + cb * dk;
      if (KIND == 2) { st4(cd, i0, dk, vec, dp[0], dp[1], dp[2], dp[3]); st4(cd, i0 + 4, dk, vec, dp[4], dp[5], dp[6], dp[7]); }
      else { st4(cd, i0, dk, vec, dps, dps, dps, dps); st4(cd, i0 + 4, dk, vec, dps, dps, dps, dps); }
    }
  } else if (last_chunk) {
    store_tile(sp);
  }
}

// ------------------------------------------------------------------------------------------------ gated_rmsnorm
struct GnArgs {
  const float* o; int64_t ldo;
  const float* gate; int64_t ldg;
  const float* weight;
  const float* skip_x; int64_t ldx;
  const float* skip_d;
  int C, groups, H, gate_act, gate_first;
  float eps;
};
__device__ __forceinline__ float gate_fn(float g, int kind) {
  if (kind == 1) return g / (1.f + expf(-g));
  if (kind == 2) return 1.f / (1.f + expf(-g));
  return g;
}
__device__ __forceinline__ float gn_value(const GnArgs& a, int64_t t, int c) {
  float v = a.o[t * a.ldo + c];
  if (a.skip_x != nullptr) v = fmaf(a.skip_d[c / (a.C / a.H)], a.skip_x[t * a.ldx + c], v);
  if (a.gate != nullptr && a.gate_first) v *= gate_fn(a.gate[t * a.ldg + c], a.gate_act);
  return v;
}
// one block per row; a warp per group while there are at least as many groups as warps, else the block per group
template <typename T>
__global__ void __launch_bounds__(256) gated_rmsnorm_kernel(GnArgs a, T* __restrict__ out) {
  __shared__ float red[32];
  const int64_t t = blockIdx.x;
  const int gs = a.C / a.groups, lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
  const bool per_warp = a.groups >= nw;
  for (int g = per_warp ? warp : 0; g < a.groups; g += per_warp ? nw : 1) {
    float ss = 0.f;
    for (int c = per_warp ? lane : threadIdx.x; c < gs; c += per_warp ? 32 : blockDim.x) {
      const float v = gn_value(a, t, g * gs + c);
      ss = fmaf(v, v, ss);
    }
    ss = per_warp ? warp_sum(ss) : block_sum(ss, red);
    const float r = rsqrtf(ss / gs + a.eps);
    for (int c = per_warp ? lane : threadIdx.x; c < gs; c += per_warp ? 32 : blockDim.x) {
      const int cc = g * gs + c;
      float v = gn_value(a, t, cc) * r;
      if (a.weight != nullptr) v *= a.weight[cc];
      if (a.gate != nullptr && !a.gate_first) v *= gate_fn(a.gate[t * a.ldg + cc], a.gate_act);
      out[t * a.C + cc] = from_f32<T>(v);
    }
  }
}

int grid_for(int64_t n) {
  const int64_t b = (n + 255) / 256;
  return (int)(b < 148 * 8 ? b : 148 * 8);
}

int pow2_at_least(int n) {
  int p = 1;
  while (p < n) p <<= 1;
  return p;
}

}  // namespace

LLMSS_API int llmss_embed_bigram(const int* tokens, const void* wte, const void* table, float* out, int T_, int W, int vocab,
                                 int64_t mul_prev, int64_t mul_cur, int buckets, const int* cu_q, const int* seq_lens,
                                 const int* slots, int B, int max_q, int* prev_state, int dtype, cudaStream_t stream) {
  if (B <= 0 || T_ <= 0) return 0;
  const dim3 grid(B, max(1, min(max_q, 256)));
  LLMSS_BY_DTYPE(dtype, (embed_bigram_kernel<T><<<grid, 128, 0, stream>>>(tokens, (const T*)wte, (const T*)table, out, W, vocab, mul_prev,
                                                                          mul_cur, buckets, cu_q, seq_lens, slots, prev_state)));
  LLMSS_CHECK_CUDA(cudaGetLastError());
  return 0;
}

LLMSS_API int llmss_postnorm_residual(const float* y, int64_t ldy, const float* y2, int64_t ldy2, const float* w_a, const float* w_b,
                                      const float* weight, const float* resid, int64_t ldr, float* new_resid, void* out, int T_,
                                      int W, float eps, int one_plus, int dtype, cudaStream_t stream) {
  if (T_ <= 0) return 0;
  LLMSS_REQUIRE(y2 == nullptr || (w_a != nullptr && w_b != nullptr), "postnorm_residual: two branches need two weights");
  LLMSS_BY_DTYPE(dtype, (postnorm_kernel<T><<<T_, 256, 0, stream>>>(y, ldy, y2, ldy2, w_a, w_b, weight, resid, ldr, new_resid, (T*)out, W,
                                                                    eps, one_plus)));
  LLMSS_CHECK_CUDA(cudaGetLastError());
  return 0;
}

LLMSS_API int llmss_token_shift(const float* x, int64_t ldx, const float* mu, int S, void* out, int T_, int W, const int* cu_q,
                                const int* seq_lens, const int* slots, int B, int max_q, float* prev_state, int dtype,
                                cudaStream_t stream) {
  if (B <= 0 || T_ <= 0) return 0;
  // a decode batch has one row per sequence: spread its columns over blocks instead
  const bool vec = W % 4 == 0 && ldx % 4 == 0 && ((((uintptr_t)x) | ((uintptr_t)mu) | ((uintptr_t)out) | ((uintptr_t)prev_state)) & 15) == 0;
  const int per_block = vec ? 512 : 128;       // columns one block covers per pass
  const dim3 grid(B, max(1, min(max_q, 1024)), max_q < 8 ? max(1, min((W + per_block - 1) / per_block, 32)) : 1);
  if (vec)
    LLMSS_BY_DTYPE(dtype, (token_shift_kernel<T, 4><<<grid, 128, 0, stream>>>(x, ldx, mu, S, (T*)out, (int64_t)T_, W, cu_q, seq_lens, slots,
                                                                              prev_state)));
  else
    LLMSS_BY_DTYPE(dtype, (token_shift_kernel<T, 1><<<grid, 128, 0, stream>>>(x, ldx, mu, S, (T*)out, (int64_t)T_, W, cu_q, seq_lens, slots,
                                                                              prev_state)));
  LLMSS_CHECK_CUDA(cudaGetLastError());
  return 0;
}

template <typename TO>
static int causal_conv_launch(const float* u, int64_t ldu, const float* w, const float* bias, TO* out, int T_, int C, int taps,
                              int act, const int* cu_q, const int* seq_lens, const int* slots, int B, int max_q, float* state,
                              cudaStream_t stream) {
  const int chunks = max(1, min((max_q + kConvChunk - 1) / kConvChunk, 64));
  if (taps <= 4 && C % 4 == 0 && ldu % 4 == 0 &&
      ((((uintptr_t)u) | ((uintptr_t)out) | ((uintptr_t)bias) | ((uintptr_t)state)) & 15) == 0) {
    // (a null bias or state is aligned; the state's rows are C floats apart)
    const dim3 grid4(B, (C / 4 + 127) / 128, max(1, min((max_q + 15) / 16, 128)));
    causal_conv4_kernel<4, 16, TO><<<grid4, 128, 0, stream>>>(u, ldu, w, bias, out, C, taps, act, cu_q, seq_lens, slots, state);
    LLMSS_CHECK_CUDA(cudaGetLastError());
    return 0;
  }
  const dim3 grid(B, (C + 127) / 128, chunks);
  if (taps <= 4) causal_conv_kernel<4, TO><<<grid, 128, 0, stream>>>(u, ldu, w, bias, out, C, taps, act, cu_q, seq_lens, slots, state);
  else if (taps <= 8) causal_conv_kernel<8, TO><<<grid, 128, 0, stream>>>(u, ldu, w, bias, out, C, taps, act, cu_q, seq_lens, slots, state);
  else causal_conv_kernel<16, TO><<<grid, 128, 0, stream>>>(u, ldu, w, bias, out, C, taps, act, cu_q, seq_lens, slots, state);
  LLMSS_CHECK_CUDA(cudaGetLastError());
  return 0;
}

// out: [T, C] in out_dtype (32-bit, or the 16-bit type of the GEMM that reads it); the arithmetic and the tails are 32-bit
LLMSS_API int llmss_causal_conv_to(const float* u, int64_t ldu, const float* w, const float* bias, void* out, int out_dtype, int T_,
                                   int C, int taps, int act, const int* cu_q, const int* seq_lens, const int* slots, int B, int max_q,
                                   float* state, cudaStream_t stream) {
  LLMSS_REQUIRE(taps >= 1 && taps <= kMaxTapsAny, "causal_conv: %d taps (1..%d)", taps, kMaxTapsAny);
  LLMSS_REQUIRE(taps == 1 || state != nullptr, "causal_conv: more than one tap needs a state");
  if (B <= 0 || T_ <= 0) return 0;
  LLMSS_BY_DTYPE(out_dtype, return (causal_conv_launch<T>(u, ldu, w, bias, (T*)out, T_, C, taps, act, cu_q, seq_lens, slots, B, max_q,
                                                           state, stream)));
}

LLMSS_API int llmss_causal_conv(const float* u, int64_t ldu, const float* w, const float* bias, float* out, int T_, int C, int taps,
                                int act, const int* cu_q, const int* seq_lens, const int* slots, int B, int max_q, float* state,
                                cudaStream_t stream) {
  return llmss_causal_conv_to(u, ldu, w, bias, out, LLMSS_F32, T_, C, taps, act, cu_q, seq_lens, slots, B, max_q, state, stream);
}

LLMSS_API int llmss_unary_f32(const float* x, int64_t ldx, void* out, int rows, int cols, int op, int out_dtype, cudaStream_t stream) {
  const int64_t n = (int64_t)rows * cols;
  if (n <= 0) return 0;
  LLMSS_BY_DTYPE(out_dtype, (unary_kernel<T><<<grid_for(n), 256, 0, stream>>>(x, ldx, (T*)out, n, cols, op)));
  LLMSS_CHECK_CUDA(cudaGetLastError());
  return 0;
}

LLMSS_API int llmss_ssm_dt(const float* raw, int64_t ldr, const float* dt_bias, const float* a_log, float* dt, float* logdecay,
                           int T_, int H, cudaStream_t stream) {
  const int64_t n = (int64_t)T_ * H;
  if (n <= 0) return 0;
  ssm_dt_kernel<<<grid_for(n), 256, 0, stream>>>(raw, ldr, dt_bias, a_log, dt, logdecay, n, H);
  LLMSS_CHECK_CUDA(cudaGetLastError());
  return 0;
}

LLMSS_API int64_t llmss_linear_scan_scratch_floats(int B, int heads, int dk, int dv, int max_q, int chunk) {
  const int nch = chunk > 0 ? (max_q + chunk - 1) / chunk : 0;
  return (int64_t)B * heads * ((int64_t)dv * dk + (int64_t)nch * ((int64_t)dv * dk + dk));
}

// chunk > 0 (and scratch of llmss_linear_scan_scratch_floats floats): two passes over chunks of that many tokens (a
// multiple of 16) -- for prompt rounds whose sequences are long and few; chunk = 0: one pass.
LLMSS_API int llmss_linear_scan(const float* q, int64_t ldq, const float* k, int64_t ldk, const float* v, int64_t ldv,
                                const float* decay, int64_t ldd, int decay_kind, const float* bonus, const float* vscale,
                                int64_t ldvs, float* out, float* state, const int* cu_q, const int* seq_lens, const int* slots,
                                int B, int heads, int qk_heads, int dk, int dv, int read_before, float* scratch, int chunk,
                                int max_q, cudaStream_t stream) {
  LLMSS_REQUIRE(heads > 0 && qk_heads > 0 && heads % qk_heads == 0, "linear_scan: %d heads over %d q/k heads", heads, qk_heads);
  LLMSS_REQUIRE(dk > 0 && dk <= 1024, "linear_scan: key size %d (at most 1024)", dk);
  LLMSS_REQUIRE(decay_kind >= 0 && decay_kind <= 2, "linear_scan: decay kind %d", decay_kind);
  LLMSS_REQUIRE(chunk == 0 || (chunk % TCH == 0 && scratch != nullptr && max_q > 0), "linear_scan: bad chunking (%d tokens)", chunk);
  if (B <= 0) return 0;
  ScanArgs a;
  a.q = q; a.ldq = ldq; a.k = k; a.ldk = ldk; a.v = v; a.ldv = ldv; a.decay = decay; a.ldd = ldd; a.bonus = bonus;
  a.vscale = vscale; a.ldvs = ldvs; a.out = out; a.state = state; a.cu_q = cu_q; a.seq_lens = seq_lens; a.slots = slots;
  a.H = heads; a.rep = heads / qk_heads; a.dk = dk; a.dv = dv;
  a.chunk = chunk;
  a.nch = chunk > 0 ? (max_q + chunk - 1) / chunk : 1;
  a.old_copy = scratch;
  a.chunk_state = scratch != nullptr ? scratch + (int64_t)B * heads * dv * dk : nullptr;
  a.chunk_decay = scratch != nullptr ? a.chunk_state + (int64_t)B * a.nch * heads * dv * dk : nullptr;
  if (dk > 32 && dk <= 128) {
    // 8 x 8 register tiles: RG row groups of 8 key rows, value columns in groups of 8
    const int rg = dk <= 64 ? 8 : 16;
    a.R = rg;
    a.dvt = min((dv + 7) / 8 * 8, 8 * (128 / rg));
    while ((int64_t)B * heads * a.nch * ((dv + a.dvt - 1) / a.dvt) < 4 * 148 && a.dvt > 8 && (a.dvt / 2) % 8 == 0 && (a.dvt / 16) * rg >= 32) a.dvt /= 2;
    a.nslices = (dv + a.dvt - 1) / a.dvt;
    const int threads = (a.dvt / 8) * rg;
    const int row = rg * TSTR;
    const size_t smem = sizeof(float) * ((size_t)TCH * row * 2 + (decay_kind == 2 ? (size_t)TCH * row : TCH) +
                                         (read_before ? (size_t)TCH * row : 0) + (size_t)TCH * a.dvt);
    const dim3 grid(B, heads, a.nslices * (chunk > 0 ? a.nch : 1));
    LLMSS_REQUIRE(grid.y <= 65535 && grid.z <= 65535, "linear_scan: grid too large");
#define LLMSS_TILE2(RB, KIND, MODE, RG_)                                                       \
  do {                                                                                         \
    static PerDeviceSmem g;                                                                    \
    LLMSS_CHECK_CUDA(g.ensure(linear_scan_tile_kernel<RB, KIND, MODE, RG_>, (int)smem));       \
    linear_scan_tile_kernel<RB, KIND, MODE, RG_><<<grid, threads, smem, stream>>>(a);          \
  } while (0)
#define LLMSS_TILE1(RB, KIND, MODE)                                                            \
  do {                                                                                         \
    if (rg == 8) LLMSS_TILE2(RB, KIND, MODE, 8); else LLMSS_TILE2(RB, KIND, MODE, 16);         \
  } while (0)
#define LLMSS_TILE(RB, KIND)                                                                   \
  do {                                                                                         \
    if (chunk > 0) { LLMSS_TILE1(RB, KIND, 1); LLMSS_TILE1(RB, KIND, 2); }                     \
    else LLMSS_TILE1(RB, KIND, 0);                                                             \
  } while (0)
    if (read_before) {
      if (decay_kind == 0) LLMSS_TILE(true, 0); else if (decay_kind == 1) LLMSS_TILE(true, 1); else LLMSS_TILE(true, 2);
    } else {
      if (decay_kind == 0) LLMSS_TILE(false, 0); else if (decay_kind == 1) LLMSS_TILE(false, 1); else LLMSS_TILE(false, 2);
    }
#undef LLMSS_TILE
#undef LLMSS_TILE1
#undef LLMSS_TILE2
    LLMSS_CHECK_CUDA(cudaGetLastError());
    return 0;
  }
  const int kpt = dk >= 48 ? 64 : 16;           // key rows per thread
  a.R = pow2_at_least((dk + kpt - 1) / kpt);
  a.dvt = min(dv, (kpt == 64 ? 128 : SCAN_THREADS) / a.R);
  a.chunk = chunk;
  a.nch = chunk > 0 ? (max_q + chunk - 1) / chunk : 1;
  // few blocks (a prompt round of few sequences): narrower value slices until the grid covers the SMs a few times over
  while ((int64_t)B * heads * a.nch * ((dv + a.dvt - 1) / a.dvt) < 4 * 148 && a.dvt * a.R > 32 && a.dvt > 4) a.dvt = (a.dvt + 1) / 2;
  a.nslices = (dv + a.dvt - 1) / a.dvt;
  a.old_copy = scratch;
  a.chunk_state = scratch != nullptr ? scratch + (int64_t)B * heads * dv * dk : nullptr;
  a.chunk_decay = scratch != nullptr ? a.chunk_state + (int64_t)B * a.nch * heads * dv * dk : nullptr;
  const int threads = ((a.dvt * a.R + 31) / 32) * 32;
  const int row = a.R * (kpt + 4);
  const size_t smem = sizeof(float) * ((size_t)TCH * row * 2 + (decay_kind == 2 ? (size_t)TCH * row : TCH) +
                                       (read_before ? (size_t)TCH * row : 0) + (size_t)TCH * a.dvt);
  const dim3 grid(B, heads, a.nslices * (chunk > 0 ? a.nch : 1));
  LLMSS_REQUIRE(grid.y <= 65535 && grid.z <= 65535, "linear_scan: grid too large");
#define LLMSS_SCAN2(RB, KIND, MODE, KP)                                                        \
  do {                                                                                         \
    static PerDeviceSmem g;                                                                    \
    LLMSS_CHECK_CUDA(g.ensure(linear_scan_kernel<RB, KIND, MODE, KP>, (int)smem));             \
    linear_scan_kernel<RB, KIND, MODE, KP><<<grid, threads, smem, stream>>>(a);                \
  } while (0)
#define LLMSS_SCAN1(RB, KIND, MODE)                                                            \
  do {                                                                                         \
    if (kpt == 64) LLMSS_SCAN2(RB, KIND, MODE, 64); else LLMSS_SCAN2(RB, KIND, MODE, 16);      \
  } while (0)
#define LLMSS_SCAN(RB, KIND)                                                                   \
  do {                                                                                         \
    if (chunk > 0) { LLMSS_SCAN1(RB, KIND, 1); LLMSS_SCAN1(RB, KIND, 2); }                     \
    else LLMSS_SCAN1(RB, KIND, 0);                                                             \
  } while (0)
  if (read_before) {
    if (decay_kind == 0) LLMSS_SCAN(true, 0); else if (decay_kind == 1) LLMSS_SCAN(true, 1); else LLMSS_SCAN(true, 2);
  } else {
    if (decay_kind == 0) LLMSS_SCAN(false, 0); else if (decay_kind == 1) LLMSS_SCAN(false, 1); else LLMSS_SCAN(false, 2);
  }
#undef LLMSS_SCAN
#undef LLMSS_SCAN1
#undef LLMSS_SCAN2
  LLMSS_CHECK_CUDA(cudaGetLastError());
  return 0;
}

LLMSS_API int llmss_gated_rmsnorm(const float* o, int64_t ldo, const float* gate, int64_t ldg, int gate_act, const float* weight,
                                  int groups, float eps, int gate_first, const float* skip_x, int64_t ldx, const float* skip_d,
                                  int H, void* out, int T_, int C, int dtype, cudaStream_t stream) {
  LLMSS_REQUIRE(groups > 0 && C % groups == 0, "gated_rmsnorm: %d channels in %d groups", C, groups);
  LLMSS_REQUIRE(skip_x == nullptr || (skip_d != nullptr && H > 0 && C % H == 0), "gated_rmsnorm: skip needs one factor per head");
  if (T_ <= 0) return 0;
  GnArgs a;
  a.o = o; a.ldo = ldo; a.gate = gate; a.ldg = ldg; a.weight = weight; a.skip_x = skip_x; a.ldx = ldx; a.skip_d = skip_d;
  a.C = C; a.groups = groups; a.H = H > 0 ? H : 1; a.gate_act = gate_act; a.gate_first = gate_first; a.eps = eps;
  LLMSS_BY_DTYPE(dtype, (gated_rmsnorm_kernel<T><<<T_, 256, 0, stream>>>(a, (T*)out)));
  LLMSS_CHECK_CUDA(cudaGetLastError());
  return 0;
}

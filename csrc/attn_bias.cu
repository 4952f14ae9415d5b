// Grouped-query softmax attention with separate key / value sizes, per-head query / key norm, a query temperature and a
// learned distance bias, over the paged cache -- the generic (any head size, 16- or 32-bit) form.
//
//   qknorm_kv_write : per token and head, rms_div(q) * q_w (times the query temperature 1 + coef * ln(floor((p + 1) /
//                     every) + 1)) -> queries in the compute type; rms_div(k) * k_w -> key page; v -> value page.  The
//                     counterpart of rope_kv_write for a design whose positions enter through distances, not rotations.
//   attention_bias  : out_ih = gate_ih * sum_j softmax_j(scale * q_ih . k_jg + bias[h][min(i - j, last)]) v_jg ,  j <= i.
//                     One CTA = one sequence x one key/value head x up to 8 (query row, query head of the group) pairs;
//                     its warps share every 32-key tile of K and V, staged once in shared memory in 32-bit.  A warp owns
//                     one pair: lane = key inside the tile for the scores, lane = output channel (mod 32) for P V.
//                     Scores, softmax and accumulation are 32-bit with full-precision exponentials.
//                     Optional: a linear penalty slopes[h] * (i - j) taken off the scores, and a sliding window (keys with
//                     i - j >= window are hidden; the key loop starts at the first row's window).
//   qkv_prepare     : the general form of qknorm_kv_write, one CTA per token: query / key norm per head or over the token's
//                     whole projection, a factor per query head, values divided by their per-head root mean square, queries
//                     only (no keys / values) for a layer that attends over another layer's pages.
// Page layouts: keys [num_blocks, kv_heads, block_size, dk], values [num_blocks, kv_heads, block_size, dv].
#include "common.cuh"

namespace {

constexpr int NW = 8, TK = 32, MAXV = 8;   // warps per CTA, keys per tile, output channels per lane (dv <= 256)

template <typename T>
__global__ void __launch_bounds__(256) qknorm_kv_write_kernel(const float* __restrict__ qkv, int64_t ld, int hq, int hkv, int dk,
                                                              int dv, const float* __restrict__ q_w, const float* __restrict__ k_w,
                                                              float eps, float coef, int every, const int* __restrict__ positions,
                                                              const int* __restrict__ slots, T* __restrict__ k_cache,
                                                              T* __restrict__ v_cache, int bs, T* __restrict__ q_out, int T_) {
  const int nh = hq + 2 * hkv;
  const int64_t unit = (int64_t)blockIdx.x * NW + (threadIdx.x >> 5);
  if (unit >= (int64_t)T_ * nh) return;
  const int64_t t = unit / nh;
  const int h = (int)(unit % nh), lane = threadIdx.x & 31;
  const float* row = qkv + t * ld;
  const int slot = slots[t];
  if (h < hq + hkv) {
    const float* x = row + (int64_t)h * dk;
    float ss = 0.f;
    for (int c = lane; c < dk; c += 32) ss = fmaf(x[c], x[c], ss);
    float r = rsqrtf(warp_sum(ss) / dk + eps);
    if (h < hq) {
      if (coef != 0.f) r *= 1.f + coef * logf((float)((positions[t] + 1) / every) + 1.f);
      for (int c = lane; c < dk; c += 32) q_out[t * hq * dk + (int64_t)h * dk + c] = from_f32<T>(x[c] * r * q_w[c]);
    } else if (slot >= 0) {
      T* dst = k_cache + (((int64_t)(slot / bs) * hkv + (h - hq)) * bs + slot % bs) * dk;
      for (int c = lane; c < dk; c += 32) dst[c] = from_f32<T>(x[c] * r * k_w[c]);
    }
  } else if (slot >= 0) {
    const int g = h - hq - hkv;
    const float* x = row + (int64_t)(hq + hkv) * dk + (int64_t)g * dv;
    T* dst = v_cache + (((int64_t)(slot / bs) * hkv + g) * bs + slot % bs) * dv;
    for (int c = lane; c < dv; c += 32) dst[c] = from_f32<T>(x[c]);
  }
}

// x[t, h * dv + c] *= sigmoid(gate[t, h]) in place: the output gate behind an attention kernel that has no gate of its own
template <typename T>
__global__ void __launch_bounds__(256) head_gate_kernel(T* __restrict__ x, int64_t ldx, const float* __restrict__ gate, int64_t ldg,
                                                        int hq, int dv) {
  const int64_t t = blockIdx.x;
  for (int c = threadIdx.x; c < hq * dv; c += 256) {
    const float g = 1.f / (1.f + expf(-gate[t * ldg + c / dv]));
    x[t * ldx + c] = from_f32<T>(to_f32(x[t * ldx + c]) * g);
  }
}

// One CTA per token.  Pass 1: the sum of squares of every head (queries, keys, values), a warp per head; pass 2: the norms
// (a head's own sum, or the sum over all query / all key heads of the token) and the writes.  whole = 1: q_w / k_w have the
// size of the whole projection; else one weight of size dk shared by the heads.
template <typename T>
__global__ void __launch_bounds__(256) qkv_prepare_kernel(const float* __restrict__ qkv, int64_t ld, int hq, int hkv, int dk, int dv,
                                                          const float* __restrict__ q_w, const float* __restrict__ k_w, float eps,
                                                          float coef, int every, const float* __restrict__ q_head_scale, int whole,
                                                          int v_norm, const int* __restrict__ positions, const int* __restrict__ slots,
                                                          T* __restrict__ k_cache, T* __restrict__ v_cache, int bs, T* __restrict__ q_out) {
  extern __shared__ float hsum[];     // [hq + 2 hkv] sums of squares, then [2] the whole-projection factors
  const int64_t t = blockIdx.x;
  const int nh = hq + 2 * hkv, lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
  const float* row = qkv + t * ld;
  const int slot = hkv > 0 ? slots[t] : -1;
  for (int h = warp; h < nh; h += nw) {
    const bool isv = h >= hq + hkv;
    const float* x = isv ? row + (int64_t)(hq + hkv) * dk + (int64_t)(h - hq - hkv) * dv : row + (int64_t)h * dk;
    const int n = isv ? dv : dk;
    float ss = 0.f;
    for (int c = lane; c < n; c += 32) ss = fmaf(x[c], x[c], ss);
    ss = warp_sum(ss);
    if (lane == 0) hsum[h] = ss;
  }
  __syncthreads();
  if (whole && threadIdx.x < 2) {
    const int lo = threadIdx.x == 0 ? 0 : hq, n = threadIdx.x == 0 ? hq : hkv;
    float tot = 0.f;
    for (int h = 0; h < n; ++h) tot += hsum[lo + h];
    hsum[nh + threadIdx.x] = n > 0 ? rsqrtf(tot / ((float)n * dk) + eps) : 0.f;
  }
  __syncthreads();
  float temp = 1.f;
  if (coef != 0.f) temp = 1.f + coef * logf((float)((positions[t] + 1) / every) + 1.f);
  for (int h = warp; h < nh; h += nw) {
    if (h < hq) {
      float r = whole ? hsum[nh] : rsqrtf(hsum[h] / dk + eps);
      r *= temp;
      if (q_head_scale != nullptr) r *= q_head_scale[h];
      const float* x = row + (int64_t)h * dk;
      const float* w = q_w + (whole ? (int64_t)h * dk : 0);
      for (int c = lane; c < dk; c += 32) q_out[t * hq * dk + (int64_t)h * dk + c] = from_f32<T>(x[c] * r * w[c]);
    } else if (slot >= 0 && h < hq + hkv) {
      const int g = h - hq;
      const float r = whole ? hsum[nh + 1] : rsqrtf(hsum[h] / dk + eps);
      const float* x = row + (int64_t)h * dk;
      const float* w = k_w + (whole ? (int64_t)g * dk : 0);
      T* dst = k_cache + (((int64_t)(slot / bs) * hkv + g) * bs + slot % bs) * dk;
      for (int c = lane; c < dk; c += 32) dst[c] = from_f32<T>(x[c] * r * w[c]);
    } else if (slot >= 0) {
      const int g = h - hq - hkv;
      const float r = v_norm ? rsqrtf(hsum[h] / dv + eps) : 1.f;
      const float* x = row + (int64_t)(hq + hkv) * dk + (int64_t)g * dv;
      T* dst = v_cache + (((int64_t)(slot / bs) * hkv + g) * bs + slot % bs) * dv;
      for (int c = lane; c < dv; c += 32) dst[c] = from_f32<T>(x[c] * r);
    }
  }
}

struct AbArgs {
  const void* q; int64_t ldq;
  const void* k_cache; const void* v_cache;
  const int* block_tables; int max_blocks, bs;
  const int* seq_lens; const int* cu_q;
  const float* bias; int n_dist;          // [hq][n_dist]
  const float* slopes;                    // [hq] linear distance penalty, or null
  int window;                             // > 0: only keys with i - j < window are visible
  const float* gate; int64_t ldg;         // [T][hq] logits, or null
  const float* sinks;                     // [hq] sink logits (one more term exp(sinks[h]) in every denominator), or null
  void* out;                              // [T][hq * dv]
  int hq, hkv, dk, dv, nh, rows, hsub;    // nh: query heads per CTA; rows: query rows per CTA; hsub: CTAs per kv head
  float scale;
};

template <typename T>
__global__ void __launch_bounds__(NW * 32) attention_bias_kernel(AbArgs a) {
  extern __shared__ float sm[];
  const int b = blockIdx.z;
  const int q0 = a.cu_q[b], ql = a.cu_q[b + 1] - q0, L = a.seq_lens[b];
  const int r0 = blockIdx.x * a.rows;
  if (r0 >= ql || L <= 0) return;
  const int g = blockIdx.y / a.hsub, hs = blockIdx.y % a.hsub;
  const int gsz = a.hq / a.hkv;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int dk = a.dk, dv = a.dv, dkp = dk + 1;
  float* qs = sm;                      // [NW][dk]
  float* ks = qs + NW * dk;            // [TK][dk + 1]
  float* vs = ks + TK * dkp;           // [TK][dv]
  // this warp's (row, head)
  const int hl = warp % a.nh, rl = warp / a.nh;
  const int hin = hs * NW + hl;                 // head inside the group
  const int row = r0 + rl;
  const bool active = rl < a.rows && row < ql && hin < gsz;
  const int h = g * gsz + hin;
  const int ctx = L - ql;
  const int qpos = ctx + row;                   // absolute position of the query
  const T* qg = reinterpret_cast<const T*>(a.q);
  if (active)
    for (int c = lane; c < dk; c += 32) qs[warp * dk + c] = to_f32(qg[(int64_t)(q0 + row) * a.ldq + (int64_t)h * dk + c]) * a.scale;
  const int last_row = min(ql, r0 + a.rows) - 1;
  const int kend = ctx + last_row + 1;          // keys 0 .. kend - 1 are visible to some row of this CTA
  float m = -INFINITY, l = 0.f, acc[MAXV];
#pragma unroll
  for (int i = 0; i < MAXV; ++i) acc[i] = 0.f;
  const T* kc = reinterpret_cast<const T*>(a.k_cache);
  const T* vc = reinterpret_cast<const T*>(a.v_cache);
  const float* brow = a.bias != nullptr ? a.bias + (int64_t)(active ? h : 0) * a.n_dist : nullptr;
  const float slope = a.slopes != nullptr && active ? a.slopes[h] : 0.f;
  const int kbeg = a.window > 0 ? max(0, ctx + r0 - a.window + 1) : 0;      // first key any row of this CTA sees
  const int klo = a.window > 0 ? qpos - a.window + 1 : 0;                   // first key this warp's row sees
  for (int k0 = kbeg; k0 < kend; k0 += TK) {
    const int nk = min(TK, kend - k0);
    __syncthreads();
    for (int idx = threadIdx.x; idx < nk * dk; idx += NW * 32) {
      const int kk = idx / dk, c = idx % dk, pos = k0 + kk;
      const int blk = a.block_tables[(int64_t)b * a.max_blocks + pos / a.bs];
      ks[kk * dkp + c] = to_f32(kc[(((int64_t)blk * a.hkv + g) * a.bs + pos % a.bs) * dk + c]);
    }
    for (int idx = threadIdx.x; idx < nk * dv; idx += NW * 32) {
      const int kk = idx / dv, c = idx % dv, pos = k0 + kk;
      const int blk = a.block_tables[(int64_t)b * a.max_blocks + pos / a.bs];
      vs[kk * dv + c] = to_f32(vc[(((int64_t)blk * a.hkv + g) * a.bs + pos % a.bs) * dv + c]);
    }
    __syncthreads();
    if (!active || k0 > qpos || k0 + nk <= klo) continue;
    const int kpos = k0 + lane;
    float sc = -INFINITY;
    if (lane < nk && kpos <= qpos && kpos >= klo) {
      float d = 0.f;
      const float* kr = ks + lane * dkp;
      const float* qr = qs + warp * dk;
      for (int c = 0; c < dk; ++c) d = fmaf(qr[c], kr[c], d);
      sc = d;
      if (brow != nullptr) sc += brow[min(qpos - kpos, a.n_dist - 1)];
      sc -= slope * (float)(qpos - kpos);
    }
    const float mt = warp_max(sc);
    if (mt == -INFINITY) continue;               // nothing of this tile is visible to the row (warp-uniform)
    const float mn = fmaxf(m, mt);
    const float corr = expf(m - mn);            // m = -inf on the first tile: 0
    const float p = sc == -INFINITY ? 0.f : expf(sc - mn);
    l = l * corr + warp_sum(p);
    m = mn;
#pragma unroll
    for (int i = 0; i < MAXV; ++i) acc[i] *= corr;
    for (int kk = 0; kk < nk; ++kk) {
      const float pk = __shfl_sync(0xffffffffu, p, kk);
      if (pk == 0.f) continue;
#pragma unroll
      for (int i = 0; i < MAXV; ++i) {
        const int c = lane + 32 * i;
        if (c < dv) acc[i] = fmaf(pk, vs[kk * dv + c], acc[i]);
      }
    }
  }
  if (!active) return;
  float gsc = 1.f / l;
  if (a.sinks != nullptr) {       // the sink is a logit only: it enlarges the denominator and adds nothing to the numerator
    const float sk = a.sinks[h];
    const float mn = fmaxf(m, sk);
    const float corr = expf(m - mn);
    gsc = corr / (l * corr + expf(sk - mn));
  }
  if (a.gate != nullptr) gsc *= 1.f / (1.f + expf(-a.gate[(int64_t)(q0 + row) * a.ldg + h]));
  T* og = reinterpret_cast<T*>(a.out) + (int64_t)(q0 + row) * a.hq * dv + (int64_t)h * dv;
#pragma unroll
  for (int i = 0; i < MAXV; ++i) {
    const int c = lane + 32 * i;
    if (c < dv) og[c] = from_f32<T>(acc[i] * gsc);
  }
}

}  // namespace

LLMSS_API int llmss_qknorm_kv_write(const float* qkv, int64_t ld, int hq, int hkv, int dk, int dv, const float* q_w, const float* k_w,
                                    float eps, float temp_coef, int temp_every, const int* positions, const int* slots,
                                    void* k_cache, void* v_cache, int block_size, void* q_out, int T_, int dtype,
                                    cudaStream_t stream) {
  LLMSS_REQUIRE(hq > 0 && hkv > 0 && temp_every > 0, "qknorm_kv_write: bad sizes");
  if (T_ <= 0) return 0;
  const int64_t units = (int64_t)T_ * (hq + 2 * hkv);
  LLMSS_BY_DTYPE(dtype, (qknorm_kv_write_kernel<T><<<(unsigned)((units + NW - 1) / NW), NW * 32, 0, stream>>>(
                            qkv, ld, hq, hkv, dk, dv, q_w, k_w, eps, temp_coef, temp_every, positions, slots, (T*)k_cache, (T*)v_cache,
                            block_size, (T*)q_out, T_)));
  LLMSS_CHECK_CUDA(cudaGetLastError());
  return 0;
}

// General form of llmss_qknorm_kv_write: norm per head (whole = 0, weights [dk]) or over the token's whole q / k projection
// (whole = 1, weights [hq * dk] / [hkv * dk]); q_head_scale [hq] or null; v_norm = 1: values / their per-head rms; hkv = 0:
// queries only (k_cache / v_cache / slots unused).
LLMSS_API int llmss_qkv_prepare(const float* qkv, int64_t ld, int hq, int hkv, int dk, int dv, const float* q_w, const float* k_w,
                                float eps, float temp_coef, int temp_every, const float* q_head_scale, int whole, int v_norm,
                                const int* positions, const int* slots, void* k_cache, void* v_cache, int block_size, void* q_out,
                                int T_, int dtype, cudaStream_t stream) {
  LLMSS_REQUIRE(hq > 0 && hkv >= 0 && temp_every > 0, "qkv_prepare: bad sizes");
  LLMSS_REQUIRE(hkv == 0 || (k_cache != nullptr && v_cache != nullptr && slots != nullptr && k_w != nullptr), "qkv_prepare: keys without pages");
  if (T_ <= 0) return 0;
  const size_t smem = sizeof(float) * (size_t)(hq + 2 * hkv + 2);
  LLMSS_REQUIRE(smem <= 48 * 1024, "qkv_prepare: too many heads");
  const int nh = hq + 2 * hkv;
  const int threads = nh >= 8 ? 256 : (nh >= 4 ? 128 : 64);
  LLMSS_BY_DTYPE(dtype, (qkv_prepare_kernel<T><<<T_, threads, smem, stream>>>(qkv, ld, hq, hkv, dk, dv, q_w, k_w, eps, temp_coef, temp_every,
                                                                             q_head_scale, whole, v_norm, positions, slots, (T*)k_cache,
                                                                             (T*)v_cache, block_size, (T*)q_out)));
  LLMSS_CHECK_CUDA(cudaGetLastError());
  return 0;
}

LLMSS_API int llmss_head_gate(void* x, int64_t ldx, const float* gate, int64_t ldg, int T_, int hq, int dv, int dtype,
                              cudaStream_t stream) {
  if (T_ <= 0) return 0;
  LLMSS_BY_DTYPE(dtype, (head_gate_kernel<T><<<T_, 256, 0, stream>>>((T*)x, ldx, gate, ldg, hq, dv)));
  LLMSS_CHECK_CUDA(cudaGetLastError());
  return 0;
}

static int attention_bias_launch(const void* q, int64_t ldq, const void* k_cache, const void* v_cache, const int* block_tables,
                                 int max_blocks, int block_size, const int* seq_lens, const int* cu_q, const float* bias,
                                 int n_dist, const float* slopes, int window, const float* gate, int64_t ldg, void* out, int B,
                                 int max_q, int hq, int hkv, int dk, int dv, float scale, int dtype, cudaStream_t stream,
                                 const float* sinks = nullptr) {
  LLMSS_REQUIRE(hq > 0 && hkv > 0 && hq % hkv == 0, "attention_bias: %d query heads over %d key/value heads", hq, hkv);
  LLMSS_REQUIRE(dv <= 32 * MAXV, "attention_bias: value size %d (at most %d)", dv, 32 * MAXV);
  LLMSS_REQUIRE(bias == nullptr || n_dist > 0, "attention_bias: empty bias table");
  if (B <= 0 || max_q <= 0) return 0;
  AbArgs a;
  a.q = q; a.ldq = ldq; a.k_cache = k_cache; a.v_cache = v_cache; a.block_tables = block_tables; a.max_blocks = max_blocks;
  a.bs = block_size; a.seq_lens = seq_lens; a.cu_q = cu_q; a.bias = bias; a.n_dist = n_dist; a.slopes = slopes; a.window = window; a.gate = gate; a.ldg = ldg; a.out = out;
  a.sinks = sinks;
  a.hq = hq; a.hkv = hkv; a.dk = dk; a.dv = dv; a.scale = scale;
  const int gsz = hq / hkv;
  a.nh = gsz < NW ? gsz : NW;
  a.rows = NW / a.nh;
  a.hsub = (gsz + NW - 1) / NW;
  const size_t smem = sizeof(float) * ((size_t)NW * dk + (size_t)TK * (dk + 1) + (size_t)TK * dv);
  LLMSS_REQUIRE(smem <= 200 * 1024, "attention_bias: key size %d / value size %d exceed shared memory", dk, dv);
  const dim3 grid((max_q + a.rows - 1) / a.rows, hkv * a.hsub, B);
  LLMSS_REQUIRE(grid.y <= 65535 && grid.z <= 65535, "attention_bias: grid too large");
#define LLMSS_AB(TT)                                                                \
  do {                                                                              \
    static PerDeviceSmem gsm;                                                       \
    LLMSS_CHECK_CUDA(gsm.ensure(attention_bias_kernel<TT>, (int)smem));             \
    attention_bias_kernel<TT><<<grid, NW * 32, smem, stream>>>(a);                  \
  } while (0)
  if (dtype == LLMSS_F16) LLMSS_AB(__half);
  else if (dtype == LLMSS_BF16) LLMSS_AB(__nv_bfloat16);
  else if (dtype == LLMSS_F32) LLMSS_AB(float);
  else LLMSS_REQUIRE(false, "bad dtype %d", dtype);
#undef LLMSS_AB
  LLMSS_CHECK_CUDA(cudaGetLastError());
  return 0;
}

LLMSS_API int llmss_attention_bias(const void* q, int64_t ldq, const void* k_cache, const void* v_cache, const int* block_tables,
                                   int max_blocks, int block_size, const int* seq_lens, const int* cu_q, const float* bias,
                                   int n_dist, const float* gate, int64_t ldg, void* out, int B, int max_q, int hq, int hkv, int dk,
                                   int dv, float scale, int dtype, cudaStream_t stream) {
  return attention_bias_launch(q, ldq, k_cache, v_cache, block_tables, max_blocks, block_size, seq_lens, cu_q, bias, n_dist, nullptr, 0,
                               gate, ldg, out, B, max_q, hq, hkv, dk, dv, scale, dtype, stream);
}

// the same with a linear distance penalty per head (slopes [hq] or null) and a sliding window (window > 0)
LLMSS_API int llmss_attention_window(const void* q, int64_t ldq, const void* k_cache, const void* v_cache, const int* block_tables,
                                     int max_blocks, int block_size, const int* seq_lens, const int* cu_q, const float* bias,
                                     int n_dist, const float* slopes, int window, const float* gate, int64_t ldg, void* out, int B,
                                     int max_q, int hq, int hkv, int dk, int dv, float scale, int dtype, cudaStream_t stream) {
  LLMSS_REQUIRE(window >= 0, "attention_window: window %d", window);
  return attention_bias_launch(q, ldq, k_cache, v_cache, block_tables, max_blocks, block_size, seq_lens, cu_q, bias, n_dist, slopes,
                               window, gate, ldg, out, B, max_q, hq, hkv, dk, dv, scale, dtype, stream);
}

// the same with an attention sink per head (sinks [hq] or null): exp(sinks[h]) joins every softmax denominator of head h
LLMSS_API int llmss_attention_sink(const void* q, int64_t ldq, const void* k_cache, const void* v_cache, const int* block_tables,
                                   int max_blocks, int block_size, const int* seq_lens, const int* cu_q, const float* bias,
                                   int n_dist, const float* slopes, int window, const float* gate, int64_t ldg, const float* sinks,
                                   void* out, int B, int max_q, int hq, int hkv, int dk, int dv, float scale, int dtype,
                                   cudaStream_t stream) {
  LLMSS_REQUIRE(window >= 0, "attention_sink: window %d", window);
  return attention_bias_launch(q, ldq, k_cache, v_cache, block_tables, max_blocks, block_size, seq_lens, cu_q, bias, n_dist, slopes,
                               window, gate, ldg, out, B, max_q, hq, hkv, dk, dv, scale, dtype, stream, sinks);
}

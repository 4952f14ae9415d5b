// Strided batched GEMM on the CUDA cores, fp32 accumulation, any shape and alignment.
//
//   out(t, h, n) = epilogue( sum_k x(t, h, k) * w(h, k, n) )      t < M, h < H, n < N, k < K
//   x(t, h, k)   = x  [t * ldx + h * sxh + k]
//   w(h, k, n)   = w  [h * swh + k * swk + n * swn]
//   out(t, h, n) = out[t * ldo + h * soh + n]
//
// Three users:
//   * true 32-bit linear layers (T = float; the tcgen05 GEMM takes 16-bit operands only), and 16-bit linear
//     layers whose K or base address misses the 16-byte rule of the TMA path: H = 1, swk = 1, swn = ldw;
//   * the per-head products of latent attention: q_h -> W_uk,h^T q_h (swk = rank, swn = 1) and
//     o_h -> W_uv,h o_h (swk = 1, swn = rank), optionally scaled per (token, head) by an output gate.
// 64 x 64 output tile per CTA, 16-deep k slices through shared memory, 4 x 4 outputs per thread.
#include "common.cuh"

namespace {

constexpr int BM = 64, BN = 64, BK = 16, NT = 256;

struct BgArgs {
  const void* x; int64_t ldx, sxh;
  const void* w; int64_t swh, swk, swn;
  const void* bias;              // [N] of T, h-independent, or null
  const float* row_scale; int64_t lds;   // scale(t, h, n) = row_scale[t * lds + h * ssh + n * ssn], or null
  int64_t ssh, ssn;                      // (1, 0): one factor per (token, head); (N, 1): one per output element
  void* out; int64_t ldo, soh;
  int M, N, K, H, act, act_start;
};

__device__ __forceinline__ float act_sq(float x, int act) {
  if (act == LLMSS_ACT_RELU2) { const float r = fmaxf(x, 0.f); return r * r; }
  return act_exact(x, act);
}

template <typename T, bool OUT_F32>
__global__ void __launch_bounds__(NT) bgemm_kernel(BgArgs a) {
  __shared__ float Xs[BK][BM + 4];
  __shared__ float Ws[BK][BN + 4];
  const int h = blockIdx.z;
  const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
  const T* x = reinterpret_cast<const T*>(a.x) + (int64_t)h * a.sxh;
  const T* w = reinterpret_cast<const T*>(a.w) + (int64_t)h * a.swh;
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;
  const bool n_fast = (a.swn == 1);
  for (int k0 = 0; k0 < a.K; k0 += BK) {
    for (int idx = threadIdx.x; idx < BM * BK; idx += NT) {
      const int m = idx / BK, k = idx % BK;
      float v = 0.f;
      if (m0 + m < a.M && k0 + k < a.K) v = to_f32(x[(int64_t)(m0 + m) * a.ldx + k0 + k]);
      Xs[k][m] = v;
    }
    for (int idx = threadIdx.x; idx < BN * BK; idx += NT) {
      int n, k;
      if (n_fast) { k = idx / BN; n = idx % BN; } else { n = idx / BK; k = idx % BK; }
      float v = 0.f;
      if (n0 + n < a.N && k0 + k < a.K) v = to_f32(w[(int64_t)(k0 + k) * a.swk + (int64_t)(n0 + n) * a.swn]);
      Ws[k][n] = v;
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < BK; ++k) {
      float av[4], bv[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) av[i] = Xs[k][ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) bv[j] = Ws[k][tx * 4 + j];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(av[i], bv[j], acc[i][j]);
    }
    __syncthreads();
  }
  using TO = typename std::conditional<OUT_F32, float, T>::type;
  TO* out = reinterpret_cast<TO*>(a.out) + (int64_t)h * a.soh;
  const T* bias = reinterpret_cast<const T*>(a.bias);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int m = m0 + ty * 4 + i;
    if (m >= a.M) continue;
    const float* rsp = a.row_scale != nullptr ? a.row_scale + (int64_t)m * a.lds + (int64_t)h * a.ssh : nullptr;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int n = n0 + tx * 4 + j;
      if (n >= a.N) continue;
      float v = acc[i][j];
      if (bias != nullptr) v += to_f32(bias[n]);
      if (a.act != LLMSS_ACT_NONE && n >= a.act_start) v = act_sq(v, a.act);
      const float rs = rsp != nullptr ? rsp[(int64_t)n * a.ssn] : 1.f;
      out[(int64_t)m * a.ldo + n] = from_f32<TO>(v * rs);
    }
  }
}


// ---------------------------------------------------------------------------------------------------------------
// The same strided batched product on the warp-level tensor-core path (mma.sync m16n8k16, 16-bit operands, 32-bit
// accumulation) for the per-head products of latent attention, whose K and N are one head wide (tens to a few
// hundred): too small for a tcgen05 tile pipeline per head, too much arithmetic for the CUDA cores at prompt sizes.
// CTA tile BM x 64 per head, k slices of 32 staged in shared memory as A[m][k] and B[n][k] (k contiguous, the
// fragment layouts of the instruction); 8 warps, each 16 rows x (64 / warps-per-row) columns.  No bias / activation.
constexpr int MK = 32, MN = 64, MPAD = 8;

template <typename T> struct MmaOp;
template <> struct MmaOp<__nv_bfloat16> {
  static __device__ __forceinline__ void run(float (&c)[4], const uint32_t (&a)[4], const uint32_t (&b)[2]) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
  }
};
template <> struct MmaOp<__half> {
  static __device__ __forceinline__ void run(float (&c)[4], const uint32_t (&a)[4], const uint32_t (&b)[2]) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
  }
};

template <typename T, bool OUT_F32, int TM>
__global__ void __launch_bounds__(NT) bgemm_mma_kernel(BgArgs a) {
  constexpr int WM = TM / 16, WN = 8 / WM, NW = MN / WN, NF = NW / 8;   // warps along m / n, columns and n-fragments per warp
  __shared__ __align__(16) T As[TM][MK + MPAD];
  __shared__ __align__(16) T Bs[MN][MK + MPAD];
  const int h = blockIdx.z;
  const int m0 = blockIdx.y * TM, n0 = blockIdx.x * MN;
  const T* x = reinterpret_cast<const T*>(a.x) + (int64_t)h * a.sxh;
  const T* w = reinterpret_cast<const T*>(a.w) + (int64_t)h * a.swh;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, gid = lane >> 2, tig = lane & 3;
  const int wm = warp % WM, wn = warp / WM;
  float acc[NF][4];
#pragma unroll
  for (int f = 0; f < NF; ++f)
#pragma unroll
    for (int i = 0; i < 4; ++i) acc[f][i] = 0.f;
  const bool n_fast = (a.swn == 1);
  const T zero = from_f32<T>(0.f);
  // 16-byte staging when every vector is whole and aligned (the usual case: head sizes are multiples of 8)
  const bool vec_ok = a.K % 8 == 0 && a.ldx % 8 == 0 && a.sxh % 8 == 0 && a.swh % 8 == 0 &&
                      (reinterpret_cast<uintptr_t>(a.x) | reinterpret_cast<uintptr_t>(a.w)) % 16 == 0 &&
                      (n_fast ? (a.N % 8 == 0 && a.swk % 8 == 0) : (a.swn % 8 == 0));
  for (int k0 = 0; k0 < a.K; k0 += MK) {
    if (vec_ok) {
      const uint4 z4 = make_uint4(0u, 0u, 0u, 0u);
      for (int v = threadIdx.x; v < TM * (MK / 8); v += NT) {
        const int m = v / (MK / 8), kv = (v % (MK / 8)) * 8;
        uint4 val = z4;
        if (m0 + m < a.M && k0 + kv < a.K) val = *reinterpret_cast<const uint4*>(x + (int64_t)(m0 + m) * a.ldx + k0 + kv);
        *reinterpret_cast<uint4*>(&As[m][kv]) = val;
      }
      if (!n_fast) {
        for (int v = threadIdx.x; v < MN * (MK / 8); v += NT) {
          const int n = v / (MK / 8), kv = (v % (MK / 8)) * 8;
          uint4 val = z4;
          if (n0 + n < a.N && k0 + kv < a.K) val = *reinterpret_cast<const uint4*>(w + (int64_t)(n0 + n) * a.swn + k0 + kv);
          *reinterpret_cast<uint4*>(&Bs[n][kv]) = val;
        }
      } else {
        for (int v = threadIdx.x; v < MK * (MN / 8); v += NT) {
          const int k = v / (MN / 8), nv = (v % (MN / 8)) * 8;
          uint4 val = z4;
          if (k0 + k < a.K && n0 + nv < a.N) val = *reinterpret_cast<const uint4*>(w + (int64_t)(k0 + k) * a.swk + n0 + nv);
          const T* e = reinterpret_cast<const T*>(&val);
#pragma unroll
          for (int i = 0; i < 8; ++i) Bs[nv + i][k] = e[i];
        }
      }
    } else {
      for (int idx = threadIdx.x; idx < TM * MK; idx += NT) {
        const int m = idx / MK, k = idx % MK;
        As[m][k] = (m0 + m < a.M && k0 + k < a.K) ? x[(int64_t)(m0 + m) * a.ldx + k0 + k] : zero;
      }
      for (int idx = threadIdx.x; idx < MN * MK; idx += NT) {
        int n, k;
        if (n_fast) { k = idx / MN; n = idx % MN; } else { n = idx / MK; k = idx % MK; }
        Bs[n][k] = (n0 + n < a.N && k0 + k < a.K) ? w[(int64_t)(k0 + k) * a.swk + (int64_t)(n0 + n) * a.swn] : zero;
      }
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < MK; kk += 16) {
      uint32_t af[4];
      const T* ar = &As[wm * 16 + gid][kk + tig * 2];
      af[0] = *reinterpret_cast<const uint32_t*>(ar);
      af[1] = *reinterpret_cast<const uint32_t*>(ar + 8 * (MK + MPAD));
      af[2] = *reinterpret_cast<const uint32_t*>(ar + 8);
      af[3] = *reinterpret_cast<const uint32_t*>(ar + 8 * (MK + MPAD) + 8);
#pragma unroll
      for (int f = 0; f < NF; ++f) {
        uint32_t bf[2];
        const T* br = &Bs[wn * NW + f * 8 + gid][kk + tig * 2];
        bf[0] = *reinterpret_cast<const uint32_t*>(br);
        bf[1] = *reinterpret_cast<const uint32_t*>(br + 8);
        MmaOp<T>::run(acc[f], af, bf);
      }
    }
    __syncthreads();
  }
  using TO = typename std::conditional<OUT_F32, float, T>::type;
  TO* out = reinterpret_cast<TO*>(a.out) + (int64_t)h * a.soh;
#pragma unroll
  for (int half = 0; half < 2; ++half) {
    const int m = m0 + wm * 16 + gid + half * 8;
    if (m >= a.M) continue;
    const float* rsp = a.row_scale != nullptr ? a.row_scale + (int64_t)m * a.lds + (int64_t)h * a.ssh : nullptr;
#pragma unroll
    for (int f = 0; f < NF; ++f)
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        const int n = n0 + wn * NW + f * 8 + tig * 2 + j;
        if (n < a.N) out[(int64_t)m * a.ldo + n] = from_f32<TO>(acc[f][half * 2 + j] * (rsp != nullptr ? rsp[(int64_t)n * a.ssn] : 1.f));
      }
  }
}

template <typename T>
int launch_bg_mma(const BgArgs& a, int out_f32, cudaStream_t stream) {
  if (a.M <= 64) {
    dim3 grid((a.N + MN - 1) / MN, (a.M + 63) / 64, a.H);
    if (out_f32) bgemm_mma_kernel<T, true, 64><<<grid, NT, 0, stream>>>(a);
    else bgemm_mma_kernel<T, false, 64><<<grid, NT, 0, stream>>>(a);
  } else {
    dim3 grid((a.N + MN - 1) / MN, (a.M + 127) / 128, a.H);
    if (out_f32) bgemm_mma_kernel<T, true, 128><<<grid, NT, 0, stream>>>(a);
    else bgemm_mma_kernel<T, false, 128><<<grid, NT, 0, stream>>>(a);
  }
  LLMSS_CHECK_CUDA(cudaGetLastError());
  return 0;
}

template <typename T>
int launch_bg(const BgArgs& a, int out_f32, cudaStream_t stream) {
  dim3 grid((a.N + BN - 1) / BN, (a.M + BM - 1) / BM, a.H);
  if (out_f32) bgemm_kernel<T, true><<<grid, NT, 0, stream>>>(a);
  else bgemm_kernel<T, false><<<grid, NT, 0, stream>>>(a);
  LLMSS_CHECK_CUDA(cudaGetLastError());
  return 0;
}

}  // namespace

// scale(t, h, n) = row_scale[t * lds + h * ssh + n * ssn]: (ssh, ssn) = (1, 0) is one factor per token and head, (N, 1) one per
// output element (an element-wise gate on the concatenated heads)
LLMSS_API int llmss_bgemm_simt_ex(const void* x, int64_t ldx, int64_t sxh, const void* w, int64_t swh, int64_t swk,
                                  int64_t swn, const void* bias, const float* row_scale, int64_t lds, int64_t ssh, int64_t ssn,
                                  void* out, int64_t ldo, int64_t soh, int M, int N, int K, int H, int act, int act_start,
                                  int dtype, int out_f32, cudaStream_t stream) {
  LLMSS_REQUIRE(M >= 0 && N > 0 && K > 0 && H > 0 && H <= 65535, "bgemm_simt: bad shape M=%d N=%d K=%d H=%d", M, N, K, H);
  LLMSS_REQUIRE((M + BM - 1) / BM <= 65535, "bgemm_simt: M=%d too large", M);
  if (M == 0) return 0;
  BgArgs a{x, ldx, sxh, w, swh, swk, swn, bias, row_scale, lds, ssh, ssn, out, ldo, soh, M, N, K, H, act, act_start};
  // 16-bit operands without bias / activation (the per-head products) take the tensor-core form; the 32-bit accumulators
  // are the same, so both forms agree to rounding of the summation order
  const bool mma_ok = dtype != LLMSS_F32 && bias == nullptr && act == LLMSS_ACT_NONE && (M + 127) / 128 <= 65535;
  if (mma_ok && dtype == LLMSS_BF16) return launch_bg_mma<__nv_bfloat16>(a, out_f32, stream);
  if (mma_ok && dtype == LLMSS_F16) return launch_bg_mma<__half>(a, out_f32, stream);
  if (dtype == LLMSS_F32) return launch_bg<float>(a, 1, stream);
  if (dtype == LLMSS_BF16) return launch_bg<__nv_bfloat16>(a, out_f32, stream);
  if (dtype == LLMSS_F16) return launch_bg<__half>(a, out_f32, stream);
  LLMSS_REQUIRE(false, "bgemm_simt: bad dtype %d", dtype);
}

LLMSS_API int llmss_bgemm_simt(const void* x, int64_t ldx, int64_t sxh, const void* w, int64_t swh, int64_t swk,
                               int64_t swn, const void* bias, const float* row_scale, int64_t lds, void* out,
                               int64_t ldo, int64_t soh, int M, int N, int K, int H, int act, int act_start,
                               int dtype, int out_f32, cudaStream_t stream) {
  return llmss_bgemm_simt_ex(x, ldx, sxh, w, swh, swk, swn, bias, row_scale, lds, 1, 0, out, ldo, soh, M, N, K, H, act, act_start,
                             dtype, out_f32, stream);
}

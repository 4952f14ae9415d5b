/* llmss_b200 -- C ABI of the hand-written sm_100a kernel library (libllmss_b200.so).
 *
 * Every entry point returns 0 on success; on failure it returns a non-zero code and
 * llmss_last_error() describes the problem.  Pointers are device pointers unless noted.
 * All launches go to the given stream; nothing here synchronises the device except the
 * symmetric-memory set-up calls.  dtype: 0 = fp16, 1 = bf16, 2 = fp32.
 *
 * Each declaration cites the reference (jongwon-jay-lee/llmss) code it replaces; see
 * SURVEY.md sections 2.5 / 2.6 for the N-number / G-number labels.
 */
#ifndef LLMSS_B200_H_
#define LLMSS_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct CUstream_st* llmss_stream_t;
typedef struct SymmWs llmss_symm_t;

enum { LLMSS_DT_F16 = 0, LLMSS_DT_BF16 = 1, LLMSS_DT_F32 = 2 };

const char* llmss_last_error(void);
int llmss_version(void);

/* ---- symmetric memory (replaces c10d/NCCL bring-up for the hot path; dist.py:44-73) ---- */
int llmss_symm_alloc(size_t buf_bytes, size_t lam_bytes, void** ptr); /* flags + Lamport area + bulk area */
int llmss_symm_free(void* ptr);
int llmss_ipc_get_handle(void* ptr, unsigned char* out64);
int llmss_ipc_open_handle(const unsigned char* in64, void** ptr);
int llmss_ipc_close(void* ptr);
size_t llmss_symm_region_bytes(size_t buf_bytes, size_t lam_bytes);
int llmss_symm_create(int rank, int nranks, void* const* peer_bases, size_t buf_bytes, size_t lam_bytes,
                      llmss_symm_t** out);
int llmss_symm_destroy(llmss_symm_t* ws);
int llmss_symm_epoch(llmss_symm_t* ws, uint32_t* out_host);

/* ---- symmetric heap on the CUDA VMM API + NVLS multicast (csrc/vmm.cu) ----
 * Each rank: llmss_vmm_padded_size (identical on all ranks) -> llmss_vmm_alloc -> llmss_symm_init_region on
 * llmss_vmm_ptr -> llmss_vmm_export_fd once per peer, descriptor sent with llmss_fdx_send / received with
 * llmss_fdx_recv (abstract Unix datagram sockets, SCM_RIGHTS) -> llmss_vmm_import.  Optional NVLS: rank 0
 * llmss_mc_create + descriptor to every peer (llmss_mc_import), all llmss_mc_add_device, barrier, all
 * llmss_mc_bind_and_map, barrier; llmss_vmm_mc_ptr is then the multicast mapping (a store lands on every GPU,
 * multimem.ld_reduce sums all copies in the switch).  llmss_symm_create2 takes the peer mappings and that pointer
 * (null: P2P only).  The reference has none of this: its buffers belong to NCCL (dist.py:44-73). */
typedef struct llmss_vmm_region llmss_vmm_region;
int llmss_vmm_caps(int* caps); /* bit 0: VMM + POSIX-fd handles, bit 1: multicast objects */
int llmss_vmm_padded_size(size_t bytes, int nranks, int want_multicast, size_t* padded);
int llmss_vmm_alloc(size_t padded, llmss_vmm_region** out);
void* llmss_vmm_ptr(llmss_vmm_region* r);
void* llmss_vmm_mc_ptr(llmss_vmm_region* r);
size_t llmss_vmm_bytes(llmss_vmm_region* r);
int llmss_vmm_export_fd(llmss_vmm_region* r, int* fd);
int llmss_vmm_import(int fd, size_t padded, void** ptr); /* closes fd */
int llmss_vmm_unmap(void* ptr, size_t padded);
int llmss_vmm_free(llmss_vmm_region* r);
int llmss_mc_create(int nranks, size_t padded, unsigned long long* mc, int* fd);
int llmss_mc_import(int fd, unsigned long long* mc);
int llmss_mc_add_device(unsigned long long mc);
int llmss_mc_bind_and_map(unsigned long long mc, llmss_vmm_region* r);
int llmss_mc_release(unsigned long long mc);
int llmss_fdx_open(const char* name, int* sock);
int llmss_fdx_send(int sock, const char* peer_name, int tag, int fd);
int llmss_fdx_recv(int sock, int timeout_ms, int* tag, int* fd);
int llmss_fdx_close(int sock);
int llmss_fd_close(int fd);
int llmss_symm_init_region(void* ptr, size_t buf_bytes, size_t lam_bytes); /* zero flags, arm the Lamport area */
int llmss_symm_create2(int rank, int nranks, void* const* peer_bases, void* mc_base, size_t buf_bytes, size_t lam_bytes,
                       llmss_symm_t** out);
int llmss_symm_has_multicast(llmss_symm_t* ws);
/* watchdog self test: waits on `flag` (a device uint32 nobody raises to `want`); the kernel traps after the 4 s spin
 * limit and the context is lost -- call it from a throw-away process only */
int llmss_debug_wait_flag(const uint32_t* flag, uint32_t want, llmss_stream_t stream);

/* ---- K4 collectives over NVLink peer memory (N1/N2: layers.py:178,213; N3: layers.py:133) ---- */
/* algo: 0 auto | 1 one-shot Lamport push | 2 two-shot with flags | 3 NVLS (stage locally, multimem.ld_reduce of the owned
 * 1/t, multimem.st broadcast) | 4 two-shot on Lamport vectors (reduce-scatter by peer stores, multicast broadcast) */
int llmss_allreduce(llmss_symm_t* ws, const void* in, void* out, int64_t n, int dtype, int algo,
                    llmss_stream_t stream);
int llmss_allgather(llmss_symm_t* ws, const void* in, void* out, int64_t bytes, llmss_stream_t stream);
/* gather along the last dimension: in [rows][row_bytes] -> out [rows][nranks * row_bytes] (N3: the vocab-parallel
 * logits all-gather + cat of layers.py:131-135 in one pass) */
int llmss_allgather_cols(llmss_symm_t* ws, const void* in, void* out, int64_t rows, int64_t row_bytes,
                         llmss_stream_t stream);

/* ---- K5/K1/K2 tcgen05 GEMM (+ fused all-reduce epilogue) (G3,G4,G9,G10,G12,G14; layers.py:62,175-179) ---- */
typedef struct llmss_gemm_plan {
  int bn, tiles, kb_total, grid;
  int split; /* 0 = stream-K persistent kernel, 1..8 = thread-block-cluster split-K factor (1: one CTA per tile) */
  int64_t sk_ws_floats;
  int64_t sk_counters;
  int64_t ar_bytes;
} llmss_gemm_plan;
/* CTA-pair kernel (tcgen05 cta_group::2) for token tiles of 129..256 rows: -1 = environment (LLMSS_GEMM_PAIR =
 * off | auto | 1 | 2 | 4), 0 = off, 1 / 2 / 4 = pairs per cluster (split-K depth), 8 = automatic */
int llmss_gemm_set_pair(int mode);
int llmss_gemm_set_debug(unsigned long long* per_cta_stamps); /* profiling aid: 8 globaltimer stamps per CTA */
int llmss_gemm_plan_query(int M, int N, int K, int nranks, int elem_bytes, int max_ctas, llmss_gemm_plan* p);
int llmss_gemm_plan_query2(int M, int N, int K, int nranks, int elem_bytes, int max_ctas, int dtype, llmss_gemm_plan* p);
int llmss_gemm(const void* x, int64_t ldx, const void* w, int64_t ldw, const void* bias, const void* residual,
               int64_t ldr, void* out, int64_t ldo, int M, int N, int K, int dtype, int out_f32, int act,
               int act_start, int gated, float* sk_ws, uint32_t* sk_counters, llmss_symm_t* ws, int max_ctas,
               llmss_stream_t stream);

/* collective: 0 none | 1 GEMM -> all-reduce (exchange chosen by size and rank count) | 2 GEMM -> reduce-scatter over
 * token rows (K2) | 3 all-gather -> GEMM (K3: x is this rank's row shard; shards are staged into every rank's own
 * buffer -- one multicast store each when the heap is multicast-bound -- and TMA-read from local memory) |
 * 4 / 5 / 6 pin the all-reduce exchange: in-switch multimem.ld_reduce / one-shot push / two-shot Lamport. */
int llmss_gemm_ex(const void* x, int64_t ldx, const void* w, int64_t ldw, const void* bias, const void* residual,
                  int64_t ldr, void* out, int64_t ldo, int M, int N, int K, int dtype, int out_f32, int act,
                  int act_start, int gated, float* sk_ws, uint32_t* sk_counters, llmss_symm_t* ws, int max_ctas,
                  int collective, void* ag_maps_dev, llmss_stream_t stream);

/* ---- K6 fused residual add + LayerNorm / RMSNorm (G2, G13, G18; layers.py:12-36,217-256) ---- */
int llmss_norm_residual(const void* x, const void* x2, const void* residual_in, void* residual_out,
                        const void* weight, const void* bias, void* out, int M, int H, int64_t ldx, int64_t ldx2,
                        int64_t ldr, int64_t ldo, float eps, int kind, int dtype, llmss_stream_t stream);

/* ---- K7 RoPE + paged KV-cache append (G5, G6; gptj_modeling.py:26-47,206-233) ---- */
int llmss_rope_kv_write(void* qkv, const int* positions, const int* slot_mapping, void* k_cache, void* v_cache,
                        int T, int64_t ld, int hq, int hkv, int d, int rotary_dim, int style, float base, int q_off,
                        int k_off, int v_off, int block_size, int dtype, llmss_stream_t stream);

/* ---- K9 paged split-KV decode attention (G7, G8, G17; gptj_modeling.py:128-169) ---- */
/* Tensor-core (tcgen05) paged decode attention for grouped / multi-query models (hq / hkv >= 2): the
 * q heads that share a KV head are the rows of one MMA, so each KV page is read once per group
 * (reference: baddbmm/softmax/bmm on a replicated KV tensor, gpt_bigcode_modeling.py:170-246).
 * Same contract as llmss_attn_decode plus num_blocks (pages in the cache); block_size must be 16.
 * Scratch size: llmss_attn_decode_scratch_floats. */
int llmss_attn_decode_tc(const void* q, int64_t ldq, const void* k_cache, const void* v_cache,
                         const int* block_tables, int max_blocks, const int* seq_lens, void* out,
                         int64_t ldo, float* scratch, int B, int hq, int hkv, int d, int block_size,
                         int num_blocks, float scale, int num_splits, int dtype, llmss_stream_t stream);
int llmss_attn_decode_tc_pick_splits(int B, int hkv, int d, int max_kv);
/* 1 if llmss_attn_decode_tc takes this grouping / head size (query tile + two key stages fit into shared memory) */
int llmss_attn_decode_tc_supported(int hq, int hkv, int d, int block_size);
/* num_splits = 0 selects the balanced mode: all key tiles of the batch are cut into equal contiguous ranges,
 * one per SM (no wave quantisation of items / SMs); its scratch is sized by the function below. */
int64_t llmss_attn_decode_tc_balanced_scratch_floats(int B, int hq, int d, int max_blocks, int block_size);
/* Merge split-KV partials (part_o [B,hq,splits,d], part_ml [B,hq,splits,2]) into out. */
int llmss_attn_decode_combine(const float* part_o, const float* part_ml, void* out, int64_t ldo, int B,
                              int hq, int d, int num_splits, int dtype, llmss_stream_t stream);
int64_t llmss_attn_decode_scratch_floats(int B, int hq, int d, int num_splits);
int llmss_attn_decode_pick_splits(int B, int hq, int hkv, int d, int max_kv, int dtype); /* wave-filling split factor */
int llmss_attn_decode(const void* q, int64_t ldq, const void* k_cache, const void* v_cache,
                      const int* block_tables, int max_blocks, const int* seq_lens, void* out, int64_t ldo,
                      float* scratch, int B, int hq, int hkv, int d, int block_size, float scale, int num_splits,
                      int dtype, llmss_stream_t stream);

/* ---- K8 causal varlen prefill attention on tcgen05 (G7, G8, G17; gpt_bigcode_modeling.py:170-246) ---- */
int llmss_attn_prefill(const void* q, int64_t ldq, const void* k, int64_t ldk, const void* v, int64_t ldv, void* out,
                       int64_t ldo, const int* cu_seqlens, int num_seqs, int max_seqlen, int total_tokens, int hq,
                       int hkv, int d, float scale, int dtype, llmss_stream_t stream);

/* Multi-token queries over prior context (chunked prefill, prefix reuse; gptj_modeling.py:128-169 with a past,
 * 229-233): same tcgen05 kernel, K / V tiles gathered page by page from the paged cache (which already holds this
 * step's keys); seq_lens[i] includes the cu_q[i+1] - cu_q[i] new tokens; block_size 16 / 32 / 64; out may alias q. */
int llmss_attn_prefill_paged(const void* q, int64_t ldq, const void* k_cache, const void* v_cache,
                             const int* block_tables, int max_blocks, const int* seq_lens, void* out, int64_t ldo,
                             const int* cu_q, int num_seqs, int max_q, int total_q, int hq, int hkv, int d,
                             int block_size, int num_blocks, float scale, int dtype, llmss_stream_t stream);

/* No counterpart in the reference (it has no native code and allocates freely through torch).
 * Same operation as llmss_attn_decode for hosts that cannot allocate: servers whose HBM is fully
 * committed to weights + KV pages, decode loops that cannot afford the device-wide sync of
 * cudaMalloc/cudaFree, and plain C hosts with no allocator to lend us scratch.  The split-KV
 * partials live in an 8 MiB array built into the library (held by every GPU that loads it).
 * Refuses B*hq*num_splits*(d+2) floats > llmss_attn_decode_static_max_floats().  The first call
 * on a device resolves the array's address: make it at start-up, before any stream capture.
 * Calls share the array; kernels of two calls that overlap on the GPU race. */
int64_t llmss_attn_decode_static_max_floats(void);
int llmss_attn_decode_static(const void* q, int64_t ldq, const void* k_cache, const void* v_cache,
                             const int* block_tables, int max_blocks, const int* seq_lens, void* out, int64_t ldo,
                             int B, int hq, int hkv, int d, int block_size, float scale, int num_splits, int dtype,
                             llmss_stream_t stream);

/* ---- 32-bit residual stream + Dynamic Tanh (y = tanh(alpha x) w + b; no statistics) ----
 * res_out = res_in + s1 * a + s2 * b (a, b: 32-bit branch outputs, s1 / s2: per-feature layer scales or null);
 * out = DyT(res_out) in `dtype` (0 half, 1 bf16, 2 float); res_out may alias res_in; out / res_out may be null. */
int llmss_dyt_residual(const float* res_in, float* res_out, const float* a, const void* s1, const float* b, const void* s2,
                       const void* w, const void* bias, void* out, float alpha, int M, int H, int64_t ldr, int64_t lda,
                       int64_t ldb, int64_t ldo, int dtype, llmss_stream_t stream);
/* token (+ learned position) embedding summed and stored in 32-bit */
int llmss_embed_f32(const int* tokens, const int* positions, const void* wte, const void* wpe, float* out, int T, int H,
                    int vocab, int max_pos, int pos_offset, int64_t ldo, int dtype, llmss_stream_t stream);
/* out[:, :Ha] = cast(a), out[:, Ha:] = cast(b): 32-bit streams -> one GEMM operand */
int llmss_cast_concat(const float* a, const float* b, void* out, int M, int Ha, int Hb, int64_t lda, int64_t ldb, int64_t ldo,
                      int dtype, llmss_stream_t stream);

/* ---- strided batched GEMM on the CUDA cores (true 32-bit layers, unaligned 16-bit layers, per-head products) ----
 * out(t,h,n) = act(sum_k x[t*ldx + h*sxh + k] * w[h*swh + k*swk + n*swn] + bias[n]) * row_scale[t*lds + h] */
int llmss_bgemm_simt(const void* x, int64_t ldx, int64_t sxh, const void* w, int64_t swh, int64_t swk, int64_t swn,
                     const void* bias, const float* row_scale, int64_t lds, void* out, int64_t ldo, int64_t soh, int M, int N,
                     int K, int H, int act, int act_start, int dtype, int out_f32, llmss_stream_t stream);

/* ---- latent (low-rank KV) attention, absorbed form, paged cache [num_blocks, block_size, R] ----
 * prep: y is the 32-bit output of the fused input projection; columns [c_off, c_off + R) are RMS-normed with norm_w and
 * written to the cache slot of each token (slot < 0: not written), columns [q_off, q_off + n_q) are cast to q_out, columns
 * [g_off, g_off + H) go through a sigmoid into gate [T, H] (gate may be null). */
int llmss_latent_prep(const float* y, int64_t ldy, int q_off, int c_off, int g_off, int n_q, int R, int H, const void* norm_w,
                      float eps, const int* slots, void* cache, void* q_out, int64_t ldq, float* gate, int T, int dtype,
                      llmss_stream_t stream);
int64_t llmss_latent_attn_scratch_floats(int T, int H, int R, int splits);
/* q: absorbed queries [T, H * R] (32-bit); token i of sequence b sees cache positions 0 .. seq_lens[b] - q_len_b + i */
int llmss_latent_attn(const float* q, int64_t ldq, const void* cache, const int* block_tables, int max_blocks, int block_size,
                      const int* seq_lens, const int* cu_q, void* out, int64_t ldo, float* scratch, int T, int num_seqs,
                      int max_q, int H, int R, float scale, int splits, int dtype, llmss_stream_t stream);

/* ---- routed mixture of experts ----
 * route: softmax over E logits, group-limited top-k (ids / wts: [T, top]; dense: optional [T, E], 0 = not chosen) */
int llmss_moe_route(const float* z, int64_t ldz, int T, int E, int top, int groups, int keep, float route_scale, int* ids,
                    float* wts, float* dense, llmss_stream_t stream);
/* out[t] = sum_k wts[t,k] * W_down[ids[t,k]] act(W_up[ids[t,k]] h[t]); w_up [E, F, W]; w_down [W, E * F] (the experts' down matrices side by side,
 * row stride ldd); act_scratch [T, top, F] */
int llmss_moe_experts(const void* h, int64_t ldh, const int* ids, const float* wts, const void* w_up, const void* w_down,
                      int64_t ldd, void* act_scratch, float* out, int64_t ldo, int T, int W, int F, int top, int act, int gated,
                      int dtype, llmss_stream_t stream);   /* gated: w_up rows interleave (gate_f, up_f), hidden = act(gate) * up */
/* grouped form: count pairs per expert; (host turns counts into offsets); ordered permutation perm[row] = pair,
 * inv[pair] = row; gather the pairs' token rows; (per-expert GEMMs on contiguous rows); weighted sum per token */
int llmss_moe_count(const int* ids, int P, int E, int* counts, llmss_stream_t stream);
int llmss_moe_permute(const int* ids, int P, int E, const int* offsets, int* perm, int* inv, llmss_stream_t stream);
int llmss_moe_gather_rows(const void* h, int64_t ldh, const int* perm, int top, void* xs, int P, int W, int dtype,
                          llmss_stream_t stream);
int llmss_moe_combine(const float* y, const int* inv, const float* wts, float* out, int64_t ldo, int T, int W, int top,
                      llmss_stream_t stream);
int llmss_moe_scale(void* a, int64_t lda, const float* dense, int T, int E, int F, int dtype, llmss_stream_t stream);

/* ---- K10 embedding gather (G1; layers.py:182-214) ---- */
int llmss_embed(const int* tokens, const int* positions, const void* wte, const void* wpe, void* out, int T, int H,
                int vocab, int max_pos, int pos_offset, int64_t ldo, int dtype, llmss_stream_t stream);

/* ---- K11 (greedy case) vocab-parallel argmax: per-rank candidate, gathered with llmss_allgather_cols (16 bytes
 * per row and rank), merged on every rank -- no [B, V] logits all-gather (generate.py:111, layers.py:131-135) ---- */
int llmss_argmax_local(const float* logits, int64_t ld, int B, int n_valid, int idx_offset, void* cand,
                       llmss_stream_t stream);
int llmss_argmax_merge(const void* cand_all, int nranks, int B, int* out_tokens, long long* out_tokens64,
                       llmss_stream_t stream);

/* ---- K11 (general case) vocab-parallel top-k / top-p / temperature sampling (generate.py:109-126, layers.py:131-135):
 * step 1 on every rank: one record of llmss_vp_record_floats(ks) floats per row -- [max, sum-exp, count, sum-exp at the row's temperature,
 * vals[ks], idx[ks]] -- from its fp32 shard; gather the records with llmss_allgather_cols; step 2 on every rank: merge + draw
 * (identical tokens everywhere, rng_state advanced).  Exact for 1 <= top_k <= ks; nranks * ks <= 1024. ---- */
int llmss_vp_record_floats(int ks);
int llmss_vp_summary(const float* logits, int64_t ld, int B, int n_valid, int idx_offset, const int* greedy,
                     const int* top_k, const float* temperature, float* recs, int ks, llmss_stream_t stream);
/* rows drawn from the whole distribution (top_k = 0, top_p = 1 -- what the reference's loop effectively samples, quirk Q1):
 * after the record gather every rank runs llmss_vp_multinomial_pick (the rank whose CDF interval holds the draw names the
 * token, all others answer -1; does not advance the RNG), `cand` ([B][4] int32) is gathered with llmss_allgather_cols,
 * llmss_vp_merge_sample runs for all rows and llmss_vp_multinomial_merge overwrites the tokens of those rows. */
int llmss_vp_multinomial_pick(const float* logits, int64_t ld, int B, int n_valid, int idx_offset, const float* recs_all,
                              int nranks, int rank, int ks, const int* greedy, const float* temperature, const int* top_k,
                              const float* top_p, const uint32_t* rng_state, int* cand, llmss_stream_t stream);
int llmss_vp_multinomial_merge(const int* cand_all, int nranks, int B, int* out_tokens, long long* out_tokens64,
                               llmss_stream_t stream);
int llmss_vp_merge_sample(const float* recs_all, int nranks, int ks, int B, int vocab, const int* greedy,
                          const float* temperature, const int* top_k, const float* top_p, uint32_t* rng_state,
                          int* out_tokens, long long* out_tokens64, llmss_stream_t stream);

/* ---- K11 fused sampler (G15, G16, N6; generate.py:109-144) ----
 * rng_state: [B][2] = (request seed, tokens sampled so far); the draw depends on nothing else (not on the row).
 * top_k = 0 with top_p < 1: the nucleus is searched among the 1024 most probable tokens (a wider nucleus is cut there);
 * top_k = 0 with top_p = 1 samples the whole distribution. */
int llmss_sample(const float* logits, int64_t ld, int B, int vocab, const int* greedy, const float* temperature,
                 const int* top_k, const float* top_p, uint32_t* rng_state, int* out_tokens,
                 long long* out_tokens64, llmss_stream_t stream);
/* the tcgen05 paged flash kernel with a distance bias (bias_over_scale [hq][n_dist] = bias / scale) and a per-head output
 * gate sigmoid(gate[token][head]); 16-bit, head_dim 64 / 128 / 256 for keys and values alike */
int llmss_attn_prefill_paged_bias(const void* q, int64_t ldq, const void* k_cache, const void* v_cache, const int* block_tables,
                                  int max_blocks, const int* seq_lens, void* out, int64_t ldo, const int* cu_q, int num_seqs,
                                  int max_q, int total_q, int hq, int hkv, int d, int block_size, int num_blocks, float scale,
                                  int dtype, const float* bias_over_scale, int n_dist, const float* gate, int64_t ldg,
                                  llmss_stream_t stream);

/* ---- recurrent token mixers and the post-normed 32-bit residual stream (csrc/recurrent.cu, csrc/attn_bias.cu).
 * Batch convention: sequence b owns rows cu_q[b]..cu_q[b+1], holds seq_lens[b] tokens including them, and keeps its state
 * in row slots[b] of every state tensor (slot < 0: inert row).  A sequence at position 0 starts from zeros. */
int llmss_embed_bigram(const int* tokens, const void* wte, const void* table, float* out, int T, int W, int vocab, int64_t mul_prev,
                       int64_t mul_cur, int buckets, const int* cu_q, const int* seq_lens, const int* slots, int B, int max_q,
                       int* prev_state, int dtype, llmss_stream_t stream);
int llmss_postnorm_residual(const float* y, int64_t ldy, const float* y2, int64_t ldy2, const float* w_a, const float* w_b,
                            const float* weight, const float* resid, int64_t ldr, float* new_resid, void* out, int T, int W,
                            float eps, int one_plus, int dtype, llmss_stream_t stream);
int llmss_token_shift(const float* x, int64_t ldx, const float* mu, int S, void* out, int T, int W, const int* cu_q,
                      const int* seq_lens, const int* slots, int B, int max_q, float* prev_state, int dtype, llmss_stream_t stream);
int llmss_causal_conv(const float* u, int64_t ldu, const float* w, const float* bias, float* out, int T, int C, int taps, int act,
                      const int* cu_q, const int* seq_lens, const int* slots, int B, int max_q, float* state, llmss_stream_t stream);
int llmss_unary_f32(const float* x, int64_t ldx, void* out, int rows, int cols, int op, int out_dtype, llmss_stream_t stream);
int llmss_ssm_dt(const float* raw, int64_t ldr, const float* dt_bias, const float* a_log, float* dt, float* logdecay, int T, int H,
                 llmss_stream_t stream);
/* decay_kind 0: decay[H] values; 1: [T, H] log decays; 2: [T, H * dk] log decays.  state: [slots, H, dv, dk] 32-bit.
 * chunk > 0: two passes over chunks of that many tokens (a multiple of 16), with scratch of llmss_linear_scan_scratch_floats */
int64_t llmss_linear_scan_scratch_floats(int B, int heads, int dk, int dv, int max_q, int chunk);
int llmss_linear_scan(const float* q, int64_t ldq, const float* k, int64_t ldk, const float* v, int64_t ldv, const float* decay,
                      int64_t ldd, int decay_kind, const float* bonus, const float* vscale, int64_t ldvs, float* out, float* state,
                      const int* cu_q, const int* seq_lens, const int* slots, int B, int heads, int qk_heads, int dk, int dv,
                      int read_before, float* scratch, int chunk, int max_q, llmss_stream_t stream);
/* tcgen05 decode attention with a score bias per head and key distance; x[t, h * dv + c] *= sigmoid(gate[t, h]) */
int llmss_attn_decode_tc_bias(const void* q, int64_t ldq, const void* k_cache, const void* v_cache, const int* block_tables,
                              int max_blocks, const int* seq_lens, void* out, int64_t ldo, float* scratch, int B, int hq, int hkv,
                              int d, int block_size, int num_blocks, float scale, int num_splits, int dtype,
                              const float* bias_over_scale, int n_dist, llmss_stream_t stream);
int llmss_head_gate(void* x, int64_t ldx, const float* gate, int64_t ldg, int T, int hq, int dv, int dtype, llmss_stream_t stream);
int llmss_gated_rmsnorm(const float* o, int64_t ldo, const float* gate, int64_t ldg, int gate_act, const float* weight, int groups,
                        float eps, int gate_first, const float* skip_x, int64_t ldx, const float* skip_d, int H, void* out, int T,
                        int C, int dtype, llmss_stream_t stream);
int llmss_qknorm_kv_write(const float* qkv, int64_t ld, int hq, int hkv, int dk, int dv, const float* q_w, const float* k_w, float eps,
                          float temp_coef, int temp_every, const int* positions, const int* slots, void* k_cache, void* v_cache,
                          int block_size, void* q_out, int T, int dtype, llmss_stream_t stream);
int llmss_attention_bias(const void* q, int64_t ldq, const void* k_cache, const void* v_cache, const int* block_tables,
                         int max_blocks, int block_size, const int* seq_lens, const int* cu_q, const float* bias, int n_dist,
                         const float* gate, int64_t ldg, void* out, int B, int max_q, int hq, int hkv, int dk, int dv, float scale,
                         int dtype, llmss_stream_t stream);

/* General query / key / value preparation: norm per head (whole = 0) or over a token's whole projection (whole = 1, weights of
 * that size), a factor per query head, values divided by their per-head rms (v_norm), hkv = 0 for queries only. */
int llmss_qkv_prepare(const float* qkv, int64_t ld, int hq, int hkv, int dk, int dv, const float* q_w, const float* k_w, float eps,
                      float temp_coef, int temp_every, const float* q_head_scale, int whole, int v_norm, const int* positions,
                      const int* slots, void* k_cache, void* v_cache, int block_size, void* q_out, int T, int dtype,
                      llmss_stream_t stream);
/* llmss_attention_bias with a linear penalty slopes[h] * distance (or null) and a sliding window (window > 0: distance < window) */
int llmss_attention_window(const void* q, int64_t ldq, const void* k_cache, const void* v_cache, const int* block_tables,
                           int max_blocks, int block_size, const int* seq_lens, const int* cu_q, const float* bias, int n_dist,
                           const float* slopes, int window, const float* gate, int64_t ldg, void* out, int B, int max_q, int hq,
                           int hkv, int dk, int dv, float scale, int dtype, llmss_stream_t stream);

/* ---- several residual streams and the gated delta rule (csrc/streams.cu, csrc/delta.cu) */
/* out [streams][T][W] = wte[tok] * scale + sinusoid(position); inv_freq: W / 2 (rounded up) 64-bit inverse frequencies */
int llmss_embed_sinusoid(const int* tokens, const int* positions, const void* wte, const double* inv_freq, float* out, int T, int W,
                         int vocab, float scale, int streams, int dtype, llmss_stream_t stream);
/* xs [streams][T][W] in place: x_t <- sum_s mix[s][t] x_s + w_out[t] y (y null: no write); then out = rms_div(sum_s w_in[s] x_s)
 * * norm_w (norm_w null: the sum itself; w_in null: no read-out) */
int llmss_hyper_residual(float* xs, int T, int W, int streams, const float* y, int64_t ldy, const float* mix, const float* w_out,
                         const float* w_in, const float* norm_w, float eps, void* out, int out_dtype, llmss_stream_t stream);
/* S <- exp(log_decay) S; u = beta (v - S^T k); S <- S + k u^T; o = S^T q.  state [slots, heads, dv, dk]; unit_eps >= 0: q, k
 * become unit vectors per head first; beta_sigmoid: beta is given before its sigmoid; max_q <= 1 (every sequence brings one
 * token) selects the form with one warp per state column */
int llmss_delta_scan(const float* q, int64_t ldq, const float* k, int64_t ldk, const float* v, int64_t ldv, const float* log_decay,
                     int64_t ldg, const float* beta, int64_t ldb, float* out, float* state, const int* cu_q, const int* seq_lens,
                     const int* slots, int B, int max_q, int heads, int qk_heads, int dk, int dv, float unit_eps, float q_scale,
                     int beta_sigmoid, llmss_stream_t stream);

/* ---- rotation by a frequency table, sandwich norms, gated linear recurrence inputs (csrc/rotary.cu) and the general forms they
 * use elsewhere.  freq: n_pairs 64-bit frequencies (the first 2 n_pairs channels of a head rotate, the rest pass); mag multiplies
 * cos and sin; interleaved: pairs (2i, 2i+1), else (i, i + n_pairs). */
/* qk [T, hq*d + hkv*d] 32-bit: q, k rotated, unit_norm: every head / its rms; keys -> k_cache, the projected keys -> v_cache */
int llmss_rope_norm_kv_write(const float* qk, int64_t ld, int hq, int hkv, int d, const double* freq, int n_pairs, float mag,
                             int interleaved, int unit_norm, float eps, const int* positions, const int* slots, void* k_cache,
                             void* v_cache, int block_size, void* q_out, int T, int dtype, llmss_stream_t stream);
/* y [T, *] 32-bit: cq_out = rmsnorm(y[q_off .. + q_rank]) * qn_w; cache row = [rmsnorm(y[c_off .. + rank]) * cn_w | rotate(next
 * rot columns) | zeros up to width]; gate = sigmoid(y[g_off .. + n_gate]) */
int llmss_latent_rope_prep(const float* y, int64_t ldy, int q_off, int q_rank, int c_off, int rank, int rot, int g_off, int n_gate,
                           const float* qn_w, const float* cn_w, float eps, const double* freq, int n_pairs, float mag,
                           const int* positions, const int* slots, void* cache, int width, void* cq_out, float* gate, int T,
                           int dtype, llmss_stream_t stream);
/* q [T, H * (d + rot)] 32-bit -> q_nope [T, H * d] and the columns [rank, width) of every head of q_abs [T, H * width] */
int llmss_latent_query_rope(const float* q, int64_t ldq, int H, int d, int rot, int rank, int width, const double* freq, int n_pairs,
                            float mag, const int* positions, void* q_nope, void* q_abs, int abs_f32, int T, int dtype,
                            llmss_stream_t stream);
/* y [T, >= 2 n_qk] = [q | f | ..]: q = silu(q), k = 1 - f, lnf = ln f with f = lower + (1 - lower) sigmoid(f) */
int llmss_hgrn_gates(const float* y, int64_t ldy, int n_qk, const float* lower, float* q, float* k, float* lnf, int T,
                     llmss_stream_t stream);
int llmss_softcap(float* z, int64_t ldz, int rows, int cols, float cap, llmss_stream_t stream);   /* z <- cap tanh(z / cap) */
/* r = resid + rms_div(y) * w_post (y null: resid); hist given: hist[index] = r, and with depth_w r = sum_(j <= index) depth_w[j]
 * hist[j]; out_r = r; w_next given: out_h = rms_div(r) * w_next in out_dtype */
int llmss_sandwich_residual(const float* resid, int64_t ldr, const float* y, int64_t ldy, const float* w_post, float* hist,
                            int index, const float* depth_w, const float* w_next, float* out_r, void* out_h, int T, int W, float eps,
                            int out_dtype, llmss_stream_t stream);
/* llmss_attention_window with a sink logit per head (sinks [hq] or null): exp(sinks[h]) joins every denominator of head h */
int llmss_attention_sink(const void* q, int64_t ldq, const void* k_cache, const void* v_cache, const int* block_tables,
                         int max_blocks, int block_size, const int* seq_lens, const int* cu_q, const float* bias, int n_dist,
                         const float* slopes, int window, const float* gate, int64_t ldg, const float* sinks, void* out, int B,
                         int max_q, int hq, int hkv, int dk, int dv, float scale, int dtype, llmss_stream_t stream);
/* the tcgen05 kernels with a sink logit per q head (sinks [hq] 32-bit; bias_over_scale and gate may be null; scale > 0) */
int llmss_attn_prefill_paged_sink(const void* q, int64_t ldq, const void* k_cache, const void* v_cache, const int* block_tables,
                                  int max_blocks, const int* seq_lens, void* out, int64_t ldo, const int* cu_q, int num_seqs,
                                  int max_q, int total_q, int hq, int hkv, int d, int block_size, int num_blocks, float scale,
                                  int dtype, const float* bias_over_scale, int n_dist, const float* gate, int64_t ldg,
                                  const float* sinks, llmss_stream_t stream);
int llmss_attn_decode_tc_sink(const void* q, int64_t ldq, const void* k_cache, const void* v_cache, const int* block_tables,
                              int max_blocks, const int* seq_lens, void* out, int64_t ldo, float* scratch, int B, int hq, int hkv,
                              int d, int block_size, int num_blocks, float scale, int num_splits, int dtype,
                              const float* bias_over_scale, int n_dist, const float* sinks, llmss_stream_t stream);
int llmss_attn_decode_combine_sink(const float* part_o, const float* part_ml, void* out, int64_t ldo, int B, int hq, int d,
                                   int num_splits, int dtype, const float* sinks, llmss_stream_t stream);
/* llmss_moe_route with score_kind (0 softmax, 1 sigmoid), a per-expert correction added for the choice only (or null), groups
 * scored by the sum of their group_top best, weights renormalised over the chosen experts or not */
int llmss_moe_route_ex(const float* z, int64_t ldz, int T, int E, int top, int groups, int keep, float route_scale, int score_kind,
                       const float* correction, int group_top, int renorm, int* ids, float* wts, float* dense, llmss_stream_t stream);
/* llmss_causal_conv with the output in out_dtype */
int llmss_causal_conv_to(const float* u, int64_t ldu, const float* w, const float* bias, void* out, int out_dtype, int T, int C,
                         int taps, int act, const int* cu_q, const int* seq_lens, const int* slots, int B, int max_q, float* state,
                         llmss_stream_t stream);
/* llmss_embed_f32 with a factor on the token row */
int llmss_embed_scaled_f32(const int* tokens, const int* positions, const void* wte, const void* wpe, float* out, int T, int H,
                           int vocab, int max_pos, int pos_offset, int64_t ldo, float scale, int dtype, llmss_stream_t stream);
/* llmss_bgemm_simt with scale(t, h, n) = row_scale[t * lds + h * ssh + n * ssn] */
int llmss_bgemm_simt_ex(const void* x, int64_t ldx, int64_t sxh, const void* w, int64_t swh, int64_t swk, int64_t swn,
                        const void* bias, const float* row_scale, int64_t lds, int64_t ssh, int64_t ssn, void* out, int64_t ldo,
                        int64_t soh, int M, int N, int K, int H, int act, int act_start, int dtype, int out_f32,
                        llmss_stream_t stream);

#ifdef __cplusplus
}
#endif
#endif /* LLMSS_B200_H_ */

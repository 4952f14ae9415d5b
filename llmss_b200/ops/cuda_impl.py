"""CUDA execution path: thin wrappers that hand torch tensors to the sm_100a kernels.

All launches use torch's current stream, so they are captured by ``torch.cuda.graph``.
Outputs are allocated with torch (graph-pool friendly); scratch for stream-K / split-KV is
a per-device arena allocated once.
"""
from __future__ import annotations

import ctypes as C
import os
from typing import Optional

import torch

from . import _lib
from .reference import ACT_NONE

_DT = {torch.float16: 0, torch.bfloat16: 1, torch.float32: 2}


def _ptr(t: Optional[torch.Tensor]):
    return None if t is None else C.c_void_p(t.data_ptr())


def _stream():
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


def _count(n: int = 1):
    _lib.LAUNCHES["count"] += n


class _Arena:
    """Per-device scratch: stream-K partials + tile counters + split-KV partials."""

    SK_FLOATS = 2 * 148 * 128 * 256
    SK_COUNTERS = 1 << 16

    def __init__(self, device):
        self.sk_ws = torch.empty(self.SK_FLOATS, dtype=torch.float32, device=device)
        self.sk_counters = torch.zeros(self.SK_COUNTERS, dtype=torch.int32, device=device)
        self.attn = None
        self.ag_maps = None
        self._retired = []  # outgrown buffers stay alive: captured CUDA graphs may still point at them

    def attn_scratch(self, nfloats: int, device):
        if self.attn is None or self.attn.numel() < nfloats:
            if self.attn is not None:
                self._retired.append(self.attn)
            self.attn = torch.empty(max(nfloats, 1 << 22), dtype=torch.float32, device=device)
        return self.attn


_ARENAS = {}


def arena(device) -> _Arena:
    key = torch.device(device).index or 0
    a = _ARENAS.get(key)
    if a is None:
        a = _ARENAS[key] = _Arena(device)
    return a


def _rows2d(x: torch.Tensor):
    assert x.dim() == 2 and x.stride(1) == 1, "expected a 2-D tensor with contiguous last dim"
    return x.shape[0], x.shape[1], x.stride(0)


# --------------------------------------------------------------------------- GEMM
def gemm_plan(M: int, N: int, K: int, nranks: int = 1, max_ctas: int = 0) -> _lib.GemmPlan:
    p = _lib.GemmPlan()
    _lib.check(_lib.load().llmss_gemm_plan_query(M, N, K, nranks, 2, max_ctas, C.byref(p)), "gemm_plan_query")
    return p


def linear(x, w, bias=None, act: int = ACT_NONE, gated: bool = False, act_start: int = 0, residual=None,
           out_dtype=None, symm=None, out=None, max_ctas: int = 0, collective: int = 1):
    """``symm``: fuse the tensor-parallel all-reduce into the epilogue.  ``collective``: 1 = library picks the
    exchange (in-switch NVLS reduction from `LLMSS_NVLS_MIN_BYTES` upwards when the workspace is multicast
    bound, else the one-shot Lamport push), 4 = NVLS, 5 = one-shot push."""
    lib = _lib.load()
    M, K, ldx = _rows2d(x)
    N, Kw, ldw = _rows2d(w)
    assert K == Kw, f"linear: x has K={K}, w has K={Kw}"
    assert x.dtype == w.dtype and x.dtype in _DT
    if not (symm is not None and symm.nranks > 1) and _needs_simt(x, w, K, ldx, ldw):
        return linear_simt(x, w, bias, act, gated, act_start, residual, out_dtype, out)
    out_f32 = 1 if out_dtype == torch.float32 else 0
    n_out = N // 2 if gated else N
    if out is None:
        out = torch.empty(M, n_out, dtype=torch.float32 if out_f32 else x.dtype, device=x.device)
    if M == 0:
        return out
    ldr = residual.stride(0) if residual is not None else 0
    ar = symm is not None and symm.nranks > 1
    a = arena(x.device)
    rc = lib.llmss_gemm_ex(_ptr(x), ldx, _ptr(w), ldw, _ptr(bias), _ptr(residual), ldr, _ptr(out), out.stride(0),
                           M, N, K, _DT[x.dtype], out_f32, act, act_start, 1 if gated else 0,
                           _ptr(a.sk_ws), _ptr(a.sk_counters), symm.handle if ar else None, max_ctas,
                           collective if ar else 0, None, _stream())
    _lib.check(rc, "llmss_gemm")
    _count()
    return out


def _needs_simt(x, w, K, ldx, ldw) -> bool:
    """True 32-bit operands, or 16-bit ones that miss the 16-byte rules of the TMA operand loads."""
    if x.dtype == torch.float32:
        return True
    return bool(K % 8 or ldx % 8 or ldw % 8 or x.data_ptr() % 16 or w.data_ptr() % 16)


def linear_simt(x, w, bias=None, act: int = ACT_NONE, gated: bool = False, act_start: int = 0, residual=None,
                out_dtype=None, out=None):
    """The same linear layer on the CUDA cores (csrc/simt_gemm.cu): true 32-bit, or shapes the tcgen05 kernel refuses."""
    if gated:
        raise NotImplementedError("the CUDA-core GEMM has no gated epilogue")
    lib = _lib.load()
    M, K, ldx = _rows2d(x)
    N, _, ldw = _rows2d(w)
    f32 = x.dtype == torch.float32 or out_dtype == torch.float32
    if out is None:
        out = torch.empty(M, N, dtype=torch.float32 if f32 else x.dtype, device=x.device)
    rc = lib.llmss_bgemm_simt(_ptr(x), ldx, 0, _ptr(w), 0, 1, ldw, _ptr(bias), None, 0, _ptr(out), out.stride(0), 0, M, N, K, 1,
                              act, act_start, _DT[x.dtype], 1 if f32 else 0, _stream())
    _lib.check(rc, "llmss_bgemm_simt")
    _count()
    if residual is not None:
        out += residual
    return out


def linear_reduce_scatter(x, w, symm, bias=None, residual_shard=None):
    """K2: row-parallel GEMM whose epilogue reduce-scatters over token rows.  Returns this rank's
    [M / t, N] shard of sum_r(x_r @ w_r.T) (+ bias, + residual_shard)."""
    lib = _lib.load()
    M, K, ldx = _rows2d(x)
    N = w.shape[0]
    rows = M // symm.nranks
    out = torch.empty(rows, N, dtype=x.dtype, device=x.device)
    a = arena(x.device)
    rc = lib.llmss_gemm_ex(_ptr(x), ldx, _ptr(w), w.stride(0), _ptr(bias), _ptr(residual_shard),
                           residual_shard.stride(0) if residual_shard is not None else 0, _ptr(out), out.stride(0),
                           M, N, K, _DT[x.dtype], 0, ACT_NONE, 0, 0, _ptr(a.sk_ws), _ptr(a.sk_counters), symm.handle, 0,
                           2, None, _stream())
    _lib.check(rc, "llmss_gemm_ex(reduce-scatter)")
    _count()
    return out


def allgather_linear(x_shard, w, symm, bias=None, act: int = ACT_NONE, gated: bool = False, act_start: int = 0,
                     out_dtype=None):
    """K3: column-parallel GEMM over the all-gather of the ranks' row shards; the gather is fused into
    the kernel's TMA loads (token tiles are pulled from the owning rank's HBM over NVLink)."""
    lib = _lib.load()
    rows, K, ldx = _rows2d(x_shard)
    M, N = rows * symm.nranks, w.shape[0]
    out_f32 = 1 if out_dtype == torch.float32 else 0
    out = torch.empty(M, N // 2 if gated else N, dtype=torch.float32 if out_f32 else x_shard.dtype, device=x_shard.device)
    a = arena(x_shard.device)
    if a.ag_maps is None:
        a.ag_maps = torch.zeros(2 * 8 * 128 + 64, dtype=torch.uint8, device=x_shard.device)
    maps_ptr = (a.ag_maps.data_ptr() + 63) // 64 * 64
    rc = lib.llmss_gemm_ex(_ptr(x_shard), ldx, _ptr(w), w.stride(0), _ptr(bias), None, 0, _ptr(out), out.stride(0),
                           M, N, K, _DT[x_shard.dtype], out_f32, act, act_start, 1 if gated else 0, _ptr(a.sk_ws),
                           _ptr(a.sk_counters), symm.handle, 0, 3, C.c_void_p(maps_ptr), _stream())
    _lib.check(rc, "llmss_gemm_ex(all-gather)")
    _count()
    return out


# --------------------------------------------------------------------------- norm
def norm_residual(x, residual, weight, bias, eps: float, kind: int, x2=None, write_residual: bool = True):
    lib = _lib.load()
    M, H, ldx = _rows2d(x)
    out = torch.empty(M, H, dtype=x.dtype, device=x.device)
    need_res = write_residual and (residual is not None or x2 is not None)
    new_res = torch.empty(M, H, dtype=x.dtype, device=x.device) if need_res else None
    # the kernel uses one stride for residual in and out
    if residual is not None and new_res is not None and residual.stride(0) != new_res.stride(0):
        residual = residual.contiguous()
    ldr = new_res.stride(0) if new_res is not None else (residual.stride(0) if residual is not None else H)
    rc = lib.llmss_norm_residual(_ptr(x), _ptr(x2), _ptr(residual), _ptr(new_res), _ptr(weight), _ptr(bias), _ptr(out),
                                 M, H, ldx, x2.stride(0) if x2 is not None else H, ldr, out.stride(0), eps, kind,
                                 _DT[x.dtype], _stream())
    _lib.check(rc, "llmss_norm_residual")
    _count()
    return out, (new_res if new_res is not None else x)


# --------------------------------------------------------------------------- rope + kv
def rope_kv_write(qkv, positions, slot_mapping, k_cache, v_cache, hq, hkv, d, rotary_dim, style, base,
                  q_off, k_off, v_off):
    lib = _lib.load()
    T, _, ld = _rows2d(qkv)
    bs = k_cache.shape[2]
    rc = lib.llmss_rope_kv_write(_ptr(qkv), _ptr(positions), _ptr(slot_mapping), _ptr(k_cache), _ptr(v_cache), T, ld,
                                 hq, hkv, d, rotary_dim, style, float(base), q_off, k_off, v_off, bs, _DT[qkv.dtype],
                                 _stream())
    _lib.check(rc, "llmss_rope_kv_write")
    _count()


# --------------------------------------------------------------------------- attention
def decode_splits(B: int, hq: int, hkv: int, d: int, max_kv: int, dtype=torch.bfloat16, block_size: int = 16) -> int:
    """Split-KV factor chosen by the library so the grid fills whole waves of resident CTAs."""
    if d not in (64, 128, 256):
        return 1
    if use_tc_decode(hq, hkv, d, block_size):
        return int(_lib.load().llmss_attn_decode_tc_pick_splits(B, hkv, d, max_kv))
    return int(_lib.load().llmss_attn_decode_pick_splits(B, hq, hkv, d, max_kv, _DT[dtype]))


_TC_MIN_GROUP = int(os.environ.get("LLMSS_ATTN_TC_MIN_GROUP", "4"))


def use_tc_decode(hq: int, hkv: int, d: int, block_size: int = 16) -> bool:
    """tcgen05 decode attention (q heads of a KV group = MMA rows): always with 64-token pages (one TMA op
    per tile: 95 % of HBM peak even for MHA), and for grouped / multi-query models with smaller pages."""
    g = hq // max(hkv, 1)
    if g > 128 or d not in (64, 128, 256) or block_size not in (16, 32, 64):
        return False
    return block_size == 64 or g >= _TC_MIN_GROUP


def attn_decode(q_view, k_cache, v_cache, block_tables, seq_lens, out_view, hq, hkv, d, scale, num_splits, bias_over_scale=None,
                sinks=None):
    """``bias_over_scale`` [hq, n_dist] (tensor-core kernel only): additive score bias per head and key distance.
    ``sinks`` [hq] 32-bit (tensor-core kernel only): a sink logit per head in the softmax denominator."""
    lib = _lib.load()
    B = q_view.shape[0]
    bs = k_cache.shape[2]
    scratch = None
    tc = use_tc_decode(hq, hkv, d, bs)
    if num_splits == 0 and not tc:
        num_splits = 1  # balanced partition exists only in the tensor-core kernel
    if num_splits > 1:
        n = lib.llmss_attn_decode_scratch_floats(B, hq, d, num_splits)
        scratch = arena(q_view.device).attn_scratch(n, q_view.device)
    elif num_splits == 0:
        n = lib.llmss_attn_decode_tc_balanced_scratch_floats(B, hq, d, block_tables.shape[1], bs)
        scratch = arena(q_view.device).attn_scratch(n, q_view.device)
    assert (bias_over_scale is None and sinks is None) or tc, "score bias and sink ride on the tensor-core decode kernel only"
    if tc and sinks is not None:
        rc = lib.llmss_attn_decode_tc_sink(_ptr(q_view), q_view.stride(0), _ptr(k_cache), _ptr(v_cache), _ptr(block_tables),
                                           block_tables.shape[1], _ptr(seq_lens), _ptr(out_view), out_view.stride(0),
                                           _ptr(scratch), B, hq, hkv, d, bs, k_cache.shape[0], float(scale), num_splits,
                                           _DT[q_view.dtype], _ptr(bias_over_scale),
                                           bias_over_scale.shape[1] if bias_over_scale is not None else 0, _ptr(sinks), _stream())
        _lib.check(rc, "llmss_attn_decode_tc_sink")
        _count(1 if num_splits == 1 else 2)
        return
    if tc and bias_over_scale is not None:
        rc = lib.llmss_attn_decode_tc_bias(_ptr(q_view), q_view.stride(0), _ptr(k_cache), _ptr(v_cache), _ptr(block_tables),
                                           block_tables.shape[1], _ptr(seq_lens), _ptr(out_view), out_view.stride(0),
                                           _ptr(scratch), B, hq, hkv, d, bs, k_cache.shape[0], float(scale), num_splits,
                                           _DT[q_view.dtype], _ptr(bias_over_scale), bias_over_scale.shape[1], _stream())
        _lib.check(rc, "llmss_attn_decode_tc_bias")
        _count(1 if num_splits == 1 else 2)
        return
    if tc:
        rc = lib.llmss_attn_decode_tc(_ptr(q_view), q_view.stride(0), _ptr(k_cache), _ptr(v_cache), _ptr(block_tables),
                                      block_tables.shape[1], _ptr(seq_lens), _ptr(out_view), out_view.stride(0),
                                      _ptr(scratch), B, hq, hkv, d, bs, k_cache.shape[0], float(scale), num_splits,
                                      _DT[q_view.dtype], _stream())
        _lib.check(rc, "llmss_attn_decode_tc")
        _count(1 if num_splits == 1 else 2)
        return
    rc = lib.llmss_attn_decode(_ptr(q_view), q_view.stride(0), _ptr(k_cache), _ptr(v_cache), _ptr(block_tables),
                               block_tables.shape[1], _ptr(seq_lens), _ptr(out_view), out_view.stride(0),
                               _ptr(scratch), B, hq, hkv, d, bs, float(scale), num_splits, _DT[q_view.dtype],
                               _stream())
    _lib.check(rc, "llmss_attn_decode")
    _count(2 if num_splits > 1 else 1)


def attn_prefill(q, k, v, out, cu_seqlens, num_seqs, max_seqlen, hq, hkv, d, scale):
    lib = _lib.load()
    rc = lib.llmss_attn_prefill(_ptr(q), q.stride(0), _ptr(k), k.stride(0), _ptr(v), v.stride(0), _ptr(out),
                                out.stride(0), _ptr(cu_seqlens), num_seqs, max_seqlen, q.shape[0], hq, hkv, d,
                                float(scale), _DT[q.dtype], _stream())
    _lib.check(rc, "llmss_attn_prefill")
    _count()


def attn_prefill_paged(q_view, k_cache, v_cache, block_tables, seq_lens, out_view, cu_q, num_seqs, max_q, hq, hkv, d, scale):
    """Multi-token queries over prior context: K / V (this step's included) are read from the paged cache."""
    lib = _lib.load()
    rc = lib.llmss_attn_prefill_paged(_ptr(q_view), q_view.stride(0), _ptr(k_cache), _ptr(v_cache), _ptr(block_tables),
                                      block_tables.shape[1], _ptr(seq_lens), _ptr(out_view), out_view.stride(0), _ptr(cu_q),
                                      num_seqs, max_q, q_view.shape[0], hq, hkv, d, k_cache.shape[2], k_cache.shape[0],
                                      float(scale), _DT[q_view.dtype], _stream())
    _lib.check(rc, "llmss_attn_prefill_paged")
    _count()


# --------------------------------------------------------------------------- embed / sample
def embed(tokens, wte, positions=None, wpe=None, pos_offset: int = 0):
    lib = _lib.load()
    T = tokens.numel()
    V, H = wte.shape
    out = torch.empty(T, H, dtype=wte.dtype, device=wte.device)
    rc = lib.llmss_embed(_ptr(tokens), _ptr(positions), _ptr(wte), _ptr(wpe), _ptr(out), T, H, V,
                         wpe.shape[0] if wpe is not None else 0, pos_offset, out.stride(0), _DT[wte.dtype], _stream())
    _lib.check(rc, "llmss_embed")
    _count()
    return out


def sample(logits, greedy, temperature, top_k, top_p, rng_state, vocab=None, out=None):
    lib = _lib.load()
    B, Vp = logits.shape
    assert logits.dtype == torch.float32 and logits.stride(1) == 1
    if out is None:
        out = torch.empty(B, dtype=torch.int32, device=logits.device)
    o32 = _ptr(out) if out.dtype == torch.int32 else None
    o64 = _ptr(out) if out.dtype == torch.int64 else None
    rc = lib.llmss_sample(_ptr(logits), logits.stride(0), B, vocab or Vp, _ptr(greedy), _ptr(temperature), _ptr(top_k),
                          _ptr(top_p), _ptr(rng_state), o32, o64, _stream())
    _lib.check(rc, "llmss_sample")
    _count()
    return out


def greedy_vocab_parallel(local_logits, symm, vocab: int, out=None):
    """K11 (greedy case): argmax over vocab-sharded fp32 logits [B, V/t] without gathering them.  Every rank
    reduces its shard to one 16-byte (value, global index) candidate per row, the candidates are gathered
    column-wise and merged identically on every rank."""
    lib = _lib.load()
    B, Vb = local_logits.shape
    assert local_logits.dtype == torch.float32 and local_logits.stride(1) == 1
    off = symm.rank * Vb
    n_valid = max(0, min(Vb, vocab - off))
    cand = torch.empty(B, 4, dtype=torch.int32, device=local_logits.device)
    _lib.check(lib.llmss_argmax_local(_ptr(local_logits), local_logits.stride(0), B, n_valid, off, _ptr(cand), _stream()),
               "llmss_argmax_local")
    allc = symm.all_gather_cols(cand)  # [B, t * 4]
    if out is None:
        out = torch.empty(B, dtype=torch.int32, device=local_logits.device)
    o32 = _ptr(out) if out.dtype == torch.int32 else None
    o64 = _ptr(out) if out.dtype == torch.int64 else None
    _lib.check(lib.llmss_argmax_merge(_ptr(allc), symm.nranks, B, o32, o64, _stream()), "llmss_argmax_merge")
    _count(2)
    return out


VP_KS = 128  # candidates a rank contributes per row: exact for 1 <= top_k <= 128 (8 ranks x 128 = the merge's 1024 slots)


def vp_summary(local_logits, n_valid: int, idx_offset: int, greedy, top_k, ks: int = VP_KS, temperature=None):
    """Per-row record of this rank's shard: [max, sum-exp, count, 0, vals[ks], idx[ks]] (fp32 / int32 bits)."""
    lib = _lib.load()
    B = local_logits.shape[0]
    assert local_logits.dtype == torch.float32 and local_logits.stride(1) == 1
    rec = torch.empty(B, 4 + 2 * ks, dtype=torch.float32, device=local_logits.device)
    _lib.check(lib.llmss_vp_summary(_ptr(local_logits), local_logits.stride(0), B, n_valid, idx_offset, _ptr(greedy),
                                    _ptr(top_k), _ptr(temperature), _ptr(rec), ks, _stream()), "llmss_vp_summary")
    _count()
    return rec


def vp_merge_sample(recs_all, nranks: int, vocab: int, greedy, temperature, top_k, top_p, rng_state, out=None,
                    ks: int = VP_KS):
    """recs_all: [B, nranks * (4 + 2 ks)] column-gathered records -> tokens [B]; advances rng_state."""
    lib = _lib.load()
    B = recs_all.shape[0]
    assert recs_all.is_contiguous() and recs_all.shape[1] == nranks * (4 + 2 * ks)
    if out is None:
        out = torch.empty(B, dtype=torch.int32, device=recs_all.device)
    o32 = _ptr(out) if out.dtype == torch.int32 else None
    o64 = _ptr(out) if out.dtype == torch.int64 else None
    _lib.check(lib.llmss_vp_merge_sample(_ptr(recs_all), nranks, ks, B, vocab, _ptr(greedy), _ptr(temperature),
                                         _ptr(top_k), _ptr(top_p), _ptr(rng_state), o32, o64, _stream()),
               "llmss_vp_merge_sample")
    _count()
    return out


def vp_multinomial_pick(local_logits, n_valid: int, idx_offset: int, recs_all, nranks: int, rank: int, greedy, temperature,
                        top_k, top_p, rng_state, ks: int = VP_KS):
    """Whole-distribution rows (top_k = 0, top_p = 1): the rank whose CDF interval holds the draw names the token; every
    other rank (and every other kind of row) answers -1.  Returns [B, 4] int32 (16 bytes per row for the gather)."""
    lib = _lib.load()
    B = local_logits.shape[0]
    cand = torch.empty(B, 4, dtype=torch.int32, device=local_logits.device)
    _lib.check(lib.llmss_vp_multinomial_pick(_ptr(local_logits), local_logits.stride(0), B, n_valid, idx_offset, _ptr(recs_all),
                                             nranks, rank, ks, _ptr(greedy), _ptr(temperature), _ptr(top_k), _ptr(top_p),
                                             _ptr(rng_state), _ptr(cand), _stream()), "llmss_vp_multinomial_pick")
    _count()
    return cand


def vp_multinomial_merge(cand_all, nranks: int, out):
    lib = _lib.load()
    o32 = _ptr(out) if out.dtype == torch.int32 else None
    o64 = _ptr(out) if out.dtype == torch.int64 else None
    _lib.check(lib.llmss_vp_multinomial_merge(_ptr(cand_all), nranks, out.shape[0], o32, o64, _stream()),
               "llmss_vp_multinomial_merge")
    _count()
    return out


def sample_vocab_parallel(local_logits, symm, vocab: int, greedy, temperature, top_k, top_p, rng_state, out=None,
                          whole_distribution_rows: bool = False):
    """K11: top-k / top-p / temperature sampling over vocab-sharded logits [B, V/t] without gathering them
    (reference path: list all_gather of [B, S, V/t] at layers.py:131-135 + rank-0 warpers + broadcast,
    generate.py:109-144).  Three launches: shard summary, 1 KiB-per-row record gather, identical merge + draw; batches
    with whole-distribution rows (top_k = 0, top_p = 1) add the owner pick, a 16-byte-per-row gather and its merge."""
    B, Vb = local_logits.shape
    off = symm.rank * Vb
    n_valid = max(0, min(Vb, vocab - off))
    rec = vp_summary(local_logits, n_valid, off, greedy, top_k, temperature=temperature)
    allr = symm.all_gather_cols(rec)
    cand_all = None
    if whole_distribution_rows:
        cand = vp_multinomial_pick(local_logits, n_valid, off, allr, symm.nranks, symm.rank, greedy, temperature, top_k, top_p,
                                   rng_state)
        cand_all = symm.all_gather_cols(cand)
    out = vp_merge_sample(allr, symm.nranks, vocab, greedy, temperature, top_k, top_p, rng_state, out)
    if cand_all is not None:
        vp_multinomial_merge(cand_all, symm.nranks, out)
    return out


# --------------------------------------------------------------------------- 32-bit residual stream, Dynamic Tanh
def embed_f32(tokens, wte, positions=None, wpe=None, pos_offset: int = 0, scale: float = 1.0, out=None):
    lib = _lib.load()
    T = tokens.numel()
    V, H = wte.shape
    if out is None:
        out = torch.empty(T, H, dtype=torch.float32, device=wte.device)
    assert out.dtype == torch.float32 and out.shape == (T, H) and out.stride(1) == 1 and wte.is_contiguous()
    rc = lib.llmss_embed_scaled_f32(_ptr(tokens), _ptr(positions), _ptr(wte), _ptr(wpe), _ptr(out), T, H, V,
                                    wpe.shape[0] if wpe is not None else 0, pos_offset, out.stride(0), float(scale), _DT[wte.dtype],
                                    _stream())
    _lib.check(rc, "llmss_embed_scaled_f32")
    _count()
    return out


def dyt_residual(resid, alpha, weight, bias, a=None, scale_a=None, b=None, scale_b=None, out_dtype=None, want_norm=True):
    lib = _lib.load()
    M, H, ldr = _rows2d(resid)
    assert resid.dtype == torch.float32 and all(t is None or t.dtype == torch.float32 for t in (a, b))
    dt = out_dtype or weight.dtype
    assert weight.dtype == dt, "dyt_residual: the norm weight has the compute type"
    out = torch.empty(M, H, dtype=dt, device=resid.device) if want_norm else None
    fold = a is not None or b is not None
    new_res = torch.empty_like(resid) if fold else resid
    rc = lib.llmss_dyt_residual(_ptr(resid), _ptr(new_res) if fold else None, _ptr(a), _ptr(scale_a), _ptr(b), _ptr(scale_b),
                                _ptr(weight), _ptr(bias), _ptr(out), float(alpha), M, H, ldr,
                                a.stride(0) if a is not None else 0, b.stride(0) if b is not None else 0,
                                out.stride(0) if out is not None else 0, _DT[dt], _stream())
    _lib.check(rc, "llmss_dyt_residual")
    _count()
    return out, new_res


def cast_concat(a, b, dtype):
    lib = _lib.load()
    M, Ha, lda = _rows2d(a)
    _, Hb, ldb = _rows2d(b)
    out = torch.empty(M, Ha + Hb, dtype=dtype, device=a.device)
    rc = lib.llmss_cast_concat(_ptr(a), _ptr(b), _ptr(out), M, Ha, Hb, lda, ldb, out.stride(0), _DT[dtype], _stream())
    _lib.check(rc, "llmss_cast_concat")
    _count()
    return out


# --------------------------------------------------------------------------- latent attention
def latent_prep(y, q_off, c_off, g_off, n_q, rank, heads, norm_w, eps, slot_mapping, cache, dtype):
    lib = _lib.load()
    T, _, ldy = _rows2d(y)
    assert y.dtype == torch.float32 and cache.dtype == dtype and cache.is_contiguous()
    q = torch.empty(T, n_q, dtype=dtype, device=y.device)
    gate = torch.empty(T, heads, dtype=torch.float32, device=y.device) if g_off >= 0 else None
    rc = lib.llmss_latent_prep(_ptr(y), ldy, q_off, c_off, g_off, n_q, rank, heads, _ptr(norm_w), float(eps), _ptr(slot_mapping),
                               _ptr(cache), _ptr(q), q.stride(0), _ptr(gate), T, _DT[dtype], _stream())
    _lib.check(rc, "llmss_latent_prep")
    _count()
    return q, gate


def heads_matmul(x, w, heads, k, n, w_is_kn, row_scale=None, out_dtype=None, x_head_stride=None, elem_scale=None, out=None,
                 out_head_stride=None):
    lib = _lib.load()
    T, _, ldx = _rows2d(x)
    assert x.dtype == w.dtype and w.is_contiguous() and not (row_scale is not None and elem_scale is not None)
    if out is None:
        f32 = x.dtype == torch.float32 or out_dtype == torch.float32
        out = torch.empty(T, heads * n, dtype=torch.float32 if f32 else x.dtype, device=x.device)
    else:
        f32 = out.dtype == torch.float32
        assert f32 or out.dtype == x.dtype
    assert out.stride(1) == 1
    swh, swk, swn = (k * n, n, 1) if w_is_kn else (n * k, 1, k)
    scale, lds, ssh, ssn = row_scale, (row_scale.stride(0) if row_scale is not None else 0), 1, 0
    if elem_scale is not None:      # one factor per output element: [T, heads * n]
        assert elem_scale.dtype == torch.float32 and elem_scale.stride(1) == 1
        scale, lds, ssh, ssn = elem_scale, elem_scale.stride(0), n, 1
    rc = lib.llmss_bgemm_simt_ex(_ptr(x), ldx, x_head_stride or k, _ptr(w), swh, swk, swn, None, _ptr(scale), lds, ssh, ssn, _ptr(out),
                                 out.stride(0), out_head_stride or n, T, n, k, heads, ACT_NONE, 0, _DT[x.dtype], 1 if f32 else 0,
                                 _stream())
    _lib.check(rc, "llmss_bgemm_simt(heads)")
    _count()
    return out


_LATENT_TC = os.environ.get("LLMSS_LATENT_TC", "1") == "1"


def latent_decode_splits(B: int, heads: int, max_kv: int) -> int:
    """Key-range split of the generic latent kernel for decode: enough CTAs to cover the SMs, at least 256 keys each."""
    ctas = B * -(-heads // 16)
    return int(max(1, min(32, 296 // max(1, ctas), max_kv // 256)))


def _latent_decode_groups(heads: int, rank: int, block_size: int):
    """Head ranges of one tensor-core decode call each: all heads at once where the kernel's query tile holds them, else
    groups of eight (every group reads the latent pages again, which is still far cheaper than the generic kernel)."""
    if not use_tc_decode(heads, 1, rank, block_size) or _lib.load().llmss_attn_decode_tc_supported(heads, 1, rank, block_size):
        return [(0, heads)]
    if not _lib.load().llmss_attn_decode_tc_supported(8, 1, rank, block_size):
        return None
    return [(h, min(8, heads - h)) for h in range(0, heads, 8)]


def latent_attention(q_abs, cache, batch, heads, rank, scale, out_dtype):
    lib = _lib.load()
    T = q_abs.shape[0]
    bs = cache.shape[1]
    dt = cache.dtype
    out = torch.empty(T, heads * rank, dtype=out_dtype, device=q_abs.device)
    if latent_uses_tc(dt, rank, bs, heads) and q_abs.dtype == dt and out_dtype == dt:
        kv = cache.view(cache.shape[0], 1, bs, rank)       # one shared "KV head" that is key and value at once
        if batch.is_decode:
            for h0, n in _latent_decode_groups(heads, rank, bs):
                qv, ov = q_abs[:, h0 * rank:(h0 + n) * rank], out[:, h0 * rank:(h0 + n) * rank]
                splits = batch.decode_splits or decode_splits(batch.num_seqs, n, 1, rank, batch.max_kv, dt, bs)
                attn_decode(qv, kv, kv, batch.block_tables, batch.seq_lens, ov, n, 1, rank, scale, splits)
            return out
        if _lib.has("llmss_attn_prefill_paged"):
            attn_prefill_paged(q_abs, kv, kv, batch.block_tables, batch.seq_lens, out, batch.cu_q, batch.num_seqs, batch.max_q,
                               heads, 1, rank, scale)
            return out
    assert q_abs.dtype == torch.float32, "the generic latent kernel takes 32-bit absorbed queries"
    splits = latent_decode_splits(batch.num_seqs, heads, batch.max_kv) if batch.is_decode else 1
    scratch = None
    if splits > 1:
        scratch = arena(q_abs.device).attn_scratch(lib.llmss_latent_attn_scratch_floats(T, heads, rank, splits), q_abs.device)
    rc = lib.llmss_latent_attn(_ptr(q_abs), q_abs.stride(0), _ptr(cache), _ptr(batch.block_tables), batch.block_tables.shape[1],
                               bs, _ptr(batch.seq_lens), _ptr(batch.cu_q), _ptr(out), out.stride(0), _ptr(scratch), T,
                               batch.num_seqs, batch.max_q, heads, rank, float(scale), splits, _DT[dt], _stream())
    _lib.check(rc, "llmss_latent_attn")
    _count(2 if splits > 1 else 1)
    return out


def latent_uses_tc(dtype, rank: int, block_size: int, heads: int) -> bool:
    """Whether latent_attention() will run on the tcgen05 multi-query kernels (then it wants 16-bit absorbed queries)."""
    if not (_LATENT_TC and dtype != torch.float32 and rank in (64, 128, 256) and block_size in (16, 32, 64) and heads <= 128):
        return False
    # all heads form one query group over the single latent "KV head": the decode kernel must be able to hold that tile,
    # at once or in groups of eight heads
    return _latent_decode_groups(heads, rank, block_size) is not None


# --------------------------------------------------------------------------- routed experts
def moe_route(z, experts, top, groups, keep, route_scale, dense: bool = False, score: str = "softmax", correction=None,
              group_top: int = 1, renorm: bool = True):
    lib = _lib.load()
    T, _, ldz = _rows2d(z)
    assert z.dtype == torch.float32
    ids = torch.empty(T, top, dtype=torch.int32, device=z.device)
    wts = torch.empty(T, top, dtype=torch.float32, device=z.device)
    dn = torch.empty(T, experts, dtype=torch.float32, device=z.device) if dense else None
    assert score in ("softmax", "sigmoid") and (correction is None or (correction.dtype == torch.float32 and correction.numel() == experts))
    rc = lib.llmss_moe_route_ex(_ptr(z), ldz, T, experts, top, groups, keep, float(route_scale), 0 if score == "softmax" else 1,
                                _ptr(correction), int(group_top), 1 if renorm else 0, _ptr(ids), _ptr(wts), _ptr(dn), _stream())
    _lib.check(rc, "llmss_moe_route")
    _count()
    return (ids, wts, dn) if dense else (ids, wts)


def moe_experts(h, ids, wts, w_up, w_down, act, gated: bool = False):
    lib = _lib.load()
    T, W, ldh = _rows2d(h)
    E, F, _ = w_up.shape
    if gated:
        F //= 2       # rows interleave (gate_f, up_f)
    top = ids.shape[1]
    assert w_up.is_contiguous() and w_down.is_contiguous() and h.dtype == w_up.dtype
    scratch = torch.empty(T, top, F, dtype=h.dtype, device=h.device)
    out = torch.empty(T, W, dtype=torch.float32, device=h.device)
    rc = lib.llmss_moe_experts(_ptr(h), ldh, _ptr(ids), _ptr(wts), _ptr(w_up), _ptr(w_down), w_down.stride(0), _ptr(scratch), _ptr(out),
                               out.stride(0), T, W, F, top, act, 1 if gated else 0, _DT[h.dtype], _stream())
    _lib.check(rc, "llmss_moe_experts")
    _count(2)
    return out


def moe_scale(a, dense, experts: int, ff: int):
    lib = _lib.load()
    rc = lib.llmss_moe_scale(_ptr(a), a.stride(0), _ptr(dense), a.shape[0], experts, ff, _DT[a.dtype], _stream())
    _lib.check(rc, "llmss_moe_scale")
    _count()
    return a


def moe_experts_grouped(h, ids, wts, w_up, w_down, act, gated: bool = False):
    """Long prompts: sort the (token, expert) pairs by expert on the device and run every expert as one pair of tensor-core
    GEMMs over its contiguous rows -- top / experts of the dense form's FLOPs.  Reads the per-expert counts on the host (one
    small synchronising copy), so it is for prompt processing, not for graph-captured decode steps."""
    lib = _lib.load()
    T, W, ldh = _rows2d(h)
    E, F, _ = w_up.shape
    if gated:
        F //= 2
    top = ids.shape[1]
    P, dev = T * top, h.device
    counts = torch.empty(E, dtype=torch.int32, device=dev)
    _lib.check(lib.llmss_moe_count(_ptr(ids), P, E, _ptr(counts), _stream()), "llmss_moe_count")
    cnt = counts.tolist()
    offs, o = [], 0
    for c in cnt:
        offs.append(o)
        o += c
    offsets = torch.tensor(offs, dtype=torch.int32).to(dev)
    perm = torch.empty(P, dtype=torch.int32, device=dev)
    inv = torch.empty(P, dtype=torch.int32, device=dev)
    _lib.check(lib.llmss_moe_permute(_ptr(ids), P, E, _ptr(offsets), _ptr(perm), _ptr(inv), _stream()), "llmss_moe_permute")
    xs = torch.empty(P, W, dtype=h.dtype, device=dev)
    _lib.check(lib.llmss_moe_gather_rows(_ptr(h), ldh, _ptr(perm), top, _ptr(xs), P, W, _DT[h.dtype], _stream()),
               "llmss_moe_gather_rows")
    _count(3)
    a = torch.empty(P, F, dtype=h.dtype, device=dev)
    y = torch.empty(P, W, dtype=torch.float32, device=dev)
    for e, (lo, c) in enumerate(zip(offs, cnt)):
        if c:
            linear(xs[lo:lo + c], w_up[e], act=act, gated=gated, out=a[lo:lo + c])
            linear(a[lo:lo + c], w_down[:, e * F:(e + 1) * F], out_dtype=torch.float32, out=y[lo:lo + c])
    out = torch.empty(T, W, dtype=torch.float32, device=dev)
    _lib.check(lib.llmss_moe_combine(_ptr(y), _ptr(inv), _ptr(wts), _ptr(out), out.stride(0), T, W, top, _stream()),
               "llmss_moe_combine")
    _count()
    return out


# --------------------------------------------------------------------------- recurrent layers, post-norm residual
def _f32rows(x):
    assert x.dtype == torch.float32 and x.dim() == 2 and x.stride(1) == 1, "expected a 32-bit 2-D tensor with contiguous rows"
    return x.shape[0], x.shape[1], x.stride(0)


def _bq(batch):
    assert batch.state_slots is not None, "the batch names no state slots"
    return _ptr(batch.cu_q), _ptr(batch.seq_lens), _ptr(batch.state_slots), batch.num_seqs, max(1, batch.max_q)


def embed_bigram(tokens, wte, table, mul_prev, mul_cur, buckets, batch, prev_state):
    lib = _lib.load()
    T = tokens.numel()
    V, W = wte.shape
    assert table.shape[0] > buckets and table.dtype == wte.dtype and wte.is_contiguous() and table.is_contiguous()
    out = torch.empty(T, W, dtype=torch.float32, device=wte.device)
    cu, sl, ss, B, mq = _bq(batch)
    rc = lib.llmss_embed_bigram(_ptr(tokens), _ptr(wte), _ptr(table), _ptr(out), T, W, V, int(mul_prev), int(mul_cur), int(buckets),
                                cu, sl, ss, B, mq, _ptr(prev_state), _DT[wte.dtype], _stream())
    _lib.check(rc, "llmss_embed_bigram")
    _count()
    return out


def postnorm_residual(y, weight, eps, resid=None, y2=None, w_a=None, w_b=None, one_plus=True, out_dtype=None):
    lib = _lib.load()
    T, W, ldy = _f32rows(y)
    dt = out_dtype or torch.float32
    out = torch.empty(T, W, dtype=dt, device=y.device)
    new_res = torch.empty(T, W, dtype=torch.float32, device=y.device) if resid is not None else None
    rc = lib.llmss_postnorm_residual(_ptr(y), ldy, _ptr(y2), y2.stride(0) if y2 is not None else 0, _ptr(w_a), _ptr(w_b), _ptr(weight),
                                     _ptr(resid), resid.stride(0) if resid is not None else 0, _ptr(new_res), _ptr(out), T, W,
                                     float(eps), 1 if one_plus else 0, _DT[dt], _stream())
    _lib.check(rc, "llmss_postnorm_residual")
    _count()
    return out, new_res


def token_shift(x, mu, batch, prev_state, out_dtype=None):
    lib = _lib.load()
    T, W, ldx = _f32rows(x)
    S = mu.shape[0]
    dt = out_dtype or torch.float32
    out = torch.empty(S, T, W, dtype=dt, device=x.device)
    cu, sl, ss, B, mq = _bq(batch)
    rc = lib.llmss_token_shift(_ptr(x), ldx, _ptr(mu), S, _ptr(out), T, W, cu, sl, ss, B, mq, _ptr(prev_state), _DT[dt], _stream())
    _lib.check(rc, "llmss_token_shift")
    _count()
    return out


def causal_conv(u, w, bias, act, batch, state, out_dtype=None):
    lib = _lib.load()
    T, C, ldu = _f32rows(u)
    assert w.dtype == torch.float32 and w.is_contiguous() and w.shape[0] == C
    dt = out_dtype or torch.float32
    out = torch.empty(T, C, dtype=dt, device=u.device)
    cu, sl, ss, B, mq = _bq(batch)
    rc = lib.llmss_causal_conv_to(_ptr(u), ldu, _ptr(w), _ptr(bias), _ptr(out), _DT[dt], T, C, w.shape[1], act, cu, sl, ss, B, mq,
                                  _ptr(state), _stream())
    _lib.check(rc, "llmss_causal_conv")
    _count()
    return out


def unary(x, op, out_dtype=None):
    lib = _lib.load()
    T, C, ldx = _f32rows(x)
    dt = out_dtype or torch.float32
    out = torch.empty(T, C, dtype=dt, device=x.device)
    _lib.check(lib.llmss_unary_f32(_ptr(x), ldx, _ptr(out), T, C, op, _DT[dt], _stream()), "llmss_unary_f32")
    _count()
    return out


def ssm_dt(dt_raw, dt_bias, a_log):
    lib = _lib.load()
    T, H, ldr = _f32rows(dt_raw)
    dt = torch.empty(T, H, dtype=torch.float32, device=dt_raw.device)
    ld = torch.empty(T, H, dtype=torch.float32, device=dt_raw.device)
    _lib.check(lib.llmss_ssm_dt(_ptr(dt_raw), ldr, _ptr(dt_bias), _ptr(a_log), _ptr(dt), _ptr(ld), T, H, _stream()), "llmss_ssm_dt")
    _count()
    return dt, ld


_SCAN_CHUNK = int(os.environ.get("LLMSS_SCAN_CHUNK", "128"))          # tokens per chunk of the two-pass recurrence
_SCAN_CHUNK_MIN = int(os.environ.get("LLMSS_SCAN_CHUNK_MIN", "256"))   # portions from this length on run in two passes


def linear_scan(q, k, v, decay, decay_kind, batch, state, heads, qk_heads, dk, dv, bonus=None, v_scale=None, read_before=False):
    lib = _lib.load()
    T, _, ldv = _f32rows(v)
    _, _, ldq = _f32rows(q)
    _, _, ldk = _f32rows(k)
    assert decay.dtype == torch.float32 and state.dtype == torch.float32 and state.is_contiguous()
    out = torch.empty(T, heads * dv, dtype=torch.float32, device=v.device)
    cu, sl, ss, B, mq = _bq(batch)
    # long portions of few sequences: two passes over chunks, every chunk a block (a recurrence is a chain per token)
    chunk, scratch = 0, None
    if mq >= _SCAN_CHUNK_MIN and not torch.cuda.is_current_stream_capturing():
        chunk = _SCAN_CHUNK
        scratch = torch.empty(lib.llmss_linear_scan_scratch_floats(B, heads, dk, dv, mq, chunk), dtype=torch.float32, device=v.device)
    rc = lib.llmss_linear_scan(_ptr(q), ldq, _ptr(k), ldk, _ptr(v), ldv, _ptr(decay), decay.stride(0) if decay.dim() == 2 else 0,
                               decay_kind, _ptr(bonus), _ptr(v_scale), v_scale.stride(0) if v_scale is not None else 0, _ptr(out),
                               _ptr(state), cu, sl, ss, B, heads, qk_heads, dk, dv, 1 if read_before else 0, _ptr(scratch), chunk, mq,
                               _stream())
    _lib.check(rc, "llmss_linear_scan")
    _count(2 if chunk else 1)
    return out


_INV_FREQ = {}


def _inv_freq(W: int, base: float, device):
    """64-bit inverse frequencies base^(-2 i / W), i = 0 .. ceil(W / 2) - 1, kept per (width, base, device)."""
    key = (W, float(base), str(device))
    t = _INV_FREQ.get(key)
    if t is None:
        i = torch.arange((W + 1) // 2, dtype=torch.float64)
        t = _INV_FREQ[key] = torch.pow(torch.tensor(float(base), dtype=torch.float64), -(2.0 * i) / W).to(device)
    return t


def embed_sinusoid(tokens, wte, scale, positions, streams=1, base=10000.0):
    lib = _lib.load()
    T = tokens.numel()
    V, W = wte.shape
    assert wte.is_contiguous()
    out = torch.empty(streams, T, W, dtype=torch.float32, device=wte.device)
    rc = lib.llmss_embed_sinusoid(_ptr(tokens), _ptr(positions), _ptr(wte), _ptr(_inv_freq(W, base, wte.device)), _ptr(out), T, W, V,
                                  float(scale), int(streams), _DT[wte.dtype], _stream())
    _lib.check(rc, "llmss_embed_sinusoid")
    _count()
    return out


def hyper_residual(xs, y=None, mix=None, w_out=None, w_in=None, norm_w=None, eps=0.0, out_dtype=None):
    lib = _lib.load()
    assert xs.dtype == torch.float32 and xs.dim() == 3 and xs.is_contiguous()
    S, T, W = xs.shape
    ldy = 0
    if y is not None:
        _, Wy, ldy = _f32rows(y)
        assert Wy == W and mix.dtype == torch.float32 and mix.is_contiguous() and mix.shape == (S, S) and w_out.numel() == S
    dt = out_dtype or torch.float32
    out = torch.empty(T, W, dtype=dt, device=xs.device) if w_in is not None else None
    rc = lib.llmss_hyper_residual(_ptr(xs), T, W, S, _ptr(y), ldy, _ptr(mix), _ptr(w_out), _ptr(w_in), _ptr(norm_w), float(eps), _ptr(out),
                                  _DT[dt], _stream())
    _lib.check(rc, "llmss_hyper_residual")
    _count()
    return out


def delta_scan(q, k, v, log_decay, beta, batch, state, heads, qk_heads, dk, dv, unit_eps=None, q_scale=1.0, beta_sigmoid=False):
    lib = _lib.load()
    T, _, ldv = _f32rows(v)
    _, _, ldq = _f32rows(q)
    _, _, ldk = _f32rows(k)
    _, _, ldg = _f32rows(log_decay)
    _, _, ldb = _f32rows(beta)
    assert state.dtype == torch.float32 and state.is_contiguous() and state[0].numel() == heads * dk * dv
    out = torch.empty(T, heads * dv, dtype=torch.float32, device=v.device)
    cu, sl, ss, B, mq = _bq(batch)
    rc = lib.llmss_delta_scan(_ptr(q), ldq, _ptr(k), ldk, _ptr(v), ldv, _ptr(log_decay), ldg, _ptr(beta), ldb, _ptr(out), _ptr(state),
                              cu, sl, ss, B, mq, heads, qk_heads, dk, dv, -1.0 if unit_eps is None else float(unit_eps), float(q_scale),
                              1 if beta_sigmoid else 0, _stream())
    _lib.check(rc, "llmss_delta_scan")
    _count()
    return out


def gated_rmsnorm(o, gate, gate_act, weight, groups, eps, gate_first, skip_x=None, skip_d=None, out_dtype=None):
    lib = _lib.load()
    T, C, ldo = _f32rows(o)
    dt = out_dtype or torch.float32
    out = torch.empty(T, C, dtype=dt, device=o.device)
    rc = lib.llmss_gated_rmsnorm(_ptr(o), ldo, _ptr(gate), gate.stride(0) if gate is not None else 0, gate_act, _ptr(weight), groups,
                                 float(eps), 1 if gate_first else 0, _ptr(skip_x), skip_x.stride(0) if skip_x is not None else 0,
                                 _ptr(skip_d), skip_d.numel() if skip_d is not None else 0, _ptr(out), T, C, _DT[dt], _stream())
    _lib.check(rc, "llmss_gated_rmsnorm")
    _count()
    return out


def qknorm_kv_write(qkv, hq, hkv, dk, dv, q_w, k_w, eps, temp_coef, temp_every, positions, slot_mapping, k_cache, v_cache,
                    out_dtype=None, norm_whole=False, v_norm=False, q_head_scale=None):
    lib = _lib.load()
    T, _, ld = _f32rows(qkv)
    dt = out_dtype or k_cache.dtype
    if hkv > 0:
        assert k_cache.dtype == dt and v_cache.dtype == dt and k_cache.is_contiguous() and v_cache.is_contiguous()
    q = torch.empty(T, hq * dk, dtype=dt, device=qkv.device)
    if norm_whole or v_norm or q_head_scale is not None or hkv == 0:
        # the general kernel (one CTA per token): norms over a token's whole projection, value norm, per-head factor, queries only
        assert q_w.numel() == (hq * dk if norm_whole else dk) and (hkv == 0 or k_w.numel() == (hkv * dk if norm_whole else dk))
        rc = lib.llmss_qkv_prepare(_ptr(qkv), ld, hq, hkv, dk, dv, _ptr(q_w), _ptr(k_w), float(eps), float(temp_coef), int(temp_every),
                                   _ptr(q_head_scale), 1 if norm_whole else 0, 1 if v_norm else 0, _ptr(positions), _ptr(slot_mapping),
                                   _ptr(k_cache), _ptr(v_cache), k_cache.shape[2] if hkv > 0 else 1, _ptr(q), T, _DT[dt], _stream())
        _lib.check(rc, "llmss_qkv_prepare")
        _count()
        return q
    rc = lib.llmss_qknorm_kv_write(_ptr(qkv), ld, hq, hkv, dk, dv, _ptr(q_w), _ptr(k_w), float(eps), float(temp_coef), int(temp_every),
                                   _ptr(positions), _ptr(slot_mapping), _ptr(k_cache), _ptr(v_cache), k_cache.shape[2], _ptr(q), T,
                                   _DT[dt], _stream())
    _lib.check(rc, "llmss_qknorm_kv_write")
    _count()
    return q


_BIAS_TC = os.environ.get("LLMSS_ATTN_BIAS_TC", "1") == "1"


def _bias_over_scale(dist_bias, scale, given=None):
    """The distance table in the units of the raw scores (the tensor-core kernels add it before their one multiply).  Callers
    that keep the table (a model layer) pass it as ``given``; otherwise it is derived per call."""
    if given is not None:
        return given
    return (dist_bias.float() / float(scale)).contiguous()


def attention_bias_uses_tc(dtype, dk: int, dv: int, block_size: int, scale: float) -> bool:
    """16-bit pages with equal key and value size 64 / 128 / 256 run on the tcgen05 paged flash kernel (bias and gate
    instantiation); everything else -- true 32-bit, other or unequal sizes -- on the generic kernel."""
    return (_BIAS_TC and dtype != torch.float32 and dk == dv and dk in (64, 128, 256) and block_size in (16, 32, 64) and scale > 0
            and _lib.has("llmss_attn_prefill_paged_bias"))


from .reference import window_bias_table  # noqa: E402  (the window and slopes as a distance table)


def attention_bias(q, k_cache, v_cache, batch, hq, hkv, dk, dv, scale, dist_bias, gate=None, out_dtype=None, bias_over_scale=None,
                   window=0, slopes=None, sinks=None):
    lib = _lib.load()
    T = q.shape[0]
    dt = q.dtype
    assert k_cache.dtype == dt and (out_dtype or dt) == dt and q.stride(1) == 1
    out = torch.empty(T, hq * dv, dtype=dt, device=q.device)
    if sinks is not None:
        assert sinks.dtype == torch.float32 and sinks.numel() == hq
        bs = k_cache.shape[2]
        if (dist_bias is None and not window and slopes is None and gate is None and _lib.has("llmss_attn_prefill_paged_sink")
                and attention_bias_uses_tc(dt, dk, dv, bs, scale) and q.data_ptr() % 16 == 0 and q.stride(0) % 8 == 0):
            # 16-bit pages of a tensor-core size: the sink joins the final normalisation of the tcgen05 kernels
            if (batch.is_decode and _lib.has("llmss_attn_decode_tc_sink") and use_tc_decode(hq, hkv, dk, bs)
                    and lib.llmss_attn_decode_tc_supported(hq, hkv, dk, bs)):
                splits = batch.decode_splits or decode_splits(batch.num_seqs, hq, hkv, dk, batch.max_kv, dt, bs)
                attn_decode(q, k_cache, v_cache, batch.block_tables, batch.seq_lens, out, hq, hkv, dk, scale, splits, sinks=sinks)
                return out
            rc = lib.llmss_attn_prefill_paged_sink(_ptr(q), q.stride(0), _ptr(k_cache), _ptr(v_cache), _ptr(batch.block_tables),
                                                   batch.block_tables.shape[1], _ptr(batch.seq_lens), _ptr(out), out.stride(0),
                                                   _ptr(batch.cu_q), batch.num_seqs, max(1, batch.max_q), T, hq, hkv, dk, bs,
                                                   k_cache.shape[0], float(scale), _DT[dt], None, 0, None, 0, _ptr(sinks), _stream())
            _lib.check(rc, "llmss_attn_prefill_paged_sink")
            _count()
            return out
        # everything else: the generic kernel (any sizes, true 32-bit; 32-bit scores, softmax and accumulation)
        rc = lib.llmss_attention_sink(_ptr(q), q.stride(0), _ptr(k_cache), _ptr(v_cache), _ptr(batch.block_tables),
                                      batch.block_tables.shape[1], k_cache.shape[2], _ptr(batch.seq_lens), _ptr(batch.cu_q),
                                      _ptr(dist_bias), dist_bias.shape[1] if dist_bias is not None else 0, _ptr(slopes),
                                      int(window or 0), _ptr(gate), gate.stride(0) if gate is not None else 0, _ptr(sinks), _ptr(out),
                                      batch.num_seqs, max(1, batch.max_q), hq, hkv, dk, dv, float(scale), _DT[dt], _stream())
        _lib.check(rc, "llmss_attention_sink")
        _count()
        return out
    tc_ok = attention_bias_uses_tc(dt, dk, dv, k_cache.shape[2], scale) and q.data_ptr() % 16 == 0 and q.stride(0) % 8 == 0
    table = None
    if window or slopes is not None:
        # 16-bit pages of a tensor-core size with a window: the window and the slopes become a distance table whose last column
        # hides the key (kept by the layer as ``bias_over_scale``, else derived here).  Everything else -- true 32-bit, other or
        # unequal sizes, slopes without a window -- runs the generic kernel, whose key loop starts at the window.
        if tc_ok and dist_bias is None and window and slopes is not None:
            table = bias_over_scale if bias_over_scale is not None else window_bias_table(slopes, int(window), scale)
            assert table.shape == (hq, int(window) + 1)
        else:
            rc = lib.llmss_attention_window(_ptr(q), q.stride(0), _ptr(k_cache), _ptr(v_cache), _ptr(batch.block_tables),
                                            batch.block_tables.shape[1], k_cache.shape[2], _ptr(batch.seq_lens), _ptr(batch.cu_q),
                                            _ptr(dist_bias), dist_bias.shape[1] if dist_bias is not None else 0, _ptr(slopes),
                                            int(window or 0), _ptr(gate), gate.stride(0) if gate is not None else 0, _ptr(out),
                                            batch.num_seqs, max(1, batch.max_q), hq, hkv, dk, dv, float(scale), _DT[dt], _stream())
            _lib.check(rc, "llmss_attention_window")
            _count()
            return out
    elif dist_bias is not None and tc_ok:
        table = _bias_over_scale(dist_bias, scale, bias_over_scale)
    if table is not None:
        bs = k_cache.shape[2]
        if (batch.is_decode and _lib.has("llmss_attn_decode_tc_bias") and use_tc_decode(hq, hkv, dk, bs)
                and lib.llmss_attn_decode_tc_supported(hq, hkv, dk, bs)):
            # one query per sequence: the split-KV decode kernel (the q heads of a group are its MMA rows), then the gate
            splits = batch.decode_splits or decode_splits(batch.num_seqs, hq, hkv, dk, batch.max_kv, dt, bs)
            attn_decode(q, k_cache, v_cache, batch.block_tables, batch.seq_lens, out, hq, hkv, dk, scale, splits,
                        bias_over_scale=table)
            if gate is not None:
                _lib.check(lib.llmss_head_gate(_ptr(out), out.stride(0), _ptr(gate), gate.stride(0), T, hq, dv, _DT[dt], _stream()),
                           "llmss_head_gate")
                _count()
            return out
        rc = lib.llmss_attn_prefill_paged_bias(_ptr(q), q.stride(0), _ptr(k_cache), _ptr(v_cache), _ptr(batch.block_tables),
                                               batch.block_tables.shape[1], _ptr(batch.seq_lens), _ptr(out), out.stride(0),
                                               _ptr(batch.cu_q), batch.num_seqs, max(1, batch.max_q), T, hq, hkv, dk,
                                               k_cache.shape[2], k_cache.shape[0], float(scale), _DT[dt], _ptr(table), table.shape[1],
                                               _ptr(gate), gate.stride(0) if gate is not None else 0, _stream())
        _lib.check(rc, "llmss_attn_prefill_paged_bias")
        _count()
        return out
    rc = lib.llmss_attention_bias(_ptr(q), q.stride(0), _ptr(k_cache), _ptr(v_cache), _ptr(batch.block_tables),
                                  batch.block_tables.shape[1], k_cache.shape[2], _ptr(batch.seq_lens), _ptr(batch.cu_q),
                                  _ptr(dist_bias), dist_bias.shape[1] if dist_bias is not None else 0, _ptr(gate),
                                  gate.stride(0) if gate is not None else 0, _ptr(out), batch.num_seqs, max(1, batch.max_q), hq, hkv,
                                  dk, dv, float(scale), _DT[dt], _stream())
    _lib.check(rc, "llmss_attention_bias")
    _count()
    return out


# --------------------------------------------------------------------------- rotation by a table, sandwich norms
_FREQ_DEV = {}


def _freq_dev(freq, device):
    """The 64-bit frequency table on the device: the caller's own tensor if it lives there (a layer keeps its table), else a copy
    kept per (table, device) for the life of the process (a captured graph points at it)."""
    if freq.is_cuda and freq.dtype == torch.float64 and freq.is_contiguous():
        return freq
    key = (tuple(freq.tolist()), str(device))
    t = _FREQ_DEV.get(key)
    if t is None:
        t = _FREQ_DEV[key] = freq.to(torch.float64).to(device).contiguous()
    return t


def rope_norm_kv_write(qk, hq, hkv, d, freq, mag, interleaved, unit_norm, eps, positions, slot_mapping, k_cache, v_cache, out_dtype=None):
    lib = _lib.load()
    T, _, ld = _f32rows(qk)
    dt = out_dtype or k_cache.dtype
    assert k_cache.dtype == dt and v_cache.dtype == dt and k_cache.is_contiguous() and v_cache.is_contiguous()
    assert k_cache.shape[1:] == (hkv, k_cache.shape[2], d) and v_cache.shape == k_cache.shape
    q = torch.empty(T, hq * d, dtype=dt, device=qk.device)
    rc = lib.llmss_rope_norm_kv_write(_ptr(qk), ld, hq, hkv, d, _ptr(_freq_dev(freq, qk.device)), freq.numel(), float(mag),
                                      1 if interleaved else 0, 1 if unit_norm else 0, float(eps), _ptr(positions), _ptr(slot_mapping),
                                      _ptr(k_cache), _ptr(v_cache), k_cache.shape[2], _ptr(q), T, _DT[dt], _stream())
    _lib.check(rc, "llmss_rope_norm_kv_write")
    _count()
    return q


def latent_rope_prep(y, q_off, q_rank, c_off, rank, rot, g_off, n_gate, qn_w, cn_w, eps, freq, mag, positions, slot_mapping, cache, dtype):
    lib = _lib.load()
    T, _, ldy = _f32rows(y)
    assert cache.dtype == dtype and cache.is_contiguous() and cn_w.dtype == torch.float32 and (q_rank == 0 or qn_w.dtype == torch.float32)
    cq = torch.empty(T, q_rank, dtype=dtype, device=y.device) if q_rank > 0 else None
    gate = torch.empty(T, n_gate, dtype=torch.float32, device=y.device) if n_gate > 0 else None
    rc = lib.llmss_latent_rope_prep(_ptr(y), ldy, q_off, q_rank, c_off, rank, rot, g_off, n_gate, _ptr(qn_w), _ptr(cn_w), float(eps),
                                    _ptr(_freq_dev(freq, y.device)), freq.numel(), float(mag), _ptr(positions), _ptr(slot_mapping),
                                    _ptr(cache), cache.shape[-1], _ptr(cq), _ptr(gate), T, _DT[dtype], _stream())
    _lib.check(rc, "llmss_latent_rope_prep")
    _count()
    return cq, gate


def latent_query_rope(q, heads, d, rot, rank, width, freq, mag, positions, dtype, abs_dtype):
    lib = _lib.load()
    T, _, ldq = _f32rows(q)
    assert abs_dtype in (torch.float32, dtype)
    q_nope = torch.empty(T, heads * d, dtype=dtype, device=q.device)
    q_abs = torch.empty(T, heads * width, dtype=abs_dtype, device=q.device)
    rc = lib.llmss_latent_query_rope(_ptr(q), ldq, heads, d, rot, rank, width, _ptr(_freq_dev(freq, q.device)), freq.numel(), float(mag),
                                     _ptr(positions), _ptr(q_nope), _ptr(q_abs), 1 if abs_dtype == torch.float32 else 0, T, _DT[dtype],
                                     _stream())
    _lib.check(rc, "llmss_latent_query_rope")
    _count()
    return q_nope, q_abs


def hgrn_gates(y, n_qk, lower):
    lib = _lib.load()
    T, C, ldy = _f32rows(y)
    assert C >= 2 * n_qk and lower.dtype == torch.float32 and lower.numel() == n_qk
    q, k, lnf = (torch.empty(T, n_qk, dtype=torch.float32, device=y.device) for _ in range(3))
    _lib.check(lib.llmss_hgrn_gates(_ptr(y), ldy, n_qk, _ptr(lower), _ptr(q), _ptr(k), _ptr(lnf), T, _stream()), "llmss_hgrn_gates")
    _count()
    return q, k, lnf


def sandwich_residual(resid, y, w_post, eps, w_next=None, history=None, index=0, depth_w=None, out_dtype=None):
    lib = _lib.load()
    T, W, ldr = _f32rows(resid)
    ldy = 0
    if y is not None:
        _, Wy, ldy = _f32rows(y)
        assert Wy == W and w_post.dtype == torch.float32 and w_post.numel() == W
    if history is not None:
        assert history.dtype == torch.float32 and history.is_contiguous() and history.shape[1:] == (T, W) and index < history.shape[0]
        assert depth_w is None or (depth_w.dtype == torch.float32 and depth_w.numel() >= index + 1)
    dt = out_dtype or torch.float32
    out_r = torch.empty(T, W, dtype=torch.float32, device=resid.device)
    out_h = torch.empty(T, W, dtype=dt, device=resid.device) if w_next is not None else None
    assert w_next is None or (w_next.dtype == torch.float32 and w_next.numel() == W)
    rc = lib.llmss_sandwich_residual(_ptr(resid), ldr, _ptr(y), ldy, _ptr(w_post), _ptr(history), int(index),
                                     _ptr(depth_w) if history is not None else None, _ptr(w_next), _ptr(out_r), _ptr(out_h), T, W,
                                     float(eps), _DT[dt], _stream())
    _lib.check(rc, "llmss_sandwich_residual")
    _count()
    return out_h, out_r


def softcap(z, cap):
    lib = _lib.load()
    assert z.dtype == torch.float32 and z.dim() == 2 and z.stride(1) == 1
    _lib.check(lib.llmss_softcap(_ptr(z), z.stride(0), z.shape[0], z.shape[1], float(cap), _stream()), "llmss_softcap")
    _count()
    return z

"""Op front door: CPU tensors run the fp32 PyTorch oracles (ops.reference), CUDA tensors run
the hand-written sm_100a kernels (ops.cuda_impl -> libllmss_b200.so).  There is no silent
fallback on CUDA: a missing library or an unsupported shape raises.

The only library (non-hand-written) kernel still reachable on the CUDA path is the
``generic`` attention fallback used for prefill-with-prior-context (chunked prefill /
HF-compat forward with a multi-token query and a non-empty cache); see attention().
"""
from __future__ import annotations

import os
from typing import Optional

import torch

from . import reference as ref
from .reference import (DECAY_HEAD, DECAY_TOKEN_CHANNEL, DECAY_TOKEN_HEAD, GATE_NONE, GATE_SIGMOID, GATE_SILU, UNARY_NEG_EXP,
                        UNARY_TANH, distance_bias_table, rotary_frequencies, window_bias_table)
from .reference import (ACT_GELU_ERF, ACT_GELU_TANH, ACT_IDS, ACT_NONE, ACT_RELU, ACT_RELU2, ACT_SILU, NORM_DYT, NORM_LAYER,
                        NORM_RMS, ROPE_GPTJ, ROPE_NEOX, ROPE_NONE)


def _cuda(t: torch.Tensor) -> bool:
    return t.is_cuda


_WARNED = set()


def _warn_once(msg: str):
    if msg not in _WARNED:
        _WARNED.add(msg)
        from ..utils.logging import logger

        logger.warning(msg)


_FUSED_PUSH_MAX = int(os.environ.get("LLMSS_FUSED_AR_MAX_PUSH", str(2 << 20)))
_TWOSHOT_MIN = int(os.environ.get("LLMSS_TWOSHOT_MIN_BYTES", str(256 << 10)))
_FUSED_TWOSHOT_MAX = int(os.environ.get("LLMSS_FUSED_TWOSHOT_MAX_BYTES", str(8 << 20)))


def _fused_ar_mode(cu, symm, M: int, N: int, K: int, esz: int) -> int:
    """How a row-parallel GEMM on CUDA performs its all-reduce: 0 = plain GEMM followed by the standalone
    collective, 5 = one-shot Lamport push in the epilogue, 6 = two-shot Lamport exchange in the epilogue
    (reduce-scatter by peer stores, result broadcast by one NVSwitch multicast store).

    Only the cluster split-K kernel fuses (each CTA owns a slice of one tile); shapes that run on the stream-K
    kernel measured slower fused than unfused.  The one-shot push is one hop but puts (t-1) x the message on
    the wire, the two-shot form two hops and ~1 x: from 4 ranks and `LLMSS_TWOSHOT_MIN_BYTES` upwards the
    latter wins (profiles/bench_gemm_ar.md).  The flag-synchronised in-switch reduction (mode 4,
    multimem.ld_reduce) costs ~15 us of latency and is left to the standalone collective for prefill sizes."""
    plan = cu.gemm_plan(M, N, K, symm.nranks)
    if plan.split <= 0 or plan.tiles > 2048:
        return 0
    msg = M * N * esz
    padded = plan.tiles * 128 * plan.bn * esz
    two_fits = padded <= _FUSED_TWOSHOT_MAX and (symm.nranks + 1) * padded <= symm.lam_bytes
    if two_fits and ((symm.nranks >= 4 and msg >= _TWOSHOT_MIN) or msg >= (1 << 20)):
        return 6   # measured: from 256 KB at 4+ ranks, from 1 MB even at 2 ranks (profiles/bench_gemm_ar.md)
    if plan.ar_bytes <= symm.lam_bytes and msg * (symm.nranks - 1) <= _FUSED_PUSH_MAX:
        return 5
    return 0


def linear(x, w, bias=None, act: int = ACT_NONE, gated: bool = False, act_start: int = 0, residual=None,
           out_dtype=None, comm=None):
    """y = epilogue(x @ w.T); with ``comm`` the product is summed over the TP group first
    (row-parallel layer: reference `TensorParallelRowLinear.forward`, layers.py:175-179) and
    bias/residual are applied once after the reduction."""
    reduce = comm is not None and not comm.single
    if _cuda(x):
        from . import cuda_impl as cu

        if not reduce:
            return cu.linear(x, w, bias, act, gated, act_start, residual, out_dtype)
        symm = comm.symm
        if symm is not None:
            mode = _fused_ar_mode(cu, symm, x.shape[0], w.shape[0], x.shape[1], x.element_size())
            if mode:
                return cu.linear(x, w, bias, ACT_NONE, False, 0, residual, None, symm=symm, collective=mode)
        y = cu.linear(x, w, None, ACT_NONE, False, 0, None, None)
        comm.all_reduce(y)
        if bias is not None:
            y = y + bias
        if residual is not None:
            y = y + residual
        return y
    if not reduce:
        return ref.linear(x, w, bias, act, gated, act_start, residual, out_dtype)
    y = ref.linear(x, w, None, ACT_NONE, False, 0, None, torch.float32)
    comm.all_reduce(y)
    if bias is not None:
        y = y + bias.float()
    if residual is not None:
        y = y + residual.float()
    return y.to(out_dtype or x.dtype)


def norm_residual(x, residual, weight, bias, eps: float, kind: int, x2=None):
    """Returns (norm(x [+x2] [+residual]), the pre-norm sum)."""
    if _cuda(x):
        from . import cuda_impl as cu

        return cu.norm_residual(x, residual, weight, bias, eps, kind, x2=x2)
    if x2 is not None:
        x = (x.float() + x2.float()).to(x.dtype)
    return ref.norm_residual(x, residual, weight, bias, eps, kind)


def rope_kv_write(qkv, positions, slot_mapping, k_cache, v_cache, hq, hkv, d, rotary_dim, style, base,
                  q_off, k_off, v_off):
    if _cuda(qkv):
        from . import cuda_impl as cu

        return cu.rope_kv_write(qkv, positions, slot_mapping, k_cache, v_cache, hq, hkv, d, rotary_dim, style, base,
                                q_off, k_off, v_off)
    return ref.rope_kv_write(qkv, positions, slot_mapping, k_cache, v_cache, hq, hkv, d, rotary_dim, style, base,
                             q_off, k_off, v_off)


def attention(qkv, out, batch, k_cache, v_cache, hq, hkv, d, scale, q_off, k_off, v_off, out_off=0):
    """Causal attention for a packed batch; writes ``out[:, out_off : out_off + hq*d]``.

    decode batches (one query per sequence) -> split-KV paged kernel (K9);
    fresh prefill (no prior context)        -> varlen causal prefill kernel (K8);
    multi-token queries over prior context  -> the same kernel in paged mode (K / V from the cache);
    unsupported head sizes / page sizes     -> generic gather path (oracle math).
    """
    T = qkv.shape[0]
    q_view = qkv[:, q_off:q_off + hq * d]
    out_view = out[:, out_off:out_off + hq * d]
    if _cuda(qkv):
        from . import cuda_impl as cu

        if d not in (64, 128, 256):
            _warn_once(f"head_dim={d} has no sm_100a attention kernel (64/128/256 do); using the generic PyTorch path")
        elif batch.is_decode:
            splits = batch.decode_splits or cu.decode_splits(batch.num_seqs, hq, hkv, d, batch.max_kv, qkv.dtype,
                                                                     k_cache.shape[2])
            cu.attn_decode(q_view, k_cache, v_cache, batch.block_tables, batch.seq_lens, out_view, hq, hkv, d, scale,
                           splits)
            return out
        elif batch.is_fresh_prefill and cu._lib.has("llmss_attn_prefill"):
            cu.attn_prefill(q_view, qkv[:, k_off:k_off + hkv * d], qkv[:, v_off:v_off + hkv * d], out_view,
                            batch.cu_q, batch.num_seqs, batch.max_q, hq, hkv, d, scale)
            return out
        elif (not batch.is_fresh_prefill and k_cache.shape[2] in (16, 32, 64) and k_cache.is_contiguous()
              and v_cache.is_contiguous() and cu._lib.has("llmss_attn_prefill_paged")):
            # multi-token queries over prior context (chunked prefill, HF-style forward with a past): same tcgen05
            # flash kernel, K / V tiles gathered page by page from the cache through the block table
            cu.attn_prefill_paged(q_view, k_cache, v_cache, batch.block_tables, batch.seq_lens, out_view, batch.cu_q,
                                  batch.num_seqs, batch.max_q, hq, hkv, d, scale)
            return out
        elif batch.is_fresh_prefill:
            # LIBRARY FALLBACK (torch SDPA), only reached when the own prefill kernel is absent from
            # the loaded library or the head_dim is unsupported by it.
            _sdpa_prefill(qkv, out_view, batch, hq, hkv, d, scale, q_off, k_off, v_off)
            return out
    o = ref.attention_paged(q_view.reshape(T, hq, d), k_cache, v_cache, batch.block_tables, batch.seq_lens,
                            batch.cu_q, scale)
    out_view.copy_(o.reshape(T, hq * d))
    return out


def _sdpa_prefill(qkv, out_view, batch, hq, hkv, d, scale, q_off, k_off, v_off):
    import torch.nn.functional as F

    cu = batch.cu_q.tolist()
    for i in range(batch.num_seqs):
        a, b = cu[i], cu[i + 1]
        if b == a:
            continue
        q = qkv[a:b, q_off:q_off + hq * d].reshape(1, b - a, hq, d).transpose(1, 2)
        k = qkv[a:b, k_off:k_off + hkv * d].reshape(1, b - a, hkv, d).transpose(1, 2)
        v = qkv[a:b, v_off:v_off + hkv * d].reshape(1, b - a, hkv, d).transpose(1, 2)
        o = F.scaled_dot_product_attention(q, k, v, is_causal=True, scale=scale, enable_gqa=(hq != hkv))
        out_view[a:b] = o.transpose(1, 2).reshape(b - a, hq * d)


def embed(tokens, wte, positions=None, wpe=None, pos_offset: int = 0, out_dtype=None, scale: float = 1.0, out=None):
    """``out_dtype=torch.float32``: rows summed and stored in 32-bit (32-bit residual stream); then ``scale`` multiplies the
    token row and ``out`` ([T, width] 32-bit, e.g. a plane of a layer-output history) receives the result."""
    if _cuda(wte):
        from . import cuda_impl as cu

        if out_dtype == torch.float32:
            return cu.embed_f32(tokens, wte, positions, wpe, pos_offset, scale, out)
        assert scale == 1.0 and out is None, "embed: scale / out belong to the 32-bit form"
        return cu.embed(tokens, wte, positions, wpe, pos_offset)
    h = ref.embed(tokens, wte, positions, wpe, pos_offset, out_dtype=out_dtype, scale=scale)
    return h if out is None else out.copy_(h)


# ----------------------------------------------------------------------------- 32-bit residual stream, Dynamic Tanh
def dyt_residual(resid, alpha: float, weight, bias, a=None, scale_a=None, b=None, scale_b=None, out_dtype=None,
                 want_norm: bool = True):
    """Fold up to two layer-scaled 32-bit branch outputs into the 32-bit residual and apply Dynamic Tanh
    (tanh(alpha x) * weight + bias): returns (normed in ``out_dtype``, new residual).  ``want_norm=False`` only
    updates the residual (before an op that is not a norm, e.g. a re-injection GEMM)."""
    if _cuda(resid):
        from . import cuda_impl as cu

        return cu.dyt_residual(resid, alpha, weight, bias, a, scale_a, b, scale_b, out_dtype, want_norm)
    return ref.dyt_residual(resid, alpha, weight, bias, a, scale_a, b, scale_b, out_dtype, want_norm)


def cast_concat(a, b, dtype):
    """[cast(a) | cast(b)] of two 32-bit [T, *] streams as one GEMM operand."""
    if _cuda(a):
        from . import cuda_impl as cu

        return cu.cast_concat(a, b, dtype)
    return ref.cast_concat(a, b, dtype)


# ----------------------------------------------------------------------------- latent attention
def latent_prep(y, q_off, c_off, g_off, n_q, rank, heads, norm_w, eps, slot_mapping, cache, dtype):
    if _cuda(y):
        from . import cuda_impl as cu

        return cu.latent_prep(y, q_off, c_off, g_off, n_q, rank, heads, norm_w, eps, slot_mapping, cache, dtype)
    return ref.latent_prep(y, q_off, c_off, g_off, n_q, rank, heads, norm_w, eps, slot_mapping, cache, dtype)


def heads_matmul(x, w, heads, k, n, w_is_kn, row_scale=None, out_dtype=None, x_head_stride=None, elem_scale=None, out=None,
                 out_head_stride=None):
    """Per-head product [T, heads * k] x [heads, k, n]; see ops.reference.heads_matmul for the strides and scales."""
    if _cuda(x):
        from . import cuda_impl as cu

        return cu.heads_matmul(x, w, heads, k, n, w_is_kn, row_scale, out_dtype, x_head_stride, elem_scale, out, out_head_stride)
    return ref.heads_matmul(x, w, heads, k, n, w_is_kn, row_scale, out_dtype, x_head_stride, elem_scale, out, out_head_stride)


def latent_query_dtype(cache, heads, rank):
    """Type in which latent_attention() wants the absorbed queries: the cache's 16-bit type where it will run on the
    tcgen05 multi-query kernels, 32-bit for the generic kernel and on CPU."""
    if _cuda(cache):
        from . import cuda_impl as cu

        if cu.latent_uses_tc(cache.dtype, rank, cache.shape[1], heads):
            return cache.dtype
    return torch.float32


def latent_attention(q_abs, cache, batch, heads, rank, scale, out_dtype):
    """Causal attention of absorbed queries [T, heads * rank] over the paged latent cache (key = value = latent).

    16-bit compute with a rank the tcgen05 multi-query kernels cover (64 / 128 / 256) runs on those (the latent
    cache has their [blocks, 1, block_size, d] layout): decode batches on the split-KV decode kernel, portions of
    prompts on the paged prefill kernel.  Every other case (true 32-bit, other ranks) runs the generic kernel."""
    if _cuda(q_abs):
        from . import cuda_impl as cu

        return cu.latent_attention(q_abs, cache, batch, heads, rank, scale, out_dtype)
    return ref.latent_attention(q_abs, cache, batch.block_tables, batch.seq_lens, batch.cu_q, heads, rank, scale, out_dtype)


# ----------------------------------------------------------------------------- routed experts
def moe_route(z, experts, top, groups, keep, route_scale, score="softmax", correction=None, group_top=1, renorm=True):
    if _cuda(z):
        from . import cuda_impl as cu

        return cu.moe_route(z, experts, top, groups, keep, route_scale, score=score, correction=correction, group_top=group_top,
                            renorm=renorm)
    return ref.moe_route(z, experts, top, groups, keep, route_scale, score, correction, group_top, renorm)


def moe_experts(h, ids, wts, w_up, w_down, act, gated: bool = False):
    if _cuda(h):
        from . import cuda_impl as cu

        return cu.moe_experts(h, ids, wts, w_up, w_down, act, gated)
    return ref.moe_experts(h, ids, wts, w_up, w_down, act, gated)


# ----------------------------------------------------------------------------- recurrent layers, post-norm residual
def _dispatch(name, probe, *args, **kw):
    if _cuda(probe):
        from . import cuda_impl as cu

        return getattr(cu, name)(*args, **kw)
    return getattr(ref, name)(*args, **kw)


def embed_bigram(tokens, wte, table, mul_prev, mul_cur, buckets, batch, prev_state):
    """Token embedding plus a hashed (previous token, token) embedding, 32-bit; see ops.reference.embed_bigram."""
    return _dispatch("embed_bigram", wte, tokens, wte, table, mul_prev, mul_cur, buckets, batch, prev_state)


def postnorm_residual(y, weight, eps, resid=None, y2=None, w_a=None, w_b=None, one_plus=True, out_dtype=None):
    """RMS norm on a sub-layer's output (optionally the mean of two normed branches first), then the 32-bit residual
    sum: the post-norm counterpart of norm_residual / dyt_residual."""
    return _dispatch("postnorm_residual", y, y, weight, eps, resid, y2, w_a, w_b, one_plus, out_dtype)


def token_shift(x, mu, batch, prev_state, out_dtype=None):
    return _dispatch("token_shift", x, x, mu, batch, prev_state, out_dtype)


def causal_conv(u, w, bias, act, batch, state, out_dtype=None):
    return _dispatch("causal_conv", u, u, w, bias, act, batch, state, out_dtype)


def qknorm_kv_write(qkv, hq, hkv, dk, dv, q_w, k_w, eps, temp_coef, temp_every, positions, slot_mapping, k_cache, v_cache,
                    out_dtype=None, norm_whole=False, v_norm=False, q_head_scale=None):
    """Query / key norm (per head, or over a token's whole projection), query temperature and per-head factor, optional
    value norm, append to the pages; hkv = 0 prepares queries only.  See ops.reference.qknorm_kv_write."""
    return _dispatch("qknorm_kv_write", qkv, qkv, hq, hkv, dk, dv, q_w, k_w, eps, temp_coef, temp_every, positions,
                     slot_mapping, k_cache, v_cache, out_dtype, norm_whole, v_norm, q_head_scale)


def attention_bias(q, k_cache, v_cache, batch, hq, hkv, dk, dv, scale, dist_bias, gate=None, out_dtype=None, bias_over_scale=None,
                   window=0, slopes=None, sinks=None):
    """Causal paged attention with separate key / value sizes, a per-head distance bias (a table, and / or a linear
    penalty ``slopes[h] * distance``), an optional sliding window, an output gate and an attention sink per head
    (``sinks`` [hq] 32-bit: exp(sinks[h]) joins every softmax denominator of head h).
    ``bias_over_scale``: dist_bias / scale, kept by the caller for the tensor-core kernels (derived per call if absent)."""
    if _cuda(q):
        from . import cuda_impl as cu

        return cu.attention_bias(q, k_cache, v_cache, batch, hq, hkv, dk, dv, scale, dist_bias, gate, out_dtype, bias_over_scale,
                                 window, slopes, sinks)
    return ref.attention_bias(q, k_cache, v_cache, batch.block_tables, batch.seq_lens, batch.cu_q, hq, hkv, dk, dv, scale,
                              dist_bias, gate, out_dtype, window, slopes, sinks)


def unary(x, op, out_dtype=None):
    return _dispatch("unary", x, x, op, out_dtype)


def ssm_dt(dt_raw, dt_bias, a_log):
    return _dispatch("ssm_dt", dt_raw, dt_raw, dt_bias, a_log)


def linear_scan(q, k, v, decay, decay_kind, batch, state, heads, qk_heads, dk, dv, bonus=None, v_scale=None,
                read_before=False):
    """Gated linear recurrence (RWKV time mixing, lightning attention, state-space duality are parameter choices)."""
    return _dispatch("linear_scan", v, q, k, v, decay, decay_kind, batch, state, heads, qk_heads, dk, dv, bonus, v_scale,
                     read_before)


def gated_rmsnorm(o, gate, gate_act, weight, groups, eps, gate_first, skip_x=None, skip_d=None, out_dtype=None):
    return _dispatch("gated_rmsnorm", o, o, gate, gate_act, weight, groups, eps, gate_first, skip_x, skip_d, out_dtype)


# ----------------------------------------------------------------------------- several residual streams, delta rule
def embed_sinusoid(tokens, wte, scale, positions, streams=1, base=10000.0):
    """Scaled token embedding plus the sinusoidal position vector, 32-bit, as ``streams`` equal copies [streams, T, W]."""
    return _dispatch("embed_sinusoid", wte, tokens, wte, scale, positions, streams, base)


def hyper_residual(xs, y=None, mix=None, w_out=None, w_in=None, norm_w=None, eps=0.0, out_dtype=None):
    """Write a sub-layer's output into the residual streams and / or read the next sub-layer's normed input from them:
    the counterpart of norm_residual / dyt_residual / postnorm_residual for hyper-connections (in place on ``xs``)."""
    return _dispatch("hyper_residual", xs, xs, y, mix, w_out, w_in, norm_w, eps, out_dtype)


def delta_scan(q, k, v, log_decay, beta, batch, state, heads, qk_heads, dk, dv, unit_eps=None, q_scale=1.0, beta_sigmoid=False):
    """Gated delta rule (decay, error-correcting write, read-out after the write); see ops.reference.delta_scan."""
    return _dispatch("delta_scan", v, q, k, v, log_decay, beta, batch, state, heads, qk_heads, dk, dv, unit_eps, q_scale,
                     beta_sigmoid)


# ----------------------------------------------------------------------------- rotation by a table, sandwich norms
def rope_norm_kv_write(qk, hq, hkv, d, freq, mag, interleaved, unit_norm, eps, positions, slot_mapping, k_cache, v_cache,
                       out_dtype=None):
    """Rotation of q and k by a frequency table, optional unit RMS per head, keys to the K pages and the projected keys
    themselves to the V pages; see ops.reference.rope_norm_kv_write."""
    return _dispatch("rope_norm_kv_write", qk, qk, hq, hkv, d, freq, mag, interleaved, unit_norm, eps, positions, slot_mapping,
                     k_cache, v_cache, out_dtype)


def latent_rope_prep(y, q_off, q_rank, c_off, rank, rot, g_off, n_gate, qn_w, cn_w, eps, freq, mag, positions, slot_mapping, cache,
                     dtype):
    """Normed query latent, normed key / value latent + rotated key part into the cache row, sigmoid gate columns."""
    return _dispatch("latent_rope_prep", y, y, q_off, q_rank, c_off, rank, rot, g_off, n_gate, qn_w, cn_w, eps, freq, mag, positions,
                     slot_mapping, cache, dtype)


def latent_query_rope(q, heads, d, rot, rank, width, freq, mag, positions, dtype, abs_dtype):
    """Split the up-projected queries into the unrotated operand of the absorption and the rotated part, placed in the
    absorbed-query buffer."""
    return _dispatch("latent_query_rope", q, q, heads, d, rot, rank, width, freq, mag, positions, dtype, abs_dtype)


def hgrn_gates(y, n_qk, lower):
    """(silu(q), 1 - f, ln f) with f = lower + (1 - lower) sigmoid(f_raw), from the stacked 32-bit projection [q | f | ...]."""
    return _dispatch("hgrn_gates", y, y, n_qk, lower)


def sandwich_residual(resid, y, w_post, eps, w_next=None, history=None, index=0, depth_w=None, out_dtype=None):
    """r = resid + rms_div(y) * w_post, optionally stored as layer output ``index`` of ``history`` and replaced by the
    depth-weighted average of the outputs so far, then h = rms_div(r) * w_next; returns (h, r).  The counterpart of
    norm_residual / postnorm_residual for sub-layers with a norm on both sides."""
    return _dispatch("sandwich_residual", resid, resid, y, w_post, eps, w_next, history, index, depth_w, out_dtype)


def softcap(z, cap):
    """cap * tanh(z / cap) in place."""
    return _dispatch("softcap", z, z, cap)


def sample(logits, greedy, temperature, top_k, top_p, rng_state, vocab: Optional[int] = None, out=None):
    if _cuda(logits):
        from . import cuda_impl as cu

        return cu.sample(logits, greedy, temperature, top_k, top_p, rng_state, vocab, out)
    tok = ref.sample(logits, greedy, temperature, top_k, top_p, rng_state, vocab).to(torch.int32)
    if out is not None:
        out.copy_(tok)
        return out
    return tok

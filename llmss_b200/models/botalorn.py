"""Botalorn: a decoder-only design of pre-normed sub-layers over several 32-bit residual streams (hyper-connections),
with sliding-window attention layers -- some of which attend over the keys and values of an earlier layer -- beside
gated-delta-rule layers, a token shift in front of every mixer, and squared-ReLU feed-forwards.

    x_1 .. x_S = embed[token] * scale + sinusoid(position)                  (S equal copies, 32-bit from here on)
    sub-layer q of a layer (1: mixer, 2: feed-forward), weights hc<q>.{in, mix, out}:
        u = sum_s in[s] x_s ;  y = f(rms_div(u) * norm<q>) ;  x_t <- sum_s mix[s, t] x_s + out[t] y   (all t from the old x)
    the mixer reads h + (h_prev - h) * shift, h_prev = the previous token's normed input (zeros at a sequence's start)
    mixers:  "attention" (window, distance slopes, optionally ``kv_from`` another layer) | "delta"    -> models/mixers.py
    ffn:     dense, W_down relu(W_up h)^2, or none
    logits = head (rms_div(sum_s x_s) * final.norm)

config.json keys: architecture, vocab, width, norm.eps, embedding.scale, streams (absent: one plain residual stream),
layers[i].{type, mixer{heads, kv_heads, dim, vdim, conv, scale, mask{size}, kv_from}, mlp{kind, ff} | null}.
Tensor names: embed, head, final.norm, l<i>.norm1, l<i>.norm2, l<i>.shift, l<i>.hc<q>.{in, mix, out}, l<i>.mix.*,
l<i>.mlp.{up, down} (listed with each loader below).

The model is a graph over the framework's ops.  What a sequence carries between steps lives in the engine's
HybridCache: pages for the keys / values of the attention layers that project their own, one state slot for the delta
states, the convolution tails and every layer's previous normed row.  Runner, block and slot allocators, batching and
sampler drive it like the other families.  It runs unsharded (TP = 1).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import List, Optional

import torch
from torch import nn

from .. import ops
from ..engine.batch import BatchInput
from ..engine.kv_cache import HybridCache
from ..ops import ACT_RELU2
from ..parallel.comm import comm_for
from ..utils.tracing import trace
from .mixers import DeltaMixer, DenseFFN, HyperConnection, LayerCacheView, WindowAttention

MIXER_TYPES = ("attention", "delta")
FFN_KINDS = ("dense",)
F32 = torch.float32


@dataclass
class BotalornSpec:
    hidden: int
    vocab: int
    eps: float
    embed_scale: float
    streams: Optional[int]                                 # None: one stream with the plain residual sum
    layers: List[dict] = field(default_factory=list)      # the config's layer entries, checked
    model_type: str = "botalorn"
    max_pos: int = 1 << 30       # sinusoidal positions and relative distances: no limit of its own
    default_seq_len: int = 4096  # block-table width when the caller names neither a length nor a pool
    learned_pos: bool = False

    @property
    def n_layers(self) -> int:
        return len(self.layers)


def botalorn_spec(config) -> BotalornSpec:
    c = config.raw if hasattr(config, "raw") else dict(config)
    layers = list(c["layers"])
    for i, lc in enumerate(layers):
        if lc["type"] not in MIXER_TYPES:
            raise ValueError(f"botalorn: layer {i} has unknown mixer type {lc['type']!r}; have {MIXER_TYPES}")
        f = lc.get("mlp")
        if f is not None and f.get("kind") not in FFN_KINDS:
            raise ValueError(f"botalorn: layer {i} has unknown feed-forward kind {f.get('kind')!r}; have {FFN_KINDS}")
        m = lc["mixer"]
        j = m.get("kv_from")
        if lc["type"] == "attention" and j is not None:
            if not (0 <= int(j) < i) or layers[int(j)]["type"] != "attention" or layers[int(j)]["mixer"].get("kv_from") is not None:
                raise ValueError(f"botalorn: layer {i} takes keys / values from layer {j}, which is not an earlier attention layer "
                                 "with projections of its own")
            o = layers[int(j)]["mixer"]
            if (int(o["kv_heads"]), int(o["dim"]), int(o["vdim"])) != (int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])):
                raise ValueError(f"botalorn: layer {i} and its lender {j} differ in key / value heads or sizes")
    streams = c.get("streams")
    return BotalornSpec(int(c["width"]), int(c["vocab"]), float(c["norm"]["eps"]), float(c.get("embedding", {}).get("scale", 1.0)),
                        None if streams is None else int(streams), layers)


def _build_mixer(kind: str, m: dict, width: int, eps: float):
    if kind == "delta":
        return DeltaMixer(width, int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"]), int(m.get("conv", 1)), eps)
    mask = m.get("mask") or {}
    window = mask.get("size")
    kv_from = m.get("kv_from")
    return WindowAttention(width, int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"]), int(m.get("conv", 1)),
                           float(m.get("scale", int(m["dim"]) ** -0.5)), None if window is None else int(window), eps,
                           kv_from=None if kv_from is None else int(kv_from))


class BotalornLayer:
    __slots__ = ("kind", "mixer", "ffn", "norm1", "norm2", "shift", "hc1", "hc2")


class BotalornLM(nn.Module):
    """The decoder core the engine drives (same surface as DecoderLM: forward / forward_hidden / logits / make_cache)."""

    needs_state = True     # the runner gives every sequence a state slot, and neither shares nor evicts its pages

    def __init__(self, spec: BotalornSpec, process_group, device, dtype):
        super().__init__()
        self.spec = spec
        self.comm = comm_for(process_group, device)
        self.tp, self.rank = self.comm.size, self.comm.rank
        if self.tp != 1:
            raise NotImplementedError("botalorn runs unsharded: start it with one rank")
        self.device, self.dtype = torch.device(device), dtype
        self.vocab_blk = spec.vocab
        self.n_streams = spec.streams or 1
        self.layers: List[BotalornLayer] = []
        for lc in spec.layers:
            L = BotalornLayer()
            L.kind = lc["type"]
            L.mixer = _build_mixer(lc["type"], lc["mixer"], spec.hidden, spec.eps)
            L.ffn = DenseFFN(act=ACT_RELU2) if lc.get("mlp") is not None else None
            L.norm1 = L.norm2 = L.shift = L.hc1 = L.hc2 = None
            self.layers.append(L)
        self.wte = self.w_head = self.final_w = None
        self.sum_in = torch.ones(self.n_streams, dtype=F32, device=self.device)   # the read-out of the final norm: x = sum_s x_s

    # ------------------------------------------------------------------ cache
    def default_block_size(self) -> int:
        return 64 if self.device.type == "cuda" else 16

    def make_cache(self, num_blocks: int, block_size: int, max_seqs: Optional[int] = None) -> HybridCache:
        kv, states = {}, {}
        for i, L in enumerate(self.layers):
            shape = L.mixer.kv_shape()
            if shape is not None:
                kv[i] = shape
            states[(i, "shift")] = ((self.spec.hidden,), F32)
            for name, sd in L.mixer.state_shapes().items():
                states[(i, name)] = sd
        return HybridCache(kv, states, num_blocks, block_size, max_seqs or 1, self.dtype, self.device)

    def num_parameters_local(self) -> int:
        ts = [self.wte, self.w_head, self.final_w]
        for L in self.layers:
            ts += [L.norm1, L.norm2, L.shift] + L.mixer.weights() + L.hc1.weights()
            if L.ffn is not None:
                ts += L.ffn.weights() + L.hc2.weights()
        return sum(t.numel() for t in ts if t is not None)

    def finalize(self):
        return self

    # ------------------------------------------------------------------ forward
    def forward_hidden(self, batch: BatchInput, kv: HybridCache, taps: Optional[list] = None) -> torch.Tensor:
        """Final-normed hidden states [T, width] of every packed token.  ``taps``: a list that receives the 32-bit
        residual stream (the sum of the streams) after every layer (debugging / tests)."""
        s, dt = self.spec, self.dtype
        assert batch.state_slots is not None, "botalorn: the batch names no state slots"
        with trace("embed"):
            xs = ops.embed_sinusoid(batch.tokens, self.wte, s.embed_scale, batch.positions, self.n_streams)
        y = hc = None           # the last sub-layer's output, not yet written into the streams, and its connection
        for i, L in enumerate(self.layers):
            lc = LayerCacheView(kv, i, pages_key=getattr(L.mixer, "kv_from", None))
            with trace("hyper_residual"):
                h = ops.hyper_residual(xs, y, hc and hc.mix, hc and hc.w_out, L.hc1.w_in, L.norm1, s.eps,
                                       out_dtype=F32 if L.shift is not None else dt)
            if L.shift is not None:
                with trace("token_shift"):
                    h = ops.token_shift(h, L.shift, batch, lc.state("shift"), out_dtype=dt)[0]
            y, hc = L.mixer.forward(h, batch, lc, dt), L.hc1
            if L.ffn is not None:
                with trace("hyper_residual"):
                    h = ops.hyper_residual(xs, y, hc.mix, hc.w_out, L.hc2.w_in, L.norm2, s.eps, out_dtype=dt)
                y, hc = L.ffn.forward(h), L.hc2
            if taps is not None:
                ops.hyper_residual(xs, y, hc.mix, hc.w_out)
                y = hc = None
                taps.append(xs.sum(0))
        with trace("final_norm"):
            return ops.hyper_residual(xs, y, hc and hc.mix, hc and hc.w_out, self.sum_in, self.final_w, s.eps, out_dtype=dt)

    def logits(self, hidden_rows: torch.Tensor) -> torch.Tensor:
        with trace("lm_head"):
            return ops.linear(hidden_rows, self.w_head, out_dtype=torch.float32)

    local_logits = logits

    def forward(self, batch: BatchInput, kv, last_only: bool = True, gather_logits: bool = True) -> torch.Tensor:
        h = self.forward_hidden(batch, kv)
        if last_only:
            h = h.index_select(0, batch.last_idx)
        return self.logits(h)


# ---------------------------------------------------------------------------------------------------- weights
def _f32(t):
    """Small per-channel parameters are kept in 32-bit whatever the compute type (the checkpoint's values are exact in it)."""
    return t.float().contiguous()


def _taps_from_tensor(mx, shape):
    """The number of taps is the convolution tensor's second size (the configuration's ``conv`` only repeats it)."""
    mx.taps = int(shape[1])


def _load_attention(mx: WindowAttention, get, w_shape, p):
    """<p>.q [heads*dim, W] + .q.conv [.., taps] + .q.norm [heads*dim]; <p>.temp [heads]; <p>.g [heads, W]; <p>.o [W, heads*vdim];
    with projections of its own also <p>.k [kv_heads*dim, W] + .k.conv + .k.norm [kv_heads*dim], <p>.v [kv_heads*vdim, W] + .v.conv."""
    own = mx.own_kv
    _taps_from_tensor(mx, w_shape(f"{p}.q.conv"))
    mx.set_weights(get(f"{p}.q"), get(f"{p}.k") if own else None, get(f"{p}.v") if own else None,
                   _f32(get(f"{p}.q.conv")), _f32(get(f"{p}.k.conv")) if own else None, _f32(get(f"{p}.v.conv")) if own else None,
                   _f32(get(f"{p}.q.norm")), _f32(get(f"{p}.k.norm")) if own else None, _f32(get(f"{p}.temp")), get(f"{p}.g"),
                   get(f"{p}.o"))
    if mx.conv_w.shape != (mx.n_conv, mx.taps):
        raise ValueError(f"{p}: convolution weights {tuple(mx.conv_w.shape)} do not fit {mx.n_conv} channels x {mx.taps} taps")


def _load_delta(mx: DeltaMixer, get, w_shape, p):
    """<p>.q / .k [kv_heads*dim, W], <p>.v / .g [heads*vdim, W], each of q k v with .conv [.., taps]; <p>.b / .a [heads, W];
    <p>.dt_bias / .A_log [heads]; <p>.norm [vdim]; <p>.o [W, heads*vdim]."""
    _taps_from_tensor(mx, w_shape(f"{p}.q.conv"))
    mx.set_weights(get(f"{p}.q"), get(f"{p}.k"), get(f"{p}.v"), _f32(get(f"{p}.q.conv")), _f32(get(f"{p}.k.conv")),
                   _f32(get(f"{p}.v.conv")), get(f"{p}.b"), get(f"{p}.a"), _f32(get(f"{p}.dt_bias")), _f32(get(f"{p}.A_log")),
                   _f32(get(f"{p}.norm")), get(f"{p}.g"), get(f"{p}.o"))
    if mx.conv_w.shape != (mx.n_conv, mx.taps):
        raise ValueError(f"{p}: convolution weights {tuple(mx.conv_w.shape)} do not fit {mx.n_conv} channels x {mx.taps} taps")


_LOADERS = {"attention": _load_attention, "delta": _load_delta}


def load_botalorn(m: BotalornLM, w):
    get = w.get_tensor

    streams = m.spec.streams
    if streams is None and w.has("l0.hc1.in"):
        # hyper-connection tensors without the configuration key: their size says how many streams there are
        streams = int(w.get_shape("l0.hc1.in")[0])
        m.n_streams, m.sum_in = streams, torch.ones(streams, dtype=F32, device=m.device)

    def connection(prefix):
        if streams is None:
            return HyperConnection.identity(m.device)
        return HyperConnection(_f32(get(f"{prefix}.in")), _f32(get(f"{prefix}.mix")), _f32(get(f"{prefix}.out")))

    m.wte, m.w_head, m.final_w = get("embed"), get("head").contiguous(), _f32(get("final.norm"))
    for i, L in enumerate(m.layers):
        p = f"l{i}"
        L.norm1 = _f32(get(f"{p}.norm1"))
        L.shift = _f32(get(f"{p}.shift")).view(1, -1) if w.has(f"{p}.shift") else None
        L.hc1 = connection(f"{p}.hc1")
        _LOADERS[L.kind](L.mixer, get, w.get_shape, f"{p}.mix")
        if L.ffn is None:
            continue
        L.norm2 = _f32(get(f"{p}.norm2"))
        L.hc2 = connection(f"{p}.hc2")
        L.ffn.w_up, L.ffn.w_down = get(f"{p}.mlp.up").contiguous(), get(f"{p}.mlp.down").contiguous()

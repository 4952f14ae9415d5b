"""Random-init HF-format checkpoints (config.json + *.safetensors) for benches and tests.

There is no network for real checkpoints, so benchmarks use random weights of the named
architecture written in the ordinary unsharded HF layout -- the same
files are then loaded by this framework *and* by the unmodified reference through its
`Weights` class.  Tensors are generated shard by shard on `device` (GPU when available) so a
6B-parameter checkpoint takes seconds, not minutes.
"""
from __future__ import annotations

import json
import os
from pathlib import Path
from typing import Dict, Iterator, List, Optional, Tuple

import torch
from safetensors.torch import save_file

PRESETS: Dict[str, dict] = {
    # GPT-J-6B shape: the largest architecture the reference itself can load
    "gptj-6b": dict(model_type="gptj", architectures=["GPTJForCausalLM"], vocab_size=50400, n_positions=2048,
                    n_embd=4096, n_layer=28, n_head=16, rotary_dim=64, n_inner=None, activation_function="gelu_new",
                    layer_norm_epsilon=1e-5, tie_word_embeddings=False, bos_token_id=50256, eos_token_id=50256),
    "gptj-tiny": dict(model_type="gptj", architectures=["GPTJForCausalLM"], vocab_size=512, n_positions=256,
                      n_embd=256, n_layer=2, n_head=4, rotary_dim=32, n_inner=None, activation_function="gelu_new",
                      layer_norm_epsilon=1e-5, tie_word_embeddings=False, bos_token_id=0, eos_token_id=0),
    "gptj-tiny8": dict(model_type="gptj", architectures=["GPTJForCausalLM"], vocab_size=512, n_positions=256,
                       n_embd=512, n_layer=2, n_head=8, rotary_dim=32, n_inner=None, activation_function="gelu_new",
                       layer_norm_epsilon=1e-5, tie_word_embeddings=False, bos_token_id=0, eos_token_id=0),
    # 8-rank test models: GQA (16 q heads over 8 kv heads: one kv head per rank at TP=8) and MQA (kv replicated)
    "llama-tiny8": dict(model_type="llama", architectures=["LlamaForCausalLM"], vocab_size=512, hidden_size=1024,
                        intermediate_size=2048, num_hidden_layers=2, num_attention_heads=16, num_key_value_heads=8,
                        max_position_embeddings=256, rms_norm_eps=1e-5, hidden_act="silu", rope_theta=10000.0,
                        tie_word_embeddings=False),
    "bigcode-tiny8": dict(model_type="gpt_bigcode", architectures=["GPTBigCodeForCausalLM"], vocab_size=512,
                          n_positions=256, n_embd=512, n_layer=2, n_head=8, n_inner=2048, multi_query=True,
                          activation_function="gelu_pytorch_tanh", layer_norm_epsilon=1e-5, tie_word_embeddings=True),
    # StarCoder shape (MQA) -- the reference's second family
    "starcoder": dict(model_type="gpt_bigcode", architectures=["GPTBigCodeForCausalLM"], vocab_size=49152,
                      n_positions=8192, n_embd=6144, n_layer=40, n_head=48, n_inner=24576, multi_query=True,
                      activation_function="gelu_pytorch_tanh", layer_norm_epsilon=1e-5, tie_word_embeddings=True),
    "llama-2-7b": dict(model_type="llama", architectures=["LlamaForCausalLM"], vocab_size=32000, hidden_size=4096,
                       intermediate_size=11008, num_hidden_layers=32, num_attention_heads=32, num_key_value_heads=32,
                       max_position_embeddings=4096, rms_norm_eps=1e-5, hidden_act="silu", rope_theta=10000.0,
                       tie_word_embeddings=False),
    "llama-2-13b": dict(model_type="llama", architectures=["LlamaForCausalLM"], vocab_size=32000, hidden_size=5120,
                        intermediate_size=13824, num_hidden_layers=40, num_attention_heads=40, num_key_value_heads=40,
                        max_position_embeddings=4096, rms_norm_eps=1e-5, hidden_act="silu", rope_theta=10000.0,
                        tie_word_embeddings=False),
    "opt-1.3b": dict(model_type="opt", architectures=["OPTForCausalLM"], vocab_size=50272, hidden_size=2048,
                     num_hidden_layers=24, ffn_dim=8192, num_attention_heads=32, max_position_embeddings=2048,
                     do_layer_norm_before=True, word_embed_proj_dim=2048, activation_function="relu",
                     tie_word_embeddings=True),
    # GPT-2 XL: 25 heads -- not divisible by 2; BASELINE config 2 names it at TP=2 (heads are padded, models/decoder.py)
    "gpt2-xl": dict(model_type="gpt2", architectures=["GPT2LMHeadModel"], vocab_size=50257, n_positions=1024, n_embd=1600,
                    n_layer=48, n_head=25, activation_function="gelu_new", layer_norm_epsilon=1e-5,
                    tie_word_embeddings=True),
    "gpt2": dict(model_type="gpt2", architectures=["GPT2LMHeadModel"], vocab_size=50257, n_positions=1024, n_embd=768,
                 n_layer=12, n_head=12, activation_function="gelu_new", layer_norm_epsilon=1e-5,
                 tie_word_embeddings=True),
}


def bedovik_config(width: int, vocab: int, max_positions: int, layers, loop=None, eps: float = 1e-5) -> dict:
    """config.json of a Bedovik model.  ``layers``: one dict per layer with keys gated (bool), heads, dim, vdim, kv_rank
    and optionally scale, experts, top, groups, keep, route_scale, ff (no ``experts``: a layer without feed-forward).
    ``loop``: (start, stop, times) or None."""
    out = []
    for L in layers:
        mlp = None
        if L.get("experts"):
            mlp = {"kind": "moe", "expert": {"ff": L["ff"]},
                   "router": {"experts": L["experts"], "top": L["top"], "scale": L.get("route_scale", 1.0),
                              "groups": {"count": L.get("groups", 1), "keep": L.get("keep", L.get("groups", 1))}}}
        out.append({"type": "latent_attention" if L.get("gated", True) else "latent_attention_2",
                    "mixer": {"heads": L["heads"], "dim": L["dim"], "vdim": L["vdim"], "kv_rank": L["kv_rank"],
                              "scale": L.get("scale", L["dim"] ** -0.5)},
                    "mlp": mlp})
    cfg = {"architecture": "Bedovik", "vocab": vocab, "width": width, "max_positions": max_positions, "norm": {"eps": eps},
           "layers": out}
    if loop is not None:
        cfg["loop"] = {"start": loop[0], "stop": loop[1], "times": loop[2]}
    return cfg


def _bedovik_shapes(cfg: dict):
    W, V, P = cfg["width"], cfg["vocab"], cfg["max_positions"]
    yield "embed", (V, W), "unit"
    yield "pos", (P, W), "emb"
    if cfg.get("loop"):
        yield "loop.in", (W, 2 * W), "fan"
        yield "loop.step", (cfg["loop"]["times"], W), "b"
    for i, L in enumerate(cfg["layers"]):
        p, m = f"l{i}", L["mixer"]
        H, d, dv, R = m["heads"], m["dim"], m["vdim"], m["kv_rank"]
        yield f"{p}.norm1", (W,), "ln_w"
        yield f"{p}.norm1.b", (W,), "ln_b"
        yield f"{p}.norm1.alpha", (), "alpha"
        yield f"{p}.mix.q", (H * d, W), "fan"
        yield f"{p}.mix.dkv", (R, W), "fan"
        yield f"{p}.mix.dkv.norm", (R,), "ln_w"
        yield f"{p}.mix.uk", (H * d, R), "fan"
        yield f"{p}.mix.uv", (H * dv, R), "fan"
        if L["type"] == "latent_attention":
            yield f"{p}.mix.g", (H, W), "fan"
        yield f"{p}.mix.o", (W, H * dv), "fan"
        yield f"{p}.ls1", (W,), "ls"
        if L.get("mlp"):
            F, E = L["mlp"]["expert"]["ff"], L["mlp"]["router"]["experts"]
            for e in range(E):
                yield f"{p}.mlp.e{e}.up", (F, W), "fan"
                yield f"{p}.mlp.e{e}.down", (W, F), "fan"
            yield f"{p}.mlp.router", (E, W), "fan2"
            yield f"{p}.ls2", (W,), "ls"
    yield "final.norm", (W,), "ln_w"
    yield "final.norm.b", (W,), "ln_b"
    yield "final.norm.alpha", (), "alpha"
    yield "head", (V, W), "fan"


def _bedovik_preset(width, vocab, heads, dim, vdim, rank, experts, top, groups, keep, ff, n_layers, loop, max_positions=4096):
    layers = [dict(gated=(i % 2 == 0), heads=heads, dim=dim, vdim=vdim, kv_rank=rank, experts=experts, top=top, groups=groups,
                   keep=keep, route_scale=2.0, ff=ff) for i in range(n_layers)]
    return bedovik_config(width, vocab, max_positions, layers, loop)


PRESETS.update({
    # latent attention + routed experts at sizes whose layers resemble a served model's (random weights); the
    # gptj-like-* presets are multi-head models of equal width, depth (= layer runs), heads and active feed-forward size
    "bedovik-tiny": _bedovik_preset(128, 320, 4, 16, 24, 64, 8, 2, 4, 2, 32, 3, (1, 3, 2), 256),
    "bedovik-2k": _bedovik_preset(2048, 32000, 16, 128, 128, 128, 16, 4, 4, 2, 1024, 10, (1, 9, 2)),
    "bedovik-4k": _bedovik_preset(4096, 32000, 32, 128, 128, 128, 32, 4, 8, 4, 1536, 10, (1, 9, 2)),
    "gptj-like-2k": dict(model_type="gptj", architectures=["GPTJForCausalLM"], vocab_size=32000, n_positions=4096, n_embd=2048,
                         n_layer=18, n_head=16, rotary_dim=64, n_inner=4096, activation_function="gelu_new",
                         layer_norm_epsilon=1e-5, tie_word_embeddings=False, bos_token_id=0, eos_token_id=0),
    "gptj-like-4k": dict(model_type="gptj", architectures=["GPTJForCausalLM"], vocab_size=32000, n_positions=4096, n_embd=4096,
                         n_layer=18, n_head=32, rotary_dim=64, n_inner=6144, activation_function="gelu_new",
                         layer_norm_epsilon=1e-5, tie_word_embeddings=False, bos_token_id=0, eos_token_id=0),
})


def ninelix_config(width: int, vocab: int, layers, buckets: int = 251, mul_prev: int = 31, mul_cur: int = 7, logit_scale: float = 1.0,
                   eps: float = 1e-6) -> dict:
    """config.json of a Ninelix model.  ``layers``: one dict per layer, {"type": "wkv", "heads", "dim", "lora"} |
    {"type": "lightning", "heads", "dim", "vdim", optionally "decay"} | {"type": "parallel", "left": {heads, kv_heads, dim, vdim, conv,
    bias_max, buckets, optionally scale, q_temp}, "right": {heads, vdim, state, groups, norm_groups, conv}}, each with
    "mlp": None | {"kind": "dense", "ff"} | {"kind": "moe", "experts", "top", "ff"}.  ``lora`` (rows of the decay's low-rank
    projection) and ``buckets`` (rows of the distance table) only size the random tensors: a model reads them off the tensors."""
    out = []
    for L in layers:
        f = L.get("mlp")
        if f is not None and f["kind"] == "moe":
            f = {"kind": "moe", "expert": {"ff": f["ff"]}, "router": {"experts": f["experts"], "top": f["top"]}}
        elif f is not None:
            f = {"kind": "dense", "ff": f["ff"]}
        if L["type"] == "wkv":
            m = {"heads": L["heads"], "dim": L["dim"], "lora": L.get("lora", 16)}
        elif L["type"] == "lightning":
            H = L["heads"]
            m = {"heads": H, "dim": L["dim"], "vdim": L["vdim"],
                 "decay": L.get("decay") or [1.0 - 2.0 ** -(1.0 + 6.0 * h / max(1, H - 1)) for h in range(H)]}
        else:
            a, r = dict(L["left"]), dict(L["right"])
            a.setdefault("scale", a["dim"] ** -0.5)
            a.setdefault("q_temp", {"coef": 0.25, "every": 32})
            a.setdefault("buckets", 16)
            m = {"left": a, "right": r}
        out.append({"type": L["type"], "mixer": m, "mlp": f})
    return {"architecture": "Ninelix", "vocab": vocab, "width": width, "norm": {"eps": eps}, "logit_scale": logit_scale,
            "embedding": {"bigram": {"buckets": buckets, "mul_prev": mul_prev, "mul_cur": mul_cur}}, "layers": out}


def _ninelix_shapes(cfg: dict):
    W, V = cfg["width"], cfg["vocab"]
    yield "embed", (V, W), "unit"
    yield "bigram", (cfg["embedding"]["bigram"]["buckets"] + 1, W), ("n", 0.0, 0.5)
    for i, L in enumerate(cfg["layers"]):
        p, m = f"l{i}", L["mixer"]
        yield f"{p}.norm1", (W,), ("n", 0.0, 0.1)
        q = f"{p}.mix"
        if L["type"] == "wkv":
            n, r = m["heads"] * m["dim"], m.get("lora", 16)
            for s in "rkvgw":
                yield f"{q}.mu.{s}", (W,), ("u", 0.0, 1.0)
            for s in "rkvg":
                yield f"{q}.{s}", (n, W), "fan"
            yield f"{q}.w1", (r, W), "fan"
            yield f"{q}.w2", (n, r), "fan"
            yield f"{q}.w0", (n,), ("n", -1.0, 1.0)
            yield f"{q}.u", (m["heads"], m["dim"]), ("n", 0.0, 0.5)
            yield f"{q}.norm", (n,), "ln_w"
            yield f"{q}.o", (W, n), "fan"
        elif L["type"] == "lightning":
            nk, nv = m["heads"] * m["dim"], m["heads"] * m["vdim"]
            yield f"{q}.q", (nk, W), "fan"
            yield f"{q}.k", (nk, W), "fan"
            yield f"{q}.v", (nv, W), "fan"
            yield f"{q}.g", (nv, W), "fan"
            yield f"{q}.norm", (nv,), "ln_w"
            yield f"{q}.o", (W, nv), "fan"
        else:
            a, r = m["left"], m["right"]
            for s, n in (("q", a["heads"] * a["dim"]), ("k", a["kv_heads"] * a["dim"]), ("v", a["kv_heads"] * a["vdim"])):
                yield f"{q}.left.{s}", (n, W), "fan"
                yield f"{q}.left.{s}.b", (n,), ("n", 0.0, 0.1)
                yield f"{q}.left.{s}.conv", (n, a["conv"]), ("n", 0.0, a["conv"] ** -0.5)
            yield f"{q}.left.q.norm", (a["dim"],), "ln_w"
            yield f"{q}.left.k.norm", (a["dim"],), "ln_w"
            yield f"{q}.left.rel", (a.get("buckets", 16), a["heads"]), ("n", 0.0, 1.0)
            yield f"{q}.left.g", (a["heads"], W), "fan"
            yield f"{q}.left.o", (W, a["heads"] * a["vdim"]), "fan"
            inner, gn = r["heads"] * r["vdim"], r["groups"] * r["state"]
            yield f"{q}.right.in", (2 * inner + 2 * gn + r["heads"], W), "fan"
            yield f"{q}.right.conv", (inner + 2 * gn, r["conv"]), ("n", 0.0, r["conv"] ** -0.5)
            yield f"{q}.right.conv.b", (inner + 2 * gn,), ("n", 0.0, 0.1)
            yield f"{q}.right.dt_bias", (r["heads"],), ("n", -1.0, 1.0)
            yield f"{q}.right.A_log", (r["heads"],), ("n", 0.0, 0.7)
            yield f"{q}.right.D", (r["heads"],), "ln_w"
            yield f"{q}.right.norm", (inner,), "ln_w"
            yield f"{q}.right.o", (W, inner), "fan"
            yield f"{q}.left.out", (W,), "ln_w"
            yield f"{q}.right.out", (W,), "ln_w"
        f = L.get("mlp")
        if f is None:
            continue
        yield f"{p}.norm2", (W,), ("n", 0.0, 0.1)
        if f["kind"] == "dense":
            yield f"{p}.mlp.up", (f["ff"], W), "fan"
            yield f"{p}.mlp.down", (W, f["ff"]), "fan"
        else:
            F = f["expert"]["ff"]
            for e in range(f["router"]["experts"]):
                yield f"{p}.mlp.e{e}.gate", (F, W), "fan"
                yield f"{p}.mlp.e{e}.up", (F, W), "fan"
                yield f"{p}.mlp.e{e}.down", (W, F), "fan"
            yield f"{p}.mlp.router", (f["router"]["experts"], W), "fan2"
    yield "final.norm", (W,), ("n", 0.0, 0.1)
    yield "head", (V, W), "fan"


def _ninelix_preset(width, vocab, heads, ff, n_blocks, experts=8, top=2, eff=None):
    """``n_blocks`` x (parallel + dense, wkv + experts, lightning + dense) at head size 64 / 128."""
    d = 64
    H = width // d
    layers = []
    for _ in range(n_blocks):
        layers += [
            {"type": "parallel", "left": dict(heads=heads, kv_heads=max(1, heads // 4), dim=128, vdim=128, conv=3, bias_max=512, buckets=32),
             "right": dict(heads=H, vdim=d, state=128, groups=max(1, H // 8), norm_groups=max(1, H // 8), conv=4),
             "mlp": {"kind": "dense", "ff": ff}},
            {"type": "wkv", "heads": H, "dim": d, "lora": 64, "mlp": {"kind": "moe", "experts": experts, "top": top, "ff": eff or ff // top}},
            {"type": "lightning", "heads": H // 2, "dim": 128, "vdim": 128, "mlp": {"kind": "dense", "ff": ff}},
        ]
    return ninelix_config(width, vocab, layers, buckets=65521, mul_prev=1000003, mul_cur=31)


PRESETS.update({
    "ninelix-tiny": ninelix_config(128, 320, [
        {"type": "parallel", "left": dict(heads=4, kv_heads=2, dim=24, vdim=16, conv=3, bias_max=40, buckets=12),
         "right": dict(heads=4, vdim=16, state=24, groups=2, norm_groups=2, conv=4), "mlp": {"kind": "dense", "ff": 192}},
        {"type": "wkv", "heads": 4, "dim": 24, "lora": 8, "mlp": {"kind": "moe", "experts": 6, "top": 2, "ff": 48}},
        {"type": "lightning", "heads": 2, "dim": 32, "vdim": 40, "mlp": {"kind": "dense", "ff": 192}}]),
    # sizes whose layers resemble a served model's (random weights), beside gptj-like-* of equal width and depth
    "ninelix-2k": _ninelix_preset(2048, 32000, 16, 4096, 6),
    "ninelix-4k": _ninelix_preset(4096, 32000, 32, 6144, 6),
})


def botalorn_config(width: int, vocab: int, layers, streams: Optional[int] = 2, embed_scale: float = 1.0, eps: float = 1e-6) -> dict:
    """config.json of a Botalorn model.  ``layers``: one dict per layer, {"type": "attention", heads, kv_heads, dim, vdim, conv,
    optionally window, scale, kv_from} | {"type": "delta", heads, kv_heads, dim, vdim, conv}, each with "mlp": None |
    {"kind": "dense", "ff"}.  ``streams`` None: one plain residual stream (no hyper-connection tensors)."""
    out = []
    for L in layers:
        m = {k: L[k] for k in ("heads", "kv_heads", "dim", "vdim", "conv")}
        if L["type"] == "attention":
            m["scale"] = L.get("scale", L["dim"] ** -0.5)
            if L.get("window") is not None:
                m["mask"] = {"size": L["window"]}
            if L.get("kv_from") is not None:
                m["kv_from"] = L["kv_from"]
        f = L.get("mlp")
        out.append({"type": L["type"], "mixer": m, "mlp": None if f is None else {"kind": "dense", "ff": f["ff"]}})
    cfg = {"architecture": "Botalorn", "vocab": vocab, "width": width, "norm": {"eps": eps}, "embedding": {"scale": embed_scale},
           "layers": out}
    if streams is not None:
        cfg["streams"] = streams
    return cfg


def _botalorn_shapes(cfg: dict):
    W, V, S = cfg["width"], cfg["vocab"], cfg.get("streams")
    yield "embed", (V, W), "unit"
    for i, L in enumerate(cfg["layers"]):
        p, m = f"l{i}", L["mixer"]
        q = f"{p}.mix"
        yield f"{p}.norm1", (W,), "ln_w"
        yield f"{p}.shift", (W,), ("u", 0.0, 1.0)
        subs = ["hc1"] + (["hc2"] if L.get("mlp") is not None else [])
        if S is not None:
            for hc in subs:
                yield f"{p}.{hc}.in", (S,), ("n", 1.0 / S, 0.2)
                yield f"{p}.{hc}.out", (S,), ("n", 0.7, 0.2)
                yield f"{p}.{hc}.mix", (S, S), ("hcmix", 0.8, 0.1)
        nq_att, nk, nv = m["heads"] * m["dim"], m["kv_heads"] * m["dim"], m["kv_heads"] * m["vdim"]
        if L["type"] == "attention":
            own = m.get("kv_from") is None
            for s, n in (("q", nq_att),) + ((("k", nk), ("v", nv)) if own else ()):
                yield f"{q}.{s}", (n, W), "fan"
                yield f"{q}.{s}.conv", (n, m["conv"]), ("n", 0.0, m["conv"] ** -0.5)
            yield f"{q}.q.norm", (nq_att,), "ln_w"
            if own:
                yield f"{q}.k.norm", (nk,), "ln_w"
            yield f"{q}.temp", (m["heads"],), ("n", 1.0, 0.2)
            yield f"{q}.g", (m["heads"], W), "fan"
            yield f"{q}.o", (W, m["heads"] * m["vdim"]), "fan"
        else:
            inner = m["heads"] * m["vdim"]
            for s, n in (("q", nk), ("k", nk), ("v", inner)):
                yield f"{q}.{s}", (n, W), "fan"
                yield f"{q}.{s}.conv", (n, m["conv"]), ("n", 0.0, m["conv"] ** -0.5)
            yield f"{q}.b", (m["heads"], W), "fan"
            yield f"{q}.a", (m["heads"], W), "fan"
            yield f"{q}.dt_bias", (m["heads"],), ("n", -1.0, 1.0)
            yield f"{q}.A_log", (m["heads"],), ("n", -1.0, 0.7)
            yield f"{q}.norm", (m["vdim"],), "ln_w"
            yield f"{q}.g", (inner, W), "fan"
            yield f"{q}.o", (W, inner), "fan"
        if L.get("mlp") is not None:
            yield f"{p}.norm2", (W,), "ln_w"
            yield f"{p}.mlp.up", (L["mlp"]["ff"], W), "fan"
            yield f"{p}.mlp.down", (W, L["mlp"]["ff"]), "fan"
    yield "final.norm", (W,), "ln_w"
    yield "head", (V, W), "fan"


def _botalorn_preset(width, vocab, heads, ff, n_blocks, window=512, kv_div=4):
    """``n_blocks`` x (attention, attention, delta, delta, attention <- keys / values of the block's second layer, delta), every layer
    with a dense feed-forward; head size 128."""
    d = 128
    att = dict(type="attention", heads=heads, kv_heads=max(1, heads // kv_div), dim=d, vdim=d, conv=4, window=window, mlp={"ff": ff})
    dlt = dict(type="delta", heads=heads, kv_heads=max(1, heads // 2), dim=d, vdim=d, conv=4, mlp={"ff": ff})
    layers = []
    for b in range(n_blocks):
        base = 6 * b
        layers += [dict(att), dict(att), dict(dlt), dict(dlt), dict(att, kv_from=base + 1), dict(dlt)]
    return botalorn_config(width, vocab, layers, streams=2, embed_scale=width ** 0.5)


PRESETS.update({
    "botalorn-tiny": botalorn_config(128, 320, [
        dict(type="attention", heads=4, kv_heads=2, dim=24, vdim=16, conv=3, window=20, mlp={"ff": 192}),
        dict(type="delta", heads=4, kv_heads=2, dim=24, vdim=16, conv=4, mlp={"ff": 192}),
        dict(type="attention", heads=4, kv_heads=2, dim=24, vdim=16, conv=2, window=33, kv_from=0, mlp=None),
        dict(type="delta", heads=2, kv_heads=2, dim=32, vdim=40, conv=3, mlp={"ff": 160})], streams=3, embed_scale=8.0),
    # sizes whose layers resemble a served model's (random weights), beside gptj-like-* of equal width and depth
    "botalorn-2k": _botalorn_preset(2048, 32000, 16, 4096, 3),
    "botalorn-4k": _botalorn_preset(4096, 32000, 32, 6144, 3),
})


def zenorax_config(width: int, vocab: int, layers, taps: int = 4, embed_scale: float = 1.0, softcap: float = 25.0,
                   eps: float = 1e-6) -> dict:
    """config.json of a Zenorax model.  ``layers``: one dict per layer,
    {"type": "latent_attention", heads, dim, rot_dim, vdim, kv_rank, q_rank, optionally scale, base, scaling} |
    {"type": "attention", heads, kv_heads, dim, optionally rot_dims, scale, base, scaling} | {"type": "hgrn2", heads, dim, vdim},
    each with "mlp": None | {"experts", "top", "ff", optionally "groups", "keep"}.  ``scaling``: None | {"factor"} (linear) |
    {"factor", "original", "fast", "slow"} (YaRN)."""
    out = []
    for L in layers:
        t = L["type"]
        if t == "latent_attention":
            rot = {"base": L.get("base", 10000.0), "dims": L.get("rot_dims", L["rot_dim"])}
            if L.get("scaling"):
                rot["scaling"] = dict(L["scaling"])
            m = {k: L[k] for k in ("heads", "dim", "rot_dim", "vdim", "kv_rank", "q_rank")}
            m.update(rot=rot, scale=L.get("scale", (L["dim"] + L["rot_dim"]) ** -0.5))
        elif t == "attention":
            rot = {"base": L.get("base", 10000.0), "dims": L.get("rot_dims", L["dim"])}
            if L.get("scaling"):
                rot["scaling"] = dict(L["scaling"])
            m = {"heads": L["heads"], "kv_heads": L["kv_heads"], "dim": L["dim"], "vdim": L["dim"], "rot": rot,
                 "scale": L.get("scale", L["dim"] ** -0.5)}
        else:
            m = {k: L[k] for k in ("heads", "dim", "vdim")}
        f = L.get("mlp")
        mlp = None
        if f is not None:
            mlp = {"kind": "moe", "expert": {"ff": f["ff"]},
                   "router": {"experts": f["experts"], "top": f["top"], "groups": {"count": f.get("groups", 1), "keep": f.get("keep", 1)}}}
        out.append({"type": t, "mixer": m, "mlp": mlp})
    return {"architecture": "Zenorax", "vocab": vocab, "width": width, "norm": {"eps": eps}, "embedding": {"scale": embed_scale},
            "canon": {"taps": taps}, "logit_softcap": softcap, "layers": out}


def _zenorax_shapes(cfg: dict):
    W, V, taps = cfg["width"], cfg["vocab"], cfg["canon"]["taps"]
    yield "embed", (V, W), ("n", 0.0, 1.0 / cfg["embedding"]["scale"])
    for i, L in enumerate(cfg["layers"]):
        p, m = f"l{i}", L["mixer"]
        q = f"{p}.mix"
        for nm in ("norm1", "norm1b") + (("norm2", "norm2b") if L.get("mlp") is not None else ()):
            yield f"{p}.{nm}", (W,), "ln_w"
        yield f"{p}.canon1", (W, taps), ("n", 0.0, 0.3)
        yield f"{p}.dwa", (i + 2,), ("dwa", 0.0, 0.0)
        if L["type"] == "latent_attention":
            H, d, r, dv, R, Q = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"], m["q_rank"]
            yield f"{q}.dq", (Q, W), "fan"
            yield f"{q}.dq.norm", (Q,), "ln_w"
            yield f"{q}.uq", (H * (d + r), Q), "fan"
            yield f"{q}.dkv", (R + r, W), "fan"
            yield f"{q}.dkv.norm", (R,), "ln_w"
            yield f"{q}.uk", (H * d, R), "fan"
            yield f"{q}.uv", (H * dv, R), "fan"
            yield f"{q}.g", (H * dv, W), "fan"
            yield f"{q}.o", (W, H * dv), "fan"
        elif L["type"] == "attention":
            H, G, d = m["heads"], m["kv_heads"], m["dim"]
            yield f"{q}.q", (H * d, W), "fan"
            yield f"{q}.k", (G * d, W), "fan"
            yield f"{q}.sink", (H,), ("n", 0.0, 1.0)
            yield f"{q}.o", (W, H * d), "fan"
        else:
            H, d, dv = m["heads"], m["dim"], m["vdim"]
            yield f"{q}.q", (H * d, W), "fan"
            yield f"{q}.f", (H * d, W), "fan"
            yield f"{q}.f.b", (H * d,), ("n", 1.0, 1.0)
            yield f"{q}.lower", (H * d,), ("u", 0.0, 0.9)
            yield f"{q}.v", (H * dv, W), "fan"
            yield f"{q}.norm", (dv,), "ln_w"
            yield f"{q}.o", (W, H * dv), "fan"
        f = L.get("mlp")
        if f is not None:
            E, F = f["router"]["experts"], f["expert"]["ff"]
            yield f"{p}.mlp.router", (E, W), "fan2"
            yield f"{p}.mlp.correction", (E,), ("n", 0.0, 0.1)
            for e in range(E):
                yield f"{p}.mlp.e{e}.up", (F, W), "fan"
                yield f"{p}.mlp.e{e}.down", (W, F), "fan"
    yield "final.norm", (W,), "ln_w"


def _zenorax_preset(width, vocab, heads, n_blocks, experts=16, top=4, groups=4, keep=2, eff=1024):
    """``n_blocks`` x (latent attention, sink attention, HGRN2), every layer with routed experts; head size 128.  The latent
    row is 192 + 64 = 256 numbers, a size the tensor-core multi-query kernels take."""
    mlp = dict(experts=experts, top=top, groups=groups, keep=keep, ff=eff)
    lat = dict(type="latent_attention", heads=heads, dim=128, rot_dim=64, vdim=128, kv_rank=192, q_rank=width // 2,
               scaling={"factor": 4.0, "original": 2048, "fast": 32.0, "slow": 1.0}, mlp=mlp)
    att = dict(type="attention", heads=heads, kv_heads=max(1, heads // 4), dim=128, scaling={"factor": 2.0}, mlp=mlp)
    rec = dict(type="hgrn2", heads=heads, dim=128, vdim=128, mlp=mlp)
    return zenorax_config(width, vocab, [dict(L) for _ in range(n_blocks) for L in (lat, att, rec)], taps=4, embed_scale=width ** 0.5)


PRESETS.update({
    "zenorax-tiny": zenorax_config(128, 320, [
        dict(type="latent_attention", heads=4, dim=16, rot_dim=8, vdim=24, kv_rank=40, q_rank=48,
             scaling={"factor": 4.0, "original": 64, "fast": 16.0, "slow": 2.0}, mlp=dict(experts=8, top=2, groups=4, keep=2, ff=32)),
        dict(type="attention", heads=4, kv_heads=2, dim=24, rot_dims=16, scaling={"factor": 2.0}, mlp=None),
        dict(type="hgrn2", heads=2, dim=24, vdim=40, mlp=dict(experts=4, top=1, groups=1, keep=1, ff=48)),
        dict(type="latent_attention", heads=2, dim=24, rot_dim=16, vdim=16, kv_rank=48, q_rank=32, mlp=dict(experts=6, top=3, groups=2, keep=1, ff=32))],
        taps=3, embed_scale=8.0),
    # sizes whose layers resemble a served model's (random weights), beside gptj-like-* of equal width and depth
    "zenorax-2k": _zenorax_preset(2048, 32000, 16, 6),
    "zenorax-4k": _zenorax_preset(4096, 32000, 32, 6, experts=32, eff=1536, groups=8, keep=4),
})


def _shapes(cfg: dict) -> Iterator[Tuple[str, Tuple[int, ...], str]]:
    """(name, shape, kind) for every tensor of the family; kind in {w, b, ln_w, ln_b, emb} (and, for architectures whose
    activations must keep unit scale without trained weights: unit, fan, fan2, alpha, ls)."""
    mt = cfg.get("model_type") or str(cfg["architecture"]).lower()
    if mt == "bedovik":
        yield from _bedovik_shapes(cfg)
    elif mt == "ninelix":
        yield from _ninelix_shapes(cfg)
    elif mt == "botalorn":
        yield from _botalorn_shapes(cfg)
    elif mt == "zenorax":
        yield from _zenorax_shapes(cfg)
    elif mt == "gptj":
        H, L, V = cfg["n_embd"], cfg["n_layer"], cfg["vocab_size"]
        F = cfg.get("n_inner") or 4 * H
        yield "transformer.wte.weight", (V, H), "emb"
        for i in range(L):
            p = f"transformer.h.{i}"
            yield f"{p}.ln_1.weight", (H,), "ln_w"
            yield f"{p}.ln_1.bias", (H,), "ln_b"
            for n in ("q_proj", "k_proj", "v_proj", "out_proj"):
                yield f"{p}.attn.{n}.weight", (H, H), "w"
            yield f"{p}.mlp.fc_in.weight", (F, H), "w"
            yield f"{p}.mlp.fc_in.bias", (F,), "b"
            yield f"{p}.mlp.fc_out.weight", (H, F), "w"
            yield f"{p}.mlp.fc_out.bias", (H,), "b"
        yield "transformer.ln_f.weight", (H,), "ln_w"
        yield "transformer.ln_f.bias", (H,), "ln_b"
        yield "lm_head.weight", (V, H), "w"
        yield "lm_head.bias", (V,), "b"
    elif mt == "gpt_bigcode":
        H, L, V, P = cfg["n_embd"], cfg["n_layer"], cfg["vocab_size"], cfg["n_positions"]
        F = cfg.get("n_inner") or 4 * H
        d = H // cfg["n_head"]
        yield "transformer.wte.weight", (V, H), "emb"
        yield "transformer.wpe.weight", (P, H), "emb"
        for i in range(L):
            p = f"transformer.h.{i}"
            for ln in ("ln_1", "ln_2"):
                yield f"{p}.{ln}.weight", (H,), "ln_w"
                yield f"{p}.{ln}.bias", (H,), "ln_b"
            yield f"{p}.attn.c_attn.weight", (H + 2 * d, H), "w"
            yield f"{p}.attn.c_attn.bias", (H + 2 * d,), "b"
            yield f"{p}.attn.c_proj.weight", (H, H), "w"
            yield f"{p}.attn.c_proj.bias", (H,), "b"
            yield f"{p}.mlp.c_fc.weight", (F, H), "w"
            yield f"{p}.mlp.c_fc.bias", (F,), "b"
            yield f"{p}.mlp.c_proj.weight", (H, F), "w"
            yield f"{p}.mlp.c_proj.bias", (H,), "b"
        yield "transformer.ln_f.weight", (H,), "ln_w"
        yield "transformer.ln_f.bias", (H,), "ln_b"
    elif mt == "gpt2":
        H, L, V, P = cfg["n_embd"], cfg["n_layer"], cfg["vocab_size"], cfg["n_positions"]
        F = cfg.get("n_inner") or 4 * H
        yield "transformer.wte.weight", (V, H), "emb"
        yield "transformer.wpe.weight", (P, H), "emb"
        for i in range(L):
            p = f"transformer.h.{i}"
            for ln in ("ln_1", "ln_2"):
                yield f"{p}.{ln}.weight", (H,), "ln_w"
                yield f"{p}.{ln}.bias", (H,), "ln_b"
            yield f"{p}.attn.c_attn.weight", (H, 3 * H), "w"   # Conv1D: [in, out]
            yield f"{p}.attn.c_attn.bias", (3 * H,), "b"
            yield f"{p}.attn.c_proj.weight", (H, H), "w"
            yield f"{p}.attn.c_proj.bias", (H,), "b"
            yield f"{p}.mlp.c_fc.weight", (H, F), "w"
            yield f"{p}.mlp.c_fc.bias", (F,), "b"
            yield f"{p}.mlp.c_proj.weight", (F, H), "w"
            yield f"{p}.mlp.c_proj.bias", (H,), "b"
        yield "transformer.ln_f.weight", (H,), "ln_w"
        yield "transformer.ln_f.bias", (H,), "ln_b"
    elif mt == "opt":
        H, L, V, P, F = (cfg["hidden_size"], cfg["num_hidden_layers"], cfg["vocab_size"],
                         cfg["max_position_embeddings"], cfg["ffn_dim"])
        yield "model.decoder.embed_tokens.weight", (V, H), "emb"
        yield "model.decoder.embed_positions.weight", (P + 2, H), "emb"
        for i in range(L):
            p = f"model.decoder.layers.{i}"
            for n in ("q_proj", "k_proj", "v_proj", "out_proj"):
                yield f"{p}.self_attn.{n}.weight", (H, H), "w"
                yield f"{p}.self_attn.{n}.bias", (H,), "b"
            for ln in ("self_attn_layer_norm", "final_layer_norm"):
                yield f"{p}.{ln}.weight", (H,), "ln_w"
                yield f"{p}.{ln}.bias", (H,), "ln_b"
            yield f"{p}.fc1.weight", (F, H), "w"
            yield f"{p}.fc1.bias", (F,), "b"
            yield f"{p}.fc2.weight", (H, F), "w"
            yield f"{p}.fc2.bias", (H,), "b"
        yield "model.decoder.final_layer_norm.weight", (H,), "ln_w"
        yield "model.decoder.final_layer_norm.bias", (H,), "ln_b"
    elif mt == "llama":
        H, L, V, F = cfg["hidden_size"], cfg["num_hidden_layers"], cfg["vocab_size"], cfg["intermediate_size"]
        hq, hkv = cfg["num_attention_heads"], cfg.get("num_key_value_heads") or cfg["num_attention_heads"]
        d = cfg.get("head_dim") or H // hq
        yield "model.embed_tokens.weight", (V, H), "emb"
        for i in range(L):
            p = f"model.layers.{i}"
            yield f"{p}.input_layernorm.weight", (H,), "ln_w"
            yield f"{p}.post_attention_layernorm.weight", (H,), "ln_w"
            yield f"{p}.self_attn.q_proj.weight", (hq * d, H), "w"
            yield f"{p}.self_attn.k_proj.weight", (hkv * d, H), "w"
            yield f"{p}.self_attn.v_proj.weight", (hkv * d, H), "w"
            yield f"{p}.self_attn.o_proj.weight", (H, hq * d), "w"
            yield f"{p}.mlp.gate_proj.weight", (F, H), "w"
            yield f"{p}.mlp.up_proj.weight", (F, H), "w"
            yield f"{p}.mlp.down_proj.weight", (H, F), "w"
        yield "model.norm.weight", (H,), "ln_w"
        if not cfg.get("tie_word_embeddings", False):
            yield "lm_head.weight", (V, H), "w"
    else:
        raise KeyError(mt)


def checkpoint_bytes(cfg: dict, elem_bytes: int = 2) -> int:
    n = 0
    for _, shape, _ in _shapes(cfg):
        k = 1
        for s in shape:
            k *= s
        n += k
    return n * elem_bytes


def write_random_checkpoint(path, preset_or_cfg, dtype=torch.float16, device=None, seed: int = 0,
                            shard_bytes: int = 2 << 30, std: float = 0.02) -> Path:
    """Create ``path/config.json`` and ``path/model-XXXXX.safetensors``; idempotent (a marker
    file records completion so concurrent ranks / reruns can skip the work)."""
    cfg = dict(PRESETS[preset_or_cfg]) if isinstance(preset_or_cfg, str) else dict(preset_or_cfg)
    path = Path(path)
    done = path / ".complete"
    if done.exists():
        return path
    path.mkdir(parents=True, exist_ok=True)
    cfg.setdefault("torch_dtype", str(dtype).replace("torch.", ""))
    (path / "config.json").write_text(json.dumps(cfg, indent=1))
    if device is None:
        device = "cuda" if torch.cuda.is_available() else "cpu"
    gen = torch.Generator(device=device)
    gen.manual_seed(seed)
    shard: Dict[str, torch.Tensor] = {}
    size, idx, total = 0, 0, 0
    weight_map: Dict[str, str] = {}

    def flush():
        nonlocal shard, size, idx
        if shard:
            fname = f"model-{idx:05d}.safetensors"
            save_file({k: v.cpu() for k, v in shard.items()}, str(path / fname), metadata={"format": "pt"})
            weight_map.update({k: fname for k in shard})
            idx += 1
            shard, size = {}, 0

    for name, shape, kind in _shapes(cfg):
        if isinstance(kind, tuple):      # ("n", mean, std): normal; ("u", lo, hi): uniform; ("hcmix", diagonal, std): near a scaled identity;
            # ("dwa", ..): depth-averaging weights
            r = (torch.rand if kind[0] == "u" else torch.randn)(shape, generator=gen, device=device, dtype=torch.float32)
            if kind[0] == "hcmix":
                t = kind[1] * torch.eye(shape[0], device=device) + kind[2] * r
            elif kind[0] == "dwa":      # depth-averaging weights: mostly the newest layer output, a little of every older one
                t = 0.1 * r.abs() / shape[0]
                t[-1] = 1.0
            else:
                t = kind[1] + kind[2] * r if kind[0] == "n" else kind[1] + (kind[2] - kind[1]) * r
        elif kind in ("unit", "fan", "fan2", "alpha", "ls"):
            r = torch.randn(shape, generator=gen, device=device, dtype=torch.float32)
            t = {"unit": r, "fan": r * shape[-1] ** -0.5 if shape else r, "fan2": 2.0 * r * shape[-1] ** -0.5 if shape else r,
                 "alpha": 0.7 + 0.1 * r, "ls": 0.4 + 0.1 * r}[kind]
        elif kind == "ln_w":
            t = 1.0 + 0.05 * torch.randn(shape, generator=gen, device=device, dtype=torch.float32)
        elif kind in ("b", "ln_b"):
            t = 0.02 * torch.randn(shape, generator=gen, device=device, dtype=torch.float32)
        else:
            t = std * torch.randn(shape, generator=gen, device=device, dtype=torch.float32)
        shard[name] = t.to(dtype)
        size += shard[name].numel() * shard[name].element_size()
        total += shard[name].numel() * shard[name].element_size()
        if size >= shard_bytes:
            flush()
    flush()
    (path / "model.safetensors.index.json").write_text(
        json.dumps({"metadata": {"total_size": total}, "weight_map": weight_map}, indent=1))
    done.write_text("ok")
    return path

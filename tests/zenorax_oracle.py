"""Plain float64 implementation of the Zenorax design: one function per mechanism, whole sequences, explicit loops where
a loop is the clearest form, no cache, no state objects, nothing imported from the package.  ``p`` maps tensor names to
float64 tensors, ``cfg`` is the parsed config.json.  The tests compare the framework against these functions."""
import math

import torch

F64 = torch.float64


def rms_div(x, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


# ----------------------------------------------------------------------------------------------- rotary positions
def rotary_frequencies(rot):
    """(frequency per pair [dims / 2], factor on cos and sin) for a ``rot`` entry {base, dims, scaling}."""
    dims, base = int(rot["dims"]), float(rot["base"])
    i = torch.arange(dims // 2, dtype=F64)
    f = base ** (-2.0 * i / dims)
    sc = rot.get("scaling")
    if not sc:
        return f, 1.0
    factor = float(sc["factor"])
    if "original" not in sc:                       # linear: every frequency divided by the factor
        return f / factor, 1.0

    def turns_to_dim(t):
        return dims * math.log(float(sc["original"]) / (2.0 * math.pi * t)) / (2.0 * math.log(base))

    lo = max(math.floor(turns_to_dim(float(sc["fast"]))), 0)
    hi = min(math.ceil(turns_to_dim(float(sc["slow"]))), dims - 1)
    ramp = ((i - lo) / max(hi - lo, 0.001)).clamp(0.0, 1.0)
    return f / factor * ramp + f * (1.0 - ramp), 0.1 * math.log(factor) + 1.0


def rotate(x, positions, rot, interleaved):
    """x [T, heads, d]: the first rot.dims channels of every head are rotated, the rest pass."""
    dims = int(rot["dims"])
    f, mag = rotary_frequencies(rot)
    ang = positions.to(F64)[:, None] * f[None, :]
    c, s = (torch.cos(ang) * mag)[:, None, :], (torch.sin(ang) * mag)[:, None, :]
    part, rest = x[..., :dims], x[..., dims:]
    if interleaved:
        u, v = part[..., 0::2], part[..., 1::2]
        out = torch.stack((u * c - v * s, v * c + u * s), dim=-1).flatten(-2)
    else:
        u, v = part[..., :dims // 2], part[..., dims // 2:]
        out = torch.cat((u * c - v * s, v * c + u * s), dim=-1)
    return torch.cat((out, rest), dim=-1)


# ----------------------------------------------------------------------------------------------- softmax attention
def causal_softmax_attention(q, k, v, scale, sink=None):
    """q [T, H, dk], k [T, H, dk], v [T, H, dv] (already one key / value head per query head).  ``sink`` [H]: one more
    term exp(sink) in every denominator."""
    T, H, _ = q.shape
    out = torch.zeros(T, H, v.shape[-1], dtype=F64)
    for h in range(H):
        for i in range(T):
            s = (k[:i + 1, h] @ q[i, h]) * scale
            m = s.max() if sink is None else torch.maximum(s.max(), sink[h])
            e = torch.exp(s - m)
            den = e.sum() + (0.0 if sink is None else torch.exp(sink[h] - m))
            out[i, h] = (e / den) @ v[:i + 1, h]
    return out


def latent_attention(h, positions, p, pre, m, eps):
    T = h.shape[0]
    H, d, r, dv, R = int(m["heads"]), int(m["dim"]), int(m["rot_dim"]), int(m["vdim"]), int(m["kv_rank"])
    cq = rms_div(h @ p[pre + "dq"].T, eps) * p[pre + "dq.norm"]
    q = (cq @ p[pre + "uq"].T).view(T, H, d + r)
    kv = h @ p[pre + "dkv"].T
    c = rms_div(kv[:, :R], eps) * p[pre + "dkv.norm"]
    k_rot = rotate(kv[:, None, R:], positions, m["rot"], True)                # one rotated part for all heads
    q_rot = rotate(q[..., d:], positions, m["rot"], True)
    k = torch.cat(((c @ p[pre + "uk"].T).view(T, H, d), k_rot.expand(T, H, r)), dim=-1)
    qq = torch.cat((q[..., :d], q_rot), dim=-1)
    v = (c @ p[pre + "uv"].T).view(T, H, dv)
    o = causal_softmax_attention(qq, k, v, float(m["scale"])).reshape(T, H * dv)
    o = o * torch.sigmoid(h @ p[pre + "g"].T)
    return o @ p[pre + "o"].T


def sink_attention(h, positions, p, pre, m, eps):
    T = h.shape[0]
    H, G, d = int(m["heads"]), int(m["kv_heads"]), int(m["dim"])
    q = (h @ p[pre + "q"].T).view(T, H, d)
    k = (h @ p[pre + "k"].T).view(T, G, d)
    v = k                                                                       # no value projection: the raw keys serve
    q = rms_div(rotate(q, positions, m["rot"], False), eps)
    kn = rms_div(rotate(k, positions, m["rot"], False), eps)
    rep = H // G
    o = causal_softmax_attention(q, kn.repeat_interleave(rep, dim=1), v.repeat_interleave(rep, dim=1), float(m["scale"]),
                                 sink=p[pre + "sink"])
    return o.reshape(T, H * d) @ p[pre + "o"].T


# ----------------------------------------------------------------------------------------------- gated linear recurrence
def hgrn2(h, p, pre, m, eps):
    T = h.shape[0]
    H, d, dv = int(m["heads"]), int(m["dim"]), int(m["vdim"])
    q = torch.nn.functional.silu(h @ p[pre + "q"].T).view(T, H, d)
    v = (h @ p[pre + "v"].T).view(T, H, dv)
    low = p[pre + "lower"]
    f = (low + (1.0 - low) * torch.sigmoid(h @ p[pre + "f"].T + p[pre + "f.b"])).view(T, H, d)
    S = torch.zeros(H, d, dv, dtype=F64)
    o = torch.zeros(T, H, dv, dtype=F64)
    for t in range(T):
        S = f[t][:, :, None] * S + (1.0 - f[t])[:, :, None] * v[t][:, None, :]
        o[t] = torch.einsum("hkv,hk->hv", S, q[t])
    o = rms_div(o, eps) * p[pre + "norm"]
    return o.reshape(T, H * dv) @ p[pre + "o"].T


# ----------------------------------------------------------------------------------------------- routed experts
def route(z, correction, top, groups, keep):
    """z [E] router logits of one token -> (chosen expert indices, their weights)."""
    E = z.shape[0]
    s = torch.sigmoid(z)
    choice = s + correction
    per = E // groups
    gscore = torch.stack([torch.sort(choice[g * per:(g + 1) * per], descending=True).values[:2].sum() for g in range(groups)])
    kept = torch.sort(gscore, descending=True, stable=True).indices[:keep].tolist()
    masked = torch.full_like(choice, -math.inf)
    for g in kept:
        masked[g * per:(g + 1) * per] = choice[g * per:(g + 1) * per]
    idx = torch.sort(masked, descending=True, stable=True).indices[:top]
    return idx, s[idx]


def experts(h, p, pre, f):
    r = f["router"]
    E, top = int(r["experts"]), int(r["top"])
    g = r.get("groups") or {"count": 1, "keep": 1}
    out = torch.zeros_like(h)
    z = h @ p[pre + "router"].T
    for t in range(h.shape[0]):
        idx, w = route(z[t], p[pre + "correction"], top, int(g["count"]), int(g["keep"]))
        for e, we in zip(idx.tolist(), w):
            a = torch.relu(p[f"{pre}e{e}.up"] @ h[t]) ** 2
            out[t] += we * (p[f"{pre}e{e}.down"] @ a)
    return out


# ----------------------------------------------------------------------------------------------- layer and model
def input_convolution(h, w):
    """h + conv(h): causal over time per channel, zeros before the start.  w [width, taps]."""
    T, taps = h.shape[0], w.shape[1]
    out = h.clone()
    for t in range(T):
        for j in range(taps):
            s = t - taps + 1 + j
            if s >= 0:
                out[t] += w[:, j] * h[s]
    return out


MIXERS = {"latent_attention": lambda h, pos, p, pre, m, eps: latent_attention(h, pos, p, pre, m, eps),
          "attention": lambda h, pos, p, pre, m, eps: sink_attention(h, pos, p, pre, m, eps),
          "hgrn2": lambda h, pos, p, pre, m, eps: hgrn2(h, p, pre, m, eps)}


def forward(cfg, p, tokens, taps=None):
    """Logits [T, vocab] of one whole sequence; ``taps`` receives what leaves every layer."""
    eps = float(cfg["norm"]["eps"])
    tok = torch.as_tensor(tokens, dtype=torch.long)
    pos = torch.arange(tok.shape[0])
    x = p["embed"][tok] * float(cfg.get("embedding", {}).get("scale", 1.0))
    history = [x]
    for i, lc in enumerate(cfg["layers"]):
        L = f"l{i}."
        h = rms_div(x, eps) * p[L + "norm1"]
        if (L + "canon1") in p:
            h = input_convolution(h, p[L + "canon1"])
        y = MIXERS[lc["type"]](h, pos, p, L + "mix.", lc["mixer"], eps)
        x = x + rms_div(y, eps) * p[L + "norm1b"]
        if lc.get("mlp") is not None:
            y = experts(rms_div(x, eps) * p[L + "norm2"], p, L + "mlp.", lc["mlp"])
            x = x + rms_div(y, eps) * p[L + "norm2b"]
        history.append(x)
        if (L + "dwa") in p:
            x = sum(p[L + "dwa"][j] * history[j] for j in range(len(history)))
        if taps is not None:
            taps.append(x.clone())
    z = (rms_div(x, eps) * p["final.norm"]) @ p["embed"].T
    cap = cfg.get("logit_softcap")
    return cap * torch.tanh(z / cap) if cap else z


def load_weights(path):
    """Every tensor of a checkpoint folder as float64."""
    from pathlib import Path

    from safetensors.torch import load_file

    out = {}
    for f in sorted(Path(path).glob("*.safetensors")):
        for k, v in load_file(str(f)).items():
            out[k] = v.double()
    return out

"""Plain float64 statement of the Botalorn design, one function per mechanism, whole sequences, explicit loops over
tokens; no cache, no state objects, nothing imported from the package.  The tests compare the framework against it.

Notation: T tokens, W width, S residual streams.  ``P`` is a dict of one mixer's tensors without the layer prefix
("q", "q.conv", "q.norm", ...), ``m`` the mixer's entry of the configuration.
"""
import math

import numpy as np

F = np.float64


def rms_div(x, eps):
    return x / np.sqrt((x * x).mean(-1, keepdims=True) + eps)


def sinusoid(n, width):
    """Row p: entry 2i = sin(p * 10000^(-2i / width)), entry 2i + 1 = cos of the same angle."""
    out = np.zeros((n, width), F)
    for p in range(n):
        for c in range(width):
            ang = p * 10000.0 ** (-(2 * (c // 2)) / width)
            out[p, c] = math.sin(ang) if c % 2 == 0 else math.cos(ang)
    return out


def embedding(tokens, table, scale):
    return table[np.asarray(tokens)].astype(F) * scale + sinusoid(len(tokens), table.shape[1])


def token_shift(h, mu):
    """h_t + (h_(t-1) - h_t) * mu, with the unshifted previous row (zeros before the first)."""
    prev = np.zeros_like(h)
    prev[1:] = h[:-1]
    return h + (prev - h) * mu


def causal_conv(u, w):
    """u [T, C], w [C, taps]: y_t = sum_j w[:, j] u_(t - taps + 1 + j); the last tap is the current token's."""
    T, C = u.shape
    taps = w.shape[1]
    y = np.zeros((T, C), F)
    for t in range(T):
        for j in range(taps):
            s = t - taps + 1 + j
            if s >= 0:
                y[t] += w[:, j] * u[s]
    return y


def silu(x):
    return x / (1.0 + np.exp(-x))


def sigmoid(x):
    return 1.0 / (1.0 + np.exp(-x))


def softplus(x):
    return np.log1p(np.exp(-np.abs(x))) + np.maximum(x, 0.0)


def attention_keys_values(h, P, m, eps):
    """What an attention layer with projections of its own keeps per token: normed keys, raw and normed values."""
    G, D, Dv = m["kv_heads"], m["dim"], m["vdim"]
    T = h.shape[0]
    k = causal_conv(h @ P["k"].T, P["k.conv"])
    k = rms_div(k, eps) * P["k.norm"]                       # over the whole projection, all heads at once
    v_raw = causal_conv(h @ P["v"].T, P["v.conv"]).reshape(T, G, Dv)
    v = rms_div(v_raw, eps)                                  # per head, no weight
    return k.reshape(T, G, D), v_raw, v


def head_slopes(H):
    return np.array([2.0 ** (-8.0 * (h + 1) / H) for h in range(H)], F)


def window_softmax(q, keys, values, factor, slopes, window):
    """q [T, H, D], keys [T, G, D], values [T, G, Dv]: query i of head h sees keys j with 0 <= i - j < window (all j <= i without
    a window); score = factor[h] q_i . k_j - slopes[h] (i - j); ordinary softmax; returns [T, H, Dv]."""
    T, H, _ = q.shape
    G = keys.shape[1]
    out = np.zeros((T, H, values.shape[2]), F)
    for hd in range(H):
        g = hd // (H // G)
        for i in range(T):
            lo = 0 if window is None else max(0, i - window + 1)
            js = np.arange(lo, i + 1)
            s = (keys[js, g] @ q[i, hd]) * factor[hd] - slopes[hd] * (i - js)
            p = np.exp(s - s.max())
            p /= p.sum()
            out[i, hd] = (p[:, None] * values[js, g]).sum(0)
    return out


def attention_mixer(h, P, m, eps, keys=None, values=None):
    """Windowed softmax attention.  ``keys`` / ``values`` given: the layer borrows them (and has no k / v tensors)."""
    H, D = m["heads"], m["dim"]
    T = h.shape[0]
    q = causal_conv(h @ P["q"].T, P["q.conv"])
    q = (rms_div(q, eps) * P["q.norm"]).reshape(T, H, D)
    if keys is None:
        keys, _, values = attention_keys_values(h, P, m, eps)
    window = (m.get("mask") or {}).get("size")
    out = window_softmax(q, keys, values, m["scale"] * P["temp"], head_slopes(H), window)
    out = out * sigmoid(h @ P["g"].T)[:, :, None]            # one gate per head
    return out.reshape(T, -1) @ P["o"].T


def delta_rule(q, k, v, decay, beta):
    """q, k [T, G, D], v [T, H, Dv], decay, beta [T, H].  Per head, token by token, in this order:
    S <- decay S ;  u = beta (v - S^T k) ;  S <- S + k u^T ;  o = S^T q.  Returns (o [T, H, Dv], the last S [H, D, Dv])."""
    T, H, Dv = v.shape
    G, D = q.shape[1], q.shape[2]
    o = np.zeros((T, H, Dv), F)
    S = np.zeros((H, D, Dv), F)
    for t in range(T):
        for hd in range(H):
            g = hd // (H // G)
            S[hd] *= decay[t, hd]
            u = beta[t, hd] * (v[t, hd] - S[hd].T @ k[t, g])
            S[hd] += np.outer(k[t, g], u)
            o[t, hd] = S[hd].T @ q[t, g]
    return o, S


def unit(x, eps=1e-6):
    return x / np.sqrt((x * x).sum(-1, keepdims=True) + eps)


def delta_mixer(h, P, m, eps):
    H, G, D, Dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    T = h.shape[0]
    q = silu(causal_conv(h @ P["q"].T, P["q.conv"])).reshape(T, G, D)
    k = silu(causal_conv(h @ P["k"].T, P["k.conv"])).reshape(T, G, D)
    v = silu(causal_conv(h @ P["v"].T, P["v.conv"])).reshape(T, H, Dv)
    beta = sigmoid(h @ P["b"].T)                             # [T, H]
    decay = np.exp(-np.exp(P["A_log"]) * softplus(h @ P["a"].T + P["dt_bias"]))
    o, _ = delta_rule(unit(q) * D ** -0.5, unit(k), v, decay, beta)
    y = rms_div(o, eps) * P["norm"] * silu(h @ P["g"].T).reshape(T, H, Dv)
    return y.reshape(T, H * Dv) @ P["o"].T


def feed_forward(h, up, down):
    a = np.maximum(h @ up.T, 0.0)
    return (a * a) @ down.T


def hyper_read(xs, w_in):
    """xs [S, T, W] -> sum_s w_in[s] xs[s]."""
    return np.tensordot(w_in, xs, axes=(0, 0))


def hyper_write(xs, y, mix, w_out):
    """All streams at once from the old ones: x_t <- sum_s mix[s, t] x_s + w_out[t] y."""
    return np.tensordot(mix.T, xs, axes=(1, 0)) + w_out[:, None, None] * y[None]


def _sub(tensors, prefix):
    return {k[len(prefix):]: np.asarray(v, F) for k, v in tensors.items() if k.startswith(prefix)}


def forward(tokens, cfg, tensors):
    """Returns (logits [T, vocab], the summed residual stream after every layer [L, T, W])."""
    eps = cfg["norm"]["eps"]
    ten = {k: np.asarray(v, F) for k, v in tensors.items()}
    x0 = embedding(tokens, ten["embed"], cfg["embedding"]["scale"])
    S = cfg.get("streams")
    xs = np.stack([x0] * (S or 1))
    kept = {}
    after = []
    for i, lc in enumerate(cfg["layers"]):
        p, m = f"l{i}.", lc["mixer"]
        P = _sub(ten, p + "mix.")

        def sublayer(q, fn, xs):
            if S is None:
                return xs + fn(xs[0])[None]
            hc = _sub(ten, f"{p}hc{q}.")
            return hyper_write(xs, fn(hyper_read(xs, hc["in"])), hc["mix"], hc["out"])

        def mixer(u):
            h = rms_div(u, eps) * ten[p + "norm1"]
            if p + "shift" in ten:
                h = token_shift(h, ten[p + "shift"])
            if lc["type"] == "delta":
                return delta_mixer(h, P, m, eps)
            if "kv_from" in m and m["kv_from"] is not None:
                # the lender's keys as it keeps them; its values come un-normed and pass this layer's own value norm,
                # which has no weight: the result equals what the lender attends over
                k, v_raw, _ = kept[m["kv_from"]]
                return attention_mixer(h, P, m, eps, keys=k, values=rms_div(v_raw, eps))
            kept[i] = attention_keys_values(h, P, m, eps)
            return attention_mixer(h, P, m, eps, keys=kept[i][0], values=kept[i][2])

        xs = sublayer(1, mixer, xs)
        if lc.get("mlp") is not None:
            xs = sublayer(2, lambda u: feed_forward(rms_div(u, eps) * ten[p + "norm2"], ten[p + "mlp.up"], ten[p + "mlp.down"]), xs)
        after.append(xs.sum(0))
    x = rms_div(xs.sum(0), eps) * ten["final.norm"]
    return x @ ten["head"].T, np.stack(after)


def load_weights(path):
    """All tensors of a checkpoint folder as float64 arrays."""
    from pathlib import Path

    import torch
    from safetensors import safe_open

    out = {}
    for f in sorted(Path(path).glob("*.safetensors")):
        with safe_open(str(f), framework="pytorch") as h:
            for k in h.keys():
                out[k] = h.get_tensor(k).to(torch.float64).numpy()
    return out

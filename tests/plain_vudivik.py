"""A plain, slow implementation of the Vudivik decoder in numpy float64: one function per
mechanism, written from the design's equations and sharing nothing with the engine.

A layer is ``x += m * norm1(mixer(x)); x += m * norm2(ff(x))`` (the sublayers read x itself,
their outputs are RMS-normed).  The mixer is two mixers side by side on the same input: a
grouped-query softmax attention (biased projections, per-head query/key norm, rotate-half
rotary encoding on the first ``rot.dims`` features with frequency-dependent scaling, a
sliding window that also keeps the sequence's first tokens) and a selective scan (short
causal convolution, input-dependent step size, a diagonal state per channel); the result
is half the sum of their RMS-normed outputs.  The feed-forward is ``down(relu(up h)^2)``,
dense or as routed experts whose router adds a correction to the softmax scores for the
choice only and whose last outputs stand for identity experts.

Everything works on one sequence; ``state`` (a dict per layer run) carries keys, values,
the scan's state and the convolution's last inputs from call to call, so that a sequence
can be fed whole, in portions, or token by token.
"""
from __future__ import annotations

import math

import numpy as np

F = np.float64


def plain_rms_norm(x, weight, eps):
    x = np.asarray(x, F)
    return x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps) * np.asarray(weight, F)


def plain_rotary_frequencies(dims, base, scaling=None):
    """f_i = base^(-2i/dims); with scaling, by wavelength l = 2 pi / f: short ones stay, long
    ones are divided by the factor, those between are blended."""
    out = []
    for i in range(dims // 2):
        f = float(base) ** (-2.0 * i / dims)
        if scaling:
            factor, low, high = float(scaling["factor"]), float(scaling["low"]), float(scaling["high"])
            orig = float(scaling["original"])
            wavelength = 2.0 * math.pi / f
            if wavelength < orig / high:
                pass
            elif wavelength > orig / low:
                f = f / factor
            else:
                s = (orig / wavelength - low) / (high - low)
                f = (1.0 - s) * f / factor + s * f
        out.append(f)
    return np.asarray(out, F)


def plain_rotate(x, positions, freqs):
    """x: [tokens, heads, dim]; the first 2*len(freqs) features are rotated, feature i paired
    with feature i + len(freqs)."""
    x = np.array(x, F)
    half = len(freqs)
    if half == 0:
        return x
    ang = np.asarray(positions, F)[:, None] * freqs[None, :]          # [tokens, half]
    c, s = np.cos(ang)[:, None, :], np.sin(ang)[:, None, :]
    u, v = x[..., :half].copy(), x[..., half:2 * half].copy()
    x[..., :half] = u * c - v * s
    x[..., half:2 * half] = v * c + u * s
    return x


def plain_visible(i, j, size=None, keep_first=0):
    """Whether position i sees position j."""
    if j > i:
        return False
    if size is None:
        return True
    return (i - j < size) or (j < keep_first)


def plain_softmax(z):
    z = np.asarray(z, F)
    e = np.exp(z - z.max(axis=-1, keepdims=True))
    return e / e.sum(axis=-1, keepdims=True)


def plain_window_attention(h, p, cfg, eps, state):
    """The left mixer.  p: q, q.b, k, k.b, v, v.b, q.norm, k.norm, o.  state: {"k", "v"} lists
    of earlier rotated keys and values (position = index)."""
    H, G, D, VD = cfg["heads"], cfg["kv_heads"], cfg["dim"], cfg["vdim"]
    n = h.shape[0]
    start = len(state.setdefault("k", []))
    state.setdefault("v", [])
    pos = np.arange(start, start + n)
    q = (h @ p["q"].T + p["q.b"]).reshape(n, H, D)
    k = (h @ p["k"].T + p["k.b"]).reshape(n, G, D)
    v = (h @ p["v"].T + p["v.b"]).reshape(n, G, VD)
    q = plain_rms_norm(q, p["q.norm"], eps)
    k = plain_rms_norm(k, p["k.norm"], eps)
    rot = cfg.get("rot")
    if rot:
        freqs = plain_rotary_frequencies(rot["dims"], rot["base"], rot.get("scaling"))
        q = plain_rotate(q, pos, freqs)
        k = plain_rotate(k, pos, freqs)
    for t in range(n):
        state["k"].append(k[t])
        state["v"].append(v[t])
    mask = cfg.get("mask") or {}
    size, keep = mask.get("size"), mask.get("keep_first", 0)
    scale = cfg["scale"]
    out = np.zeros((n, H, VD), F)
    per = H // G
    for t in range(n):
        i = start + t
        js = [j for j in range(i + 1) if plain_visible(i, j, size, keep)]
        for hh in range(H):
            g = hh // per
            keys = np.stack([state["k"][j][g] for j in js])
            vals = np.stack([state["v"][j][g] for j in js])
            w = plain_softmax(keys @ q[t, hh] * scale)
            out[t, hh] = w @ vals
    return out.reshape(n, H * VD) @ p["o"].T


def plain_silu(x):
    return x / (1.0 + np.exp(-x))


def plain_softplus(x):
    return np.where(x > 30.0, x, np.log1p(np.exp(np.minimum(x, 30.0))))


def plain_selective_scan(h, p, cfg, state):
    """The right mixer.  p: in, conv, conv.b, x, dt, dt.b, A_log, D, o.  state: {"conv": the
    last taps-1 inputs of the convolution [taps-1, inner], "S": [inner, n]}."""
    inner, N, R, taps = cfg["inner"], cfg["state"], cfg["dt_rank"], cfg["conv"]
    n = h.shape[0]
    xz = h @ p["in"].T
    x, z = xz[:, :inner], xz[:, inner:]
    past = state.get("conv")
    if past is None:
        past = np.zeros((taps - 1, inner), F)
    seq = np.concatenate([past, x], axis=0)                      # [taps-1+n, inner]
    xc = np.zeros((n, inner), F)
    for t in range(n):
        win = seq[t:t + taps]                                    # last row is the current token
        xc[t] = (win * p["conv"].T).sum(axis=0) + p["conv.b"]
    state["conv"] = seq[seq.shape[0] - (taps - 1):].copy() if taps > 1 else np.zeros((0, inner), F)
    xc = plain_silu(xc)
    proj = xc @ p["x"].T
    dt_in, B, C = proj[:, :R], proj[:, R:R + N], proj[:, R + N:R + 2 * N]
    dt = plain_softplus(dt_in @ p["dt"].T + p["dt.b"])           # [n, inner]
    A = -np.exp(p["A_log"])                                      # [inner, N]
    S = state.get("S")
    if S is None:
        S = np.zeros((inner, N), F)
    y = np.zeros((n, inner), F)
    for t in range(n):
        S = np.exp(dt[t][:, None] * A) * S + (dt[t] * xc[t])[:, None] * B[t][None, :]
        y[t] = S @ C[t] + p["D"] * xc[t]
    state["S"] = S
    return (y * plain_silu(z)) @ p["o"].T


def plain_parallel_mixer(h, p, cfg, eps, state):
    left = plain_window_attention(h, {k[5:]: v for k, v in p.items() if k.startswith("left.")
                                      and k != "left.out"},
                                  cfg["left"], eps, state.setdefault("left", {}))
    right = plain_selective_scan(h, {k[6:]: v for k, v in p.items() if k.startswith("right.")
                                     and k != "right.out"},
                                 cfg["right"], state.setdefault("right", {}))
    return 0.5 * (plain_rms_norm(left, p["left.out"], eps) + plain_rms_norm(right, p["right.out"], eps))


def plain_relu2_mlp(h, up, down):
    a = np.maximum(h @ up.T, 0.0)
    return (a * a) @ down.T


def plain_route(h, router, correction, top):
    """(chosen [tokens, top], weights [tokens, top]): softmax scores over all router outputs;
    the choice adds the correction, the weights do not; no renormalisation."""
    s = plain_softmax(h @ router.T)
    choice = s + correction
    chosen = np.argsort(-choice, axis=-1, kind="stable")[:, :top]
    return chosen, np.take_along_axis(s, chosen, axis=-1)


def plain_moe(h, p, cfg):
    r = cfg["router"]
    experts, identity, top = r["experts"], r.get("identity", 0), r["top"]
    chosen, weights = plain_route(h, p["router"], p["correction"], top)
    out = np.zeros_like(h)
    for t in range(h.shape[0]):
        for e, w in zip(chosen[t], weights[t]):
            if e >= experts:
                assert e < experts + identity
                out[t] += w * h[t]
            else:
                out[t] += w * plain_relu2_mlp(h[t:t + 1], p[f"e{e}.up"], p[f"e{e}.down"])[0]
    return out


def plain_feed_forward(h, p, cfg):
    if cfg["kind"] == "dense":
        return plain_relu2_mlp(h, p["up"], p["down"])
    if cfg["kind"] == "moe":
        return plain_moe(h, p, cfg)
    raise ValueError(cfg["kind"])


def _sub(tensors, prefix):
    return {k[len(prefix):]: np.asarray(v, F) for k, v in tensors.items() if k.startswith(prefix)}


def plain_layer(x, tensors, config, i, state):
    """One run of layer i on the rows x; returns the new residual."""
    layer = config["layers"][i]
    owner = i
    while config["layers"][owner].get("weights_of") is not None:
        owner = config["layers"][owner]["weights_of"]
    eps, m = config["norm"]["eps"], config["residual_mult"]
    if layer["type"] != "parallel":
        raise ValueError(layer["type"])
    y = plain_parallel_mixer(x, _sub(tensors, f"l{owner}.mix."), layer["mixer"], eps, state)
    x = x + m * plain_rms_norm(y, np.asarray(tensors[f"l{owner}.norm1"], F), eps)
    if layer.get("mlp") is not None:
        y = plain_feed_forward(x, _sub(tensors, f"l{owner}.mlp."), layer["mlp"])
        x = x + m * plain_rms_norm(y, np.asarray(tensors[f"l{owner}.norm2"], F), eps)
    return x


def plain_forward(tokens, tensors, config, states=None, layers_out=None):
    """Logits [len(tokens), vocab] of the next portion of one sequence.  ``states``: a list
    with one dict per layer, kept by the caller between portions (None: a fresh sequence)."""
    if states is None:
        states = [{} for _ in config["layers"]]
    x = np.asarray(tensors["embed"], F)[np.asarray(tokens)]
    for i in range(len(config["layers"])):
        x = plain_layer(x, tensors, config, i, states[i])
        if layers_out is not None:
            layers_out.append(x.copy())
    x = plain_rms_norm(x, np.asarray(tensors["final.norm"], F), config["norm"]["eps"])
    return x @ np.asarray(tensors["head"], F).T

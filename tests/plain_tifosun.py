"""Plain, slow implementation of the Tifosun decoder: one function per mechanism, written
token by token from the defining equations in float64 on the CPU.  It shares no code with
the engine; the tests compare the engine against it.

Notation: x is the residual [tokens, width]; a weight W is stored [out, in] and applied as
x @ W.T; positions count from 0.
"""
from __future__ import annotations

import math

import torch

F64 = torch.float64


def rms(x, eps):
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def norm_around_zero(x, w, eps):
    """RMS norm whose stored weight is an offset from one."""
    return rms(x, eps) * (1.0 + w)


def norm_plain(x, w, eps):
    return rms(x, eps) * w


def silu(z):
    return z * torch.sigmoid(z)


def gated_ffn(x, gate, up, down):
    return (silu(x @ gate.T) * (x @ up.T)) @ down.T


def soft_cap(z, cap):
    return cap * torch.tanh(z / cap)


# ------------------------------------------------------------------ matrix memory (mLSTM)
def mlstm_mixer(h, w, pre, cfg, eps, state=None):
    """h: [T, width] of one sequence.  state: None (start) or (S [H, dim, vdim], n [H, dim],
    m [H]); returns (output [T, width], new state).  One token at a time."""
    H, dim, vdim, cap = cfg["heads"], cfg["dim"], cfg["vdim"], cfg["gate_cap"]
    T = h.shape[0]
    q = (h @ w[pre + "q"].T).view(T, H, dim) * dim ** -0.5
    k = (h @ w[pre + "k"].T).view(T, H, dim)
    v = (h @ w[pre + "v"].T).view(T, H, vdim)
    i_gate = soft_cap(h @ w[pre + "i"].T + w[pre + "i.b"], cap)                   # [T, H]
    f_gate = torch.nn.functional.logsigmoid(soft_cap(h @ w[pre + "f"].T + w[pre + "f.b"], cap))
    if state is None:
        S = torch.zeros(H, dim, vdim, dtype=F64)
        n = torch.zeros(H, dim, dtype=F64)
        m = torch.zeros(H, dtype=F64)
    else:
        S, n, m = (t.clone() for t in state)
    out = torch.zeros(T, H, vdim, dtype=F64)
    for t in range(T):
        m_new = torch.maximum(f_gate[t] + m, i_gate[t])
        keep = torch.exp(f_gate[t] + m - m_new)
        take = torch.exp(i_gate[t] - m_new)
        S = keep[:, None, None] * S + take[:, None, None] * k[t][:, :, None] * v[t][:, None, :]
        n = keep[:, None] * n + take[:, None] * k[t]
        m = m_new
        num = torch.einsum("hdv,hd->hv", S, q[t])
        den = torch.maximum((n * q[t]).sum(-1).abs(), torch.exp(-m)) + 1e-6
        out[t] = num / den[:, None]
    o = rms(out, eps).reshape(T, H * vdim) * w[pre + "norm"]
    o = o * torch.sigmoid(h @ w[pre + "g"].T)
    return o @ w[pre + "o"].T, (S, n, m)


# ------------------------------------------------------------------ rotary positions
def rotate_interleaved(x, positions, dims, base):
    """x: [T, ..., D]; the first ``dims`` features in pairs (2i, 2i+1); the rest unchanged."""
    out = x.clone()
    for i in range(dims // 2):
        ang = positions.to(F64) * base ** (-2.0 * i / dims)
        shape = [-1] + [1] * (x.dim() - 2)
        c, s = torch.cos(ang).view(shape), torch.sin(ang).view(shape)
        u, v = x[..., 2 * i], x[..., 2 * i + 1]
        out[..., 2 * i] = u * c - v * s
        out[..., 2 * i + 1] = v * c + u * s
    return out


# ------------------------------------------------------------------ latent attention
def latent_rows(h, w, pre, cfg, eps, positions):
    """What a token leaves in the cache: the normed latent and the rotated shared key part."""
    rank, rot = cfg["kv_rank"], cfg["rot_dim"]
    d = h @ w[pre + "dkv"].T
    c = norm_plain(d[:, :rank], w[pre + "dkv.norm"], eps)
    kr = rotate_interleaved(d[:, rank:rank + rot], positions, cfg["rot"]["dims"],
                            cfg["rot"]["base"])
    return c, kr


def latent_attention_mixer(h, w, pre, cfg, eps, positions, past=None):
    """h: [T, width] at ``positions``; past: None or (c, kr) of the earlier tokens, in order.
    Returns (output, (c, kr) of all tokens so far)."""
    H, dim, rot, vdim, rank = cfg["heads"], cfg["dim"], cfg["rot_dim"], cfg["vdim"], cfg["kv_rank"]
    window = cfg["mask"]["size"] if cfg.get("mask") else None       # None: every key
    T = h.shape[0]
    q = (h @ w[pre + "q"].T).view(T, H, dim + rot)
    q_plain = q[..., :dim]
    q_rot = rotate_interleaved(q[..., dim:], positions, cfg["rot"]["dims"], cfg["rot"]["base"])
    c, kr = latent_rows(h, w, pre, cfg, eps, positions)
    if past is not None:
        c, kr = torch.cat([past[0], c]), torch.cat([past[1], kr])
    n_all = c.shape[0]
    first = n_all - T                                   # index of this call's first token
    k_plain = (c @ w[pre + "uk"].T).view(n_all, H, dim)
    val = (c @ w[pre + "uv"].T).view(n_all, H, vdim)
    out = torch.zeros(T, H, vdim, dtype=F64)
    for t in range(T):
        i = first + t
        lo = 0 if window is None else max(0, i - window + 1)
        for hh in range(H):
            s = (k_plain[lo:i + 1, hh] @ q_plain[t, hh] + kr[lo:i + 1] @ q_rot[t, hh]) * cfg["scale"]
            p = torch.softmax(s, dim=0)
            out[t, hh] = p @ val[lo:i + 1, hh]
    o = out.reshape(T, H * vdim) * torch.sigmoid(h @ w[pre + "g"].T)
    return o @ w[pre + "o"].T, (c, kr)


# ------------------------------------------------------------------ feed-forwards
def dense_ffn(h, w, pre):
    return gated_ffn(h, w[pre + "gate"], w[pre + "up"], w[pre + "down"])


def routed_ffn(h, w, pre, cfg):
    """Sigmoid scores, the ``top`` largest chosen, their scores (as they are) scale the
    expert's input; a shared expert is added for every token."""
    E, top = cfg["router"]["experts"], cfg["router"]["top"]
    scores = torch.sigmoid(h @ w[pre + "router"].T)                     # [T, E]
    out = torch.zeros(h.shape[0], w[pre + "e0.down"].shape[0], dtype=F64)
    for t in range(h.shape[0]):
        chosen = torch.topk(scores[t], top).indices.tolist()
        for e in chosen:
            p = f"{pre}e{e}."
            out[t] += gated_ffn(scores[t, e] * h[t:t + 1], w[p + "gate"], w[p + "up"],
                                w[p + "down"])[0]
    if cfg.get("shared"):
        p = pre + "shared."
        out += gated_ffn(h, w[p + "gate"], w[p + "up"], w[p + "down"])
    return out


# ------------------------------------------------------------------ the model
class PlainTifosun:
    """Runs one sequence; ``forward`` may be called with consecutive pieces of it."""

    def __init__(self, config: dict, weights: dict):
        self.cfg = config
        self.w = {k: v.to(F64) for k, v in weights.items()}
        self.eps = config["norm"]["eps"]
        self.reset()

    def reset(self):
        self.pos = 0
        self.state = [None] * len(self.cfg["layers"])

    def forward(self, tokens, collect=None):
        w, eps = self.w, self.eps
        T = len(tokens)
        positions = torch.arange(self.pos, self.pos + T)
        x = w["embed"][torch.as_tensor(tokens, dtype=torch.long)]
        for li, layer in enumerate(self.cfg["layers"]):
            p = f"l{li}."
            h = norm_around_zero(x, w[p + "norm1"], eps)
            kind = layer["type"]
            if kind in ("mlstm", "mlstm_2"):
                y, self.state[li] = mlstm_mixer(h, w, p + "mix.", layer["mixer"], eps,
                                                self.state[li])
            elif kind == "latent_attention":
                y, self.state[li] = latent_attention_mixer(h, w, p + "mix.", layer["mixer"], eps,
                                                           positions, self.state[li])
            else:
                raise ValueError(kind)
            x = x + norm_around_zero(y, w[p + "norm1b"], eps)
            mlp = layer.get("mlp")
            if mlp is not None:
                h = norm_around_zero(x, w[p + "norm2"], eps)
                if mlp["kind"] == "dense":
                    y = dense_ffn(h, w, p + "mlp.")
                elif mlp["kind"] == "moe":
                    y = routed_ffn(h, w, p + "mlp.", mlp)
                else:
                    raise ValueError(mlp["kind"])
                x = x + norm_around_zero(y, w[p + "norm2b"], eps)
            if collect is not None:
                collect.append(x.clone())
        self.pos += T
        return norm_around_zero(x, w["final.norm"], eps) @ w["head"].T

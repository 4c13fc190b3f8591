"""Small Vudivik configurations with random weights for the tests, and the plumbing to run
them through the plain implementation (the engine side is shared with the other decoder's
tests: ``tifosun_util.run_schedule`` and its comparisons)."""
from __future__ import annotations

import copy
import math

import numpy as np
import torch

import plain_vudivik as P
from tifosun_util import assert_close, relative_error, row_errors, run_schedule, tokens  # noqa: F401


def left(heads=4, kv_heads=2, dim=24, vdim=40, size=11, keep_first=3, rot_dims=16, base=10000.0,
         scaling=None, scale=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim,
         "scale": dim ** -0.5 if scale is None else scale}
    if size is not None:
        m["mask"] = {"size": size, "keep_first": keep_first}
    if rot_dims is not None:
        m["rot"] = {"base": base, "dims": rot_dims}
        if scaling is not None:
            m["rot"]["scaling"] = dict(scaling)
    return m


def right(inner=48, state=6, dt_rank=5, conv=3):
    return {"inner": inner, "state": state, "dt_rank": dt_rank, "conv": conv}


def dense(ff=72):
    return {"kind": "dense", "ff": ff}


def moe(experts=5, identity=2, top=3, ff=24):
    return {"kind": "moe", "router": {"experts": experts, "identity": identity, "top": top},
            "expert": {"ff": ff}}


def layer(l=None, r=None, mlp=None, weights_of=None):
    out = {"type": "parallel", "mixer": {"left": l or left(), "right": r or right()}, "mlp": mlp}
    if weights_of is not None:
        out["weights_of"] = weights_of
    return out


def config(layers, width=64, vocab=157, eps=1e-5, mult=0.4):
    layers = copy.deepcopy(layers)
    for i, l in enumerate(layers):       # a layer that borrows repeats the entry of its owner
        if l.get("weights_of") is not None:
            owner = layers[l["weights_of"]]
            layers[i] = dict(copy.deepcopy(owner), weights_of=l["weights_of"])
    return {"architecture": "Vudivik", "width": width, "vocab": vocab, "norm": {"eps": eps},
            "residual_mult": mult, "layers": layers}


SCALING = {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 32}

# Layers that differ in every size: query groups of 2, 1 and 3, value sizes above and below
# the key size, a head size that is no multiple of 16, all, some and none of a head rotated,
# windows shorter and longer than a page, no kept first keys / several / more than a page of
# them, a layer without a window, one to four taps, a state of one, a scan wider than 64
# states, a layer run three times and one run twice, a layer without a feed-forward, experts
# with and without identity experts.
MIXED = config([
    layer(left(4, 2, 24, 40, size=11, keep_first=3, rot_dims=16, scaling=SCALING, scale=0.35),
          right(48, 6, 5, 3), dense(72)),
    layer(left(3, 3, 16, 8, size=21, keep_first=0, rot_dims=16, base=50.0, scale=0.5),
          right(40, 1, 1, 1), moe(5, 2, 3, 24)),
    layer(weights_of=0),
    layer(left(6, 2, 20, 20, size=5, keep_first=18, rot_dims=None, scale=0.3),
          right(33, 70, 7, 4), None),
    layer(weights_of=1),
    layer(left(2, 1, 32, 48, size=None, rot_dims=8, scale=0.25), right(64, 16, 4, 2),
          moe(4, 0, 2, 16)),
    layer(weights_of=2),
])


def random_weights(cfg: dict, seed: int, sharp: float = 1.5) -> dict:
    """Checkpoint tensors (bfloat16 values).  Projections keep activations of order one; the
    query and key norm weights are ``sharp`` (at 3 a query's weight lies on a few keys, which
    the tests of the attention alone use; whole models take less, or seven layers of such
    attention amplify the rounding of bfloat16 activations beyond any use as a yardstick);
    step sizes of the scan spread over two decades and its decays over one."""
    g = torch.Generator().manual_seed(seed)
    w: dict = {}

    def mat(name, rows, cols, gain=1.0):
        w[name] = (gain * torch.randn(rows, cols, generator=g) / cols ** 0.5).to(torch.bfloat16)

    def vec(name, n, mean=0.0, std=0.1):
        w[name] = (mean + std * torch.randn(n, generator=g)).to(torch.bfloat16)

    W = cfg["width"]
    w["embed"] = torch.randn(cfg["vocab"], W, generator=g).to(torch.bfloat16)
    for i, l in enumerate(cfg["layers"]):
        if l.get("weights_of") is not None:
            continue
        p = f"l{i}."
        vec(p + "norm1", W, 1.0, 0.2)
        a, m = l["mixer"]["left"], l["mixer"]["right"]
        H, G, D, VD = a["heads"], a["kv_heads"], a["dim"], a["vdim"]
        for n, rows in (("q", H * D), ("k", G * D), ("v", G * VD)):
            mat(f"{p}mix.left.{n}", rows, W)
            vec(f"{p}mix.left.{n}.b", rows, 0.0, 0.3)
        vec(p + "mix.left.q.norm", D, sharp, 0.3)
        vec(p + "mix.left.k.norm", D, sharp, 0.3)
        mat(p + "mix.left.o", W, H * VD)
        inner, N, R, taps = m["inner"], m["state"], m["dt_rank"], m["conv"]
        mat(p + "mix.right.in", 2 * inner, W)
        mat(p + "mix.right.conv", inner, taps, 1.5)
        vec(p + "mix.right.conv.b", inner, 0.0, 0.2)
        mat(p + "mix.right.x", R + 2 * N, inner, 2.0)
        mat(p + "mix.right.dt", inner, R, 1.0)
        w[p + "mix.right.dt.b"] = (-4.0 + 3.0 * torch.rand(inner, generator=g)).to(torch.bfloat16)
        w[p + "mix.right.A_log"] = torch.log(0.5 + 8.0 * torch.rand(inner, N, generator=g)).to(
            torch.bfloat16)
        vec(p + "mix.right.D", inner, 1.0, 0.3)
        mat(p + "mix.right.o", W, inner)
        vec(p + "mix.left.out", W, 1.0, 0.2)
        vec(p + "mix.right.out", W, 1.0, 0.2)
        mlp = l["mlp"]
        if mlp is None:
            continue
        vec(p + "norm2", W, 1.0, 0.2)
        if mlp["kind"] == "dense":
            mat(p + "mlp.up", mlp["ff"], W)
            mat(p + "mlp.down", W, mlp["ff"])
        else:
            r = mlp["router"]
            outputs = r["experts"] + r.get("identity", 0)
            mat(p + "mlp.router", outputs, W, 2.0)
            vec(p + "mlp.correction", outputs, 0.0, 0.15)
            for e in range(r["experts"]):
                mat(f"{p}mlp.e{e}.up", mlp["expert"]["ff"], W)
                mat(f"{p}mlp.e{e}.down", W, mlp["expert"]["ff"])
    vec("final.norm", W, 1.0, 0.2)
    mat("head", cfg["vocab"], W)
    return w


def as_numpy(weights: dict) -> dict:
    return {k: v.double().numpy() for k, v in weights.items()}


def plain_logits(cfg: dict, weights: dict, toks: list) -> torch.Tensor:
    """float64 logits [len(toks), vocab] of one sequence."""
    return torch.from_numpy(P.plain_forward(list(toks), as_numpy(weights), cfg))


def plain_greedy(cfg: dict, weights: dict, prompt: list, n: int) -> list:
    """The n tokens that greedy decoding appends to ``prompt``, token by token through the
    plain implementation's carried state."""
    w = as_numpy(weights)
    states = [{} for _ in cfg["layers"]]
    logits = P.plain_forward(list(prompt), w, cfg, states)
    out = []
    for _ in range(n):
        out.append(int(np.argmax(logits[-1])))
        logits = P.plain_forward([out[-1]], w, cfg, states)
    return out


def load(cfg: dict, weights: dict, dtype: str):
    from mstar_b200.config.registry import config_from_dict
    from mstar_b200.engine.model import load_model

    return load_model(None, dtype=dtype, device="cuda:0", config=config_from_dict(cfg),
                      tensors=weights)


def scan_params(weights: dict, prefix: str) -> dict:
    return {k[len(prefix):]: v.double().numpy() for k, v in weights.items() if k.startswith(prefix)}


def visible_count(i: int, size, keep_first: int) -> int:
    return sum(P.plain_visible(i, j, size, keep_first) for j in range(i + 1))


assert math.isclose(visible_count(20, 5, 3), 8)

"""Small Tifosun configurations with random weights for the tests, and the plumbing to run
them through the engine's step function and through the plain implementation."""
from __future__ import annotations

import copy

import torch

import plain_tifosun as P


def mlstm_layer(heads=3, dim=24, vdim=40, cap=15.0, kind="mlstm", mlp=None):
    return {"type": kind, "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "gate_cap": cap},
            "mlp": mlp}


def attention_layer(heads=5, dim=24, rot_dim=8, rot_dims=None, vdim=16, rank=48, window=11,
                    base=10000.0, scale=None, mlp=None):
    m = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": rank,
         "rot": {"base": base, "dims": rot_dim if rot_dims is None else rot_dims},
         "scale": (dim + rot_dim) ** -0.5 if scale is None else scale}
    if window is not None:
        m["mask"] = {"size": window}
    return {"type": "latent_attention", "mixer": m, "mlp": mlp}


def dense(ff=72):
    return {"kind": "dense", "ff": ff}


def moe(experts=5, top=2, ff=24, shared=40):
    out = {"kind": "moe", "router": {"experts": experts, "top": top}, "expert": {"ff": ff}}
    if shared:
        out["shared"] = {"ff": shared}
    return out


def config(layers, width=96, vocab=211, eps=1e-5):
    return {"architecture": "Tifosun", "width": width, "vocab": vocab, "norm": {"eps": eps},
            "layers": copy.deepcopy(layers)}


# Three layers of every kind, none of whose sizes equal one another: an odd number of heads,
# value sizes that are no multiple of 32, fewer rotated dimensions than the rotated part has,
# two and three experts per token, a layer without a feed-forward, one without a shared expert.
MIXED = config([
    mlstm_layer(heads=3, dim=24, vdim=40, cap=6.0, mlp=moe(experts=5, top=2, ff=24, shared=40)),
    attention_layer(heads=5, dim=24, rot_dim=8, rot_dims=6, vdim=16, rank=48, window=11,
                    scale=0.9, mlp=dense(72)),
    mlstm_layer(heads=2, dim=72, vdim=33, cap=9.0, kind="mlstm_2", mlp=None),
    attention_layer(heads=2, dim=16, rot_dim=16, vdim=40, rank=40, window=7, base=50.0, scale=1.1,
                    mlp=moe(experts=7, top=3, ff=16, shared=0)),
])


def random_weights(cfg: dict, seed: int, gate_bias=(1.0, 2.0)) -> dict:
    """Checkpoint tensors (bfloat16 values) for ``cfg``.  Projections are drawn so that
    activations stay of order one; the gate biases move the running maximum of the matrix
    memories away from its start (``gate_bias``: mean of the input and of the forget
    bias)."""
    g = torch.Generator().manual_seed(seed)
    w: dict = {}

    def mat(name, rows, cols, gain=1.0):
        w[name] = (gain * torch.randn(rows, cols, generator=g) / cols ** 0.5).to(torch.bfloat16)

    def vec(name, n, mean=0.0, std=0.1):
        w[name] = (mean + std * torch.randn(n, generator=g)).to(torch.bfloat16)

    W = cfg["width"]
    w["embed"] = torch.randn(cfg["vocab"], W, generator=g).to(torch.bfloat16)
    for i, layer in enumerate(cfg["layers"]):
        p, m = f"l{i}.", layer["mixer"]
        for n in ("norm1", "norm1b"):
            vec(p + n, W)
        H = m["heads"]
        if layer["type"] in ("mlstm", "mlstm_2"):
            mat(p + "mix.q", H * m["dim"], W, 2.0)
            mat(p + "mix.k", H * m["dim"], W, 2.0)
            mat(p + "mix.v", H * m["vdim"], W)
            mat(p + "mix.g", H * m["vdim"], W)
            mat(p + "mix.o", W, H * m["vdim"])
            mat(p + "mix.i", H, W, 2.0)
            mat(p + "mix.f", H, W, 2.0)
            vec(p + "mix.i.b", H, gate_bias[0], 1.0)
            vec(p + "mix.f.b", H, gate_bias[1], 1.0)
            vec(p + "mix.norm", H * m["vdim"], 1.0, 0.2)
        else:
            # scores of a few units at a scale near one: a query's weight lies on one or two keys
            mat(p + "mix.q", H * (m["dim"] + m["rot_dim"]), W)
            mat(p + "mix.dkv", m["kv_rank"] + m["rot_dim"], W)
            vec(p + "mix.dkv.norm", m["kv_rank"], 1.0, 0.2)
            mat(p + "mix.uk", H * m["dim"], m["kv_rank"])
            mat(p + "mix.uv", H * m["vdim"], m["kv_rank"])
            mat(p + "mix.g", H * m["vdim"], W)
            mat(p + "mix.o", W, H * m["vdim"])
        mlp = layer["mlp"]
        if mlp is None:
            continue
        for n in ("norm2", "norm2b"):
            vec(p + n, W)
        if mlp["kind"] == "dense":
            mat(p + "mlp.gate", mlp["ff"], W)
            mat(p + "mlp.up", mlp["ff"], W)
            mat(p + "mlp.down", W, mlp["ff"])
        else:
            mat(p + "mlp.router", mlp["router"]["experts"], W, 3.0)
            names = [f"e{e}" for e in range(mlp["router"]["experts"])]
            sizes = [mlp["expert"]["ff"]] * len(names)
            if mlp.get("shared"):
                names.append("shared")
                sizes.append(mlp["shared"]["ff"])
            for n, ff in zip(names, sizes):
                mat(f"{p}mlp.{n}.gate", ff, W)
                mat(f"{p}mlp.{n}.up", ff, W)
                mat(f"{p}mlp.{n}.down", W, ff)
    vec("final.norm", W)
    mat("head", cfg["vocab"], W)
    return w


def tokens(cfg: dict, n: int, seed: int) -> list:
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, cfg["vocab"], (n,), generator=g).tolist()


def plain_logits(cfg: dict, weights: dict, toks: list) -> torch.Tensor:
    """float64 logits [len(toks), vocab] of one sequence."""
    return P.PlainTifosun(cfg, weights).forward(toks)


def load(cfg: dict, weights: dict, dtype: str):
    from mstar_b200.config.registry import config_from_dict
    from mstar_b200.engine.model import load_model

    return load_model(None, dtype=dtype, device="cuda:0", config=config_from_dict(cfg),
                      tensors=weights)


def run_schedule(stepper, reqs: dict, schedule: list) -> dict:
    """``schedule``: steps, each a list of (request id, token count); requests are admitted
    at their first entry and freed after their last token.  Returns id -> float logits
    [tokens, vocab] on the CPU, every position wanted."""
    from mstar_b200.engine.step import StepEntry

    at = {r: 0 for r in reqs}
    out = {r: [None] * len(t) for r, t in reqs.items()}
    for step in schedule:
        entries = []
        for rid, n in step:
            if not stepper.has_request(rid):
                stepper.add_request(rid)
            entries.append(StepEntry(rid, reqs[rid][at[rid]:at[rid] + n], list(range(n))))
        logits = stepper.step(entries).float().cpu()
        row = 0
        for rid, n in step:
            for k in range(n):
                out[rid][at[rid] + k] = logits[row + k].clone()
            row += n
            at[rid] += n
            if at[rid] == len(reqs[rid]):
                stepper.free_request(rid)
    assert all(at[r] == len(reqs[r]) for r in reqs), "the schedule does not feed every token"
    return {r: torch.stack(v) for r, v in out.items()}


def row_errors(got: torch.Tensor, want: torch.Tensor) -> torch.Tensor:
    """Per row rms(got - want) / rms(want), the mean over the vocabulary taken off."""
    d = got.double() - want.double()
    d = d - d.mean(-1, keepdim=True)
    ref = want.double() - want.double().mean(-1, keepdim=True)
    return d.pow(2).mean(-1).sqrt() / ref.pow(2).mean(-1).sqrt()


def relative_error(got: torch.Tensor, want: torch.Tensor) -> float:
    return float(row_errors(got, want).max())


# what rounding alone moves the logits of these small models by, with room to spare; a wrong
# key, a window off by one or a lost state moves them by tens of percent
TOLERANCE = {"float32": 2e-4, "bfloat16": 6e-2}


def assert_close(got: torch.Tensor, want: torch.Tensor, dtype: str, what) -> None:
    """float32: every row within the tolerance.  bfloat16: rounding the activations moves a
    router's logits by a percent, which now and then turns a close call between two experts
    (or two keys of nearly equal score) the other way, and that row, nothing else, then
    differs by more: so half of the rows lie within a third of the tolerance and at most one
    row in ten beyond it.  A fault of the mechanism moves most rows."""
    err = row_errors(got, want)
    if dtype == "float32":
        assert float(err.max()) < TOLERANCE[dtype], (what, dtype, float(err.max()))
        return
    tol = TOLERANCE[dtype]
    over = int((err > tol).sum())
    assert float(err.median()) < tol / 3 and over <= max(1, err.numel() // 10), (
        what, dtype, float(err.median()), over, err.numel())

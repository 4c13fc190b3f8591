"""The Vudivik decoder in the engine against the plain implementation (tests/plain_vudivik.py):
each mechanism alone, then whole models through the step function, the cache and state
manager, the scheduler and the entry point, under every kind of schedule."""
import numpy as np
import pytest
import torch

import plain_vudivik as P
import vudivik_util as U

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
DTYPES = ["float32", "bfloat16"]
TORCH = {"float32": torch.float32, "bfloat16": torch.bfloat16}


def rnd(*shape, seed=0, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    return (scale * torch.randn(*shape, generator=g)).to(torch.bfloat16)


def runtime(dtype):
    from mstar_b200.parts import Runtime
    return Runtime(dtype=TORCH[dtype], device=torch.device(DEV))


def dev(t, dtype):
    return t.to(TORCH[dtype]).to(DEV)


def step_ctx(q_lens, starts, slots=None):
    from test_gpu_parts import simple_ctx
    ctx = simple_ctx(q_lens, starts)
    if slots is not None:
        ctx.slots = torch.tensor(slots, dtype=torch.int32, device=DEV)
        ctx.host_slots = list(slots)
    return ctx


def close(got, want, dtype, what, f32=2e-5, bf16=4e-2):
    """Worst difference relative to the largest wanted value."""
    want = torch.as_tensor(np.asarray(want))
    err = (got.double().cpu() - want.double()).abs().max().item() / want.abs().max().item()
    assert err < (f32 if dtype == "float32" else bf16), (what, dtype, err)


# ------------------------------------------------------------------ mechanisms alone
@pytest.mark.parametrize("dtype", DTYPES)
def test_normed_output_joins_the_residual_with_a_multiplier(dtype):
    """h += m * norm(y) and the new residual as the next sublayer's input, one kernel; y in
    float (the mixer's mean of norms) and in the compute dtype (a feed-forward's output)."""
    from mstar_b200 import ops

    for width, m in ((64, 0.35), (200, 1.0), (1000, 2.5)):
        h, w = rnd(7, width, seed=1).float(), rnd(width, seed=3, scale=0.5).float()
        for y in (rnd(7, width, seed=2, scale=3.0).float(), dev(rnd(7, width, seed=2, scale=3.0), dtype)):
            want = h.double().numpy() + m * P.plain_rms_norm(y.double().cpu().numpy(), w.double().numpy(), 1e-5)
            resid = h.clone().to(DEV)
            rows = ops.add_postnorm_rmsnorm(resid, y.to(DEV), w.to(DEV), 1e-5, 0.0,
                                            out_dtype=TORCH[dtype], post_scale=m, plain_out=True)
            close(resid, want, "float32", "residual")
            assert rows.dtype == TORCH[dtype] and (dtype != "float32" or rows is resid)
            close(rows, want, dtype, "rows", bf16=5e-3)


@pytest.mark.parametrize("dtype", DTYPES)
def test_mean_of_normed_branches(dtype):
    from mstar_b200 import ops

    for width, n in ((64, 2), (328, 3), (1024, 1)):
        xs = [rnd(5, width, seed=10 + b, scale=1.0 + 3 * b) for b in range(n)]
        ws = [rnd(width, seed=20 + b).float() for b in range(n)]
        want = sum(P.plain_rms_norm(x.double().numpy(), w.double().numpy(), 1e-6)
                   for x, w in zip(xs, ws)) / n
        got = ops.mean_of_norms([dev(x, dtype) for x in xs], [w.to(DEV) for w in ws], 1e-6)
        assert got.dtype == torch.float32
        close(got, want, "float32", "mean of norms")
        # left uncomputed, the norm that adds it to the residual takes it along (one kernel
        # for two branches; computed first otherwise): h += m * norm(mean)
        h, w = rnd(5, width, seed=30).float(), rnd(width, seed=31, scale=0.5).float()
        after = h.double().numpy() + 0.3 * P.plain_rms_norm(want, w.double().numpy(), 1e-5)
        resid = h.clone().to(DEV)
        pending = ops.MeanOfNorms([dev(x, dtype) for x in xs], [wt.to(DEV) for wt in ws], 1e-6)
        rows = ops.add_postnorm_rmsnorm(resid, pending, w.to(DEV), 1e-5, 0.0,
                                        out_dtype=TORCH[dtype], post_scale=0.3, plain_out=True)
        close(resid, after, "float32", "mean joins the residual")
        close(rows, after, dtype, "rows after the mean", bf16=5e-3)


@pytest.mark.parametrize("dtype", DTYPES)
def test_feed_forward_without_a_gate(dtype):
    from mstar_b200 import ops
    from mstar_b200.config.layout import MLPSpec
    from mstar_b200.parts import build_part

    # a few rows (in bfloat16 the activation is the epilogue of the first product) and many;
    # a width of whole 64-byte pieces (that kernel's) and one that is not
    for rows, width in ((9, 96), (40, 96), (9, 72)):
        x = rnd(rows, width, seed=6)
        up, down = rnd(200, width, seed=4, scale=0.1), rnd(width, 200, seed=5, scale=0.1)
        part = build_part("ffn", MLPSpec(hidden_size=width, intermediate_size=200),
                          {"up.weight": dev(up, dtype), "down.weight": dev(down, dtype)},
                          runtime(dtype))
        want = P.plain_relu2_mlp(x.double().numpy(), up.double().numpy(), down.double().numpy())
        close(part.forward(dev(x, dtype), None), want, dtype, ("relu squared", rows, width), bf16=2e-2)
    if dtype == "bfloat16":
        h = ops.linear_act(dev(x, dtype)[:, :64].contiguous(), dev(up, dtype)[:, :64].contiguous(), "relu2")
        ref = torch.relu(x[:, :64].double() @ up[:, :64].double().T) ** 2
        close(h, ref, dtype, "fused up product", bf16=2e-2)
    z = rnd(3, 50, seed=7, scale=2.0).double()
    gelu = 0.5 * z * (1 + torch.tanh((2 / torch.pi) ** 0.5 * (z + 0.044715 * z ** 3)))
    close(ops.activation(dev(z, dtype), "gelu_tanh", inplace=False), gelu, dtype, "gelu", bf16=1e-2)
    close(ops.activation(dev(z, dtype), "silu", inplace=False), z * torch.sigmoid(z), dtype, "silu",
          bf16=1e-2)
    with pytest.raises(ValueError, match="swish"):
        build_part("ffn", MLPSpec(hidden_size=72, intermediate_size=200, activation="swish"),
                   {"up.weight": dev(up, dtype), "down.weight": dev(down, dtype)}, runtime(dtype))


def test_router_correction_moves_the_choice_only():
    from mstar_b200 import ops

    g = torch.Generator().manual_seed(5)
    for experts, top in ((7, 3), (14, 3), (40, 5), (3, 3), (5, 1)):
        z = torch.randn(50, experts, generator=g) * 2.0
        bias = torch.randn(experts, generator=g) * 0.3
        chosen, weight = ops.route_topk(z.to(DEV), top, softmax=True, choice_bias=bias.to(DEV))
        s = torch.softmax(z.double(), -1)
        want = torch.topk(s + bias.double(), top).indices
        assert torch.equal(chosen.cpu().long(), want)
        assert (weight.cpu().double() - torch.gather(s, 1, want)).abs().max() < 1e-6
        plain_choice = torch.topk(s, top).indices
        assert experts == top or not torch.equal(plain_choice, want)   # the bias matters here


def experts_part(mlp, width, dtype, seed):
    from mstar_b200.config.registry import config_from_dict
    from mstar_b200.parts import build_part

    cfg = U.config([U.layer(mlp=mlp)], width=width)
    w = U.random_weights(cfg, seed)
    spec = config_from_dict(cfg).layout().blocks[0].ffn
    p, n = "l0.mlp.", mlp["router"]["experts"]
    params = {"router.weight": w[p + "router"], "router.correction": w[p + "correction"],
              "experts.up.weight": torch.cat([w[f"{p}e{e}.up"] for e in range(n)]),
              "experts.down.weight": torch.cat([w[f"{p}e{e}.down"] for e in range(n)])}
    part = build_part("ffn", spec, {k: dev(v, dtype) for k, v in params.items()}, runtime(dtype))
    return part, U.scan_params(w, p)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("experts,identity,top,ff,tokens",
                         [(5, 2, 3, 24, 9), (4, 0, 2, 16, 33), (1, 3, 2, 40, 7), (6, 1, 1, 8, 40),
                          # many rows: in bfloat16 they are sorted by expert and run as tiles
                          (5, 2, 3, 24, 150), (3, 1, 4, 72, 260)])
def test_routed_experts_with_identity_experts(dtype, experts, identity, top, ff, tokens):
    mlp = U.moe(experts, identity, top, ff)
    part, p = experts_part(mlp, 96, dtype, seed=experts + identity)
    x = rnd(tokens, 96, seed=9)
    want = P.plain_moe(x.double().numpy(), p, mlp)
    chosen, _ = P.plain_route(x.double().numpy(), p["router"], p["correction"], top)
    assert identity == 0 or (chosen >= experts).any()          # identity experts are chosen
    got = part.forward(dev(x, dtype), None)
    err = U.row_errors(got.cpu(), torch.from_numpy(want))
    if dtype == "float32":
        assert float(err.max()) < 2e-5
    else:       # a close call of the router that rounding turns moves that row alone
        assert float(err.median()) < 1.5e-2 and int((err > 5e-2).sum()) <= max(1, tokens // 10)


def attention_part(m, width, dtype, seed, sharp=3.0):
    from mstar_b200.config.registry import config_from_dict
    from mstar_b200.parts import build_part

    cfg = U.config([U.layer(l=m)], width=width)
    w = U.random_weights(cfg, seed, sharp=sharp)
    spec = config_from_dict(cfg).layout().blocks[0].mixer.branches[0]
    p = "l0.mix.left."
    params = {"qkv.weight": torch.cat([w[p + "q"], w[p + "k"], w[p + "v"]]),
              "qkv.bias": torch.cat([w[p + "q.b"], w[p + "k.b"], w[p + "v.b"]]),
              "q_norm.weight": w[p + "q.norm"], "k_norm.weight": w[p + "k.norm"],
              "o.weight": w[p + "o"]}
    part = build_part("mixer", spec, {k: dev(v, dtype) for k, v in params.items()}, runtime(dtype))
    return part, spec, U.scan_params(w, p)


def paged_cache(part_spec, tokens, page, dtype, seed=1):
    """Pages scattered over a pool that holds leftovers of other requests."""
    from mstar_b200 import ops
    from mstar_b200.parts import LayerCache

    pages = -(-tokens // page)
    elems = ops.sink_page_elements(part_spec.num_kv_heads, page, part_spec.head_dim,
                                   part_spec.value_dim)
    kv = torch.full((pages + 3, elems), 7.0, dtype=TORCH[dtype], device=DEV)
    table = (torch.randperm(pages + 3, generator=torch.Generator().manual_seed(seed))[:pages]
             .to(torch.int32).to(DEV)[None])
    return LayerCache(kv=kv, page_size=page, block_table=table)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("heads,kv_heads,dim,vdim,size,keep,rot,page",
                         [(4, 2, 24, 40, 11, 3, 16, 4), (3, 3, 16, 8, 9, 0, 16, 8),
                          (6, 2, 20, 20, 5, 18, None, 16), (2, 1, 32, 48, None, 0, 8, 4),
                          (2, 2, 64, 64, 1, 1, 64, 8), (8, 1, 16, 16, 16, 16, 2, 16),
                          (5, 5, 96, 96, 33, 7, 96, 16),
                          # the two widest compiled sizes; 34 query heads on one kv head (more
                          # rows than a warp's 16 in decoding, more than a tile's 64 in prompts)
                          (4, 2, 128, 128, 20, 3, 64, 16), (2, 1, 160, 256, 7, 2, 32, 8),
                          (34, 1, 16, 24, 12, 2, 8, 4)])
def test_window_attention_alone(dtype, heads, kv_heads, dim, vdim, size, keep, rot, page):
    """The attention branch alone with scores so sharp that a query's weight lies on a few
    keys: a key that a window one too long or too short, or one kept key too many or too few,
    would take in or leave out changes the output by its whole value.  Portions down to two
    tokens and single tokens; pages scattered over the pool."""
    m = U.left(heads, kv_heads, dim, vdim, size=size, keep_first=keep, rot_dims=rot,
               scaling=U.SCALING if rot == 16 else None, scale=6.0 / dim)
    part, spec, p = attention_part(m, 96, dtype, seed=7, sharp=3.0)
    T = 70
    x = rnd(T, 96, seed=8)
    want = P.plain_window_attention(x.double().numpy(), p, m, 1e-5, {})
    cache = paged_cache(spec, T, page, dtype)
    outs, at = [], 0
    for n in (23, 2, 1, 1, 1, 1, 1, 1, 1, 1, 1, 1, 1, 29, 3, 2):
        outs.append(part.forward(dev(x[at:at + n], dtype), step_ctx([n], [at]), cache))
        at += n
    assert at == T
    close(torch.cat(outs), want, dtype, "window attention", bf16=6e-2)


def marked_inputs(p, m, width, T, marked, queries):
    """Inputs in which the key at ``marked`` carries the weight of the ``queries``: the query
    tokens lie along a direction d, the marked token along the direction whose key equals
    the query of d (a solution of W_k d' = W_q d), and its value is large with it.  A query
    token's own key points elsewhere."""
    x = rnd(T, width, seed=4, scale=0.3)
    d = rnd(width, seed=5).double().numpy()
    dim = m["dim"]
    target = p["q"][:dim] @ d                                  # the first query head
    d_key = np.linalg.lstsq(p["k"][:dim], target, rcond=None)[0]
    x[marked] = torch.from_numpy(4.0 * d_key).to(torch.bfloat16)
    for q in queries:
        x[q] += torch.from_numpy(4.0 * d).to(torch.bfloat16)
    return x


EDGES = [  # (marked key, query that sees it, query that does not, window), 4 kept first keys
    (50, 50 + 40 - 1, 50 + 40, 40),        # the window's far edge
    (3, 200, None, 40),                    # the last kept first key, from far away
    (4, 4 + 40 - 1, 4 + 40, 40),           # the first key that is not kept
    (20, 320, 321, 301),                   # 300 back, through a window of 301
]


def edge_case(marked, seen_from, unseen_from, win, width=64, keep=4, T=330):
    m = U.left(2, 1, 32, 32, size=win, keep_first=keep, rot_dims=8, scale=1.0)
    cfg = U.config([U.layer(l=m)], width=width)
    p = U.scan_params(U.random_weights(cfg, 3, sharp=1.0), "l0.mix.left.")
    queries = [q for q in (seen_from, unseen_from) if q is not None]
    x = marked_inputs(p, m, width, T, marked, queries)
    xn = x.double().numpy()
    want = P.plain_window_attention(xn, p, m, 1e-5, {})
    # how much hangs on the one key: the plain output with a window one shorter (for the
    # query that sees it) or longer (for the one that does not), or one kept key fewer
    for q, delta in zip(queries, (-1, +1)):
        other = dict(m, mask={"size": win + delta, "keep_first": keep})
        if marked < keep:
            other = dict(m, mask={"size": win, "keep_first": keep - 1})
        shifted = P.plain_window_attention(xn, p, other, 1e-5, {})
        assert np.abs(shifted[q] - want[q]).max() > 0.5 * np.abs(want[q]).max(), (marked, q)
    return m, x, want


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("marked,seen_from,unseen_from,win", EDGES)
def test_one_key_that_stands_out_at_every_edge(dtype, marked, seen_from, unseen_from, win):
    """One key is made to carry all of a query's weight, and its value is large: the query
    just inside the window sees it, the next one does not; the last kept first key is seen
    from far away, the key after it is not; a key 300 back is seen through a window of 301.
    Queries in a prompt portion and decoded alone."""
    m, x, want = edge_case(marked, seen_from, unseen_from, win)
    part, spec, _ = attention_part(m, 64, dtype, seed=3, sharp=1.0)
    T = x.shape[0]
    for first in (T, 45):                     # one prompt; a prompt and decoded tokens
        cache = paged_cache(spec, T, 16, dtype, seed=first)
        outs = [part.forward(dev(x[:first], dtype), step_ctx([first], [0]), cache)]
        outs += [part.forward(dev(x[t:t + 1], dtype), step_ctx([1], [t]), cache)
                 for t in range(first, T)]
        close(torch.cat(outs), want, dtype, ("edge", marked, first), bf16=6e-2)


def scan_part(m, width, dtype, seed):
    from mstar_b200.config.layout import SelectiveScanSpec
    from mstar_b200.parts import build_part

    cfg = U.config([U.layer(r=m)], width=width)
    w = U.random_weights(cfg, seed)
    spec = SelectiveScanSpec(hidden_size=width, inner=m["inner"], state=m["state"],
                             dt_rank=m["dt_rank"], conv=m["conv"])
    p = "l0.mix.right."
    params = {"in.weight": w[p + "in"], "conv.weight": w[p + "conv"], "conv.bias": w[p + "conv.b"],
              "x.weight": w[p + "x"], "dt.weight": w[p + "dt"], "dt.bias": w[p + "dt.b"],
              "A_log": w[p + "A_log"], "D": w[p + "D"], "o.weight": w[p + "o"]}
    part = build_part("mixer", spec, {k: dev(v, dtype) for k, v in params.items()}, runtime(dtype))
    return part, spec, U.scan_params(w, p)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("inner,state,rank,taps", [(48, 6, 5, 3), (40, 1, 1, 1), (33, 70, 7, 4),
                                                   (64, 16, 4, 2), (96, 24, 16, 4), (20, 3, 40, 6)])
def test_selective_scan_alone(dtype, inner, state, rank, taps):
    """The recurrent branch over a sequence cut into a portion, a two-token portion, single
    tokens (fewer than the convolution has taps) and more portions, in a slot that held
    another request's state, against the token-by-token recurrence; then two sequences in one
    batch in other slots."""
    from mstar_b200 import ops
    from mstar_b200.parts import LayerCache

    m = U.right(inner, state, rank, taps)
    part, spec, p = scan_part(m, 96, dtype, seed=inner)
    T = 45
    x = rnd(T, 96, seed=5)
    want = P.plain_selective_scan(x.double().numpy(), p, m, {})
    size = ops.selective_scan_state_size(inner, state, taps)
    slots = torch.randn(4, size, device=DEV)               # leftovers of earlier requests
    slots[2].zero_()
    cache = LayerCache(state=slots)
    outs, at = [], 0
    for n in (19, 2, 1, 1, 1, 17, 4):
        outs.append(part.forward(dev(x[at:at + n], dtype), step_ctx([n], [at], [2]), cache))
        at += n
    assert at == T
    close(torch.cat(outs), want, dtype, "selective scan", bf16=5e-2)
    slots2 = torch.zeros(4, size, device=DEV)
    both = part.forward(dev(torch.cat([x[:9], x[:30]]), dtype), step_ctx([9, 30], [0, 0], [3, 0]),
                        LayerCache(state=slots2))
    close(both[:9], want[:9], dtype, "first of two", bf16=5e-2)
    close(both[9:], want[:30], dtype, "second of two", bf16=5e-2)
    assert float(slots2[1].abs().max()) == 0.0 and float(slots2[3].abs().max()) > 0.0


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("inner,state,rank,taps", [(48, 6, 5, 3), (33, 70, 7, 4), (40, 1, 1, 1)])
def test_selective_scan_long_portions_in_pieces(dtype, inner, state, rank, taps):
    """A portion long enough to be cut into pieces that run side by side (their end states
    joined through the decays of the pieces between), beside a short portion of another
    request in the same batch, then more tokens of both: against the token-by-token
    recurrence; a piece size that is no divisor of the portion; and the same portion uncut."""
    from mstar_b200 import ops
    from mstar_b200.parts import LayerCache

    m = U.right(inner, state, rank, taps)
    part, spec, p = scan_part(m, 96, dtype, seed=inner)
    T = ops.SCAN_PIECES_FROM + 2 * ops.SCAN_PIECE + 37
    x = rnd(T + 20, 96, seed=6)
    want = P.plain_selective_scan(x.double().numpy(), p, m, {})
    short = P.plain_selective_scan(x[:9].double().numpy(), p, m, {})
    size = ops.selective_scan_state_size(inner, state, taps)
    slots = torch.randn(3, size, device=DEV)
    slots[:2].zero_()
    cache = LayerCache(state=slots)
    got = part.forward(dev(torch.cat([x[:5], x[:T]]), dtype), step_ctx([5, T], [0, 0], [1, 0]), cache)
    close(got[5:], want[:T], dtype, "pieces", bf16=5e-2)
    close(got[:5], short[:5], dtype, "short beside pieces", bf16=5e-2)
    more = part.forward(dev(torch.cat([x[5:9], x[T:]]), dtype), step_ctx([4, 20], [5, T], [1, 0]), cache)
    close(more[4:], want[T:], dtype, "after pieces", bf16=5e-2)
    close(more[:4], short[5:], dtype, "short after pieces", bf16=5e-2)
    slots2 = torch.zeros(1, size, device=DEV)
    whole = part.forward(dev(x[:ops.SCAN_PIECES_FROM - 1], dtype),
                         step_ctx([ops.SCAN_PIECES_FROM - 1], [0], [0]), LayerCache(state=slots2))
    close(whole, want[:ops.SCAN_PIECES_FROM - 1], dtype, "uncut", bf16=5e-2)


# ------------------------------------------------------------------ whole models
@pytest.fixture(scope="module")
def mixed_model():
    weights = U.random_weights(U.MIXED, seed=3)
    reqs = {"a": U.tokens(U.MIXED, 61, 1), "b": U.tokens(U.MIXED, 24, 2),
            "c": U.tokens(U.MIXED, 1, 3), "d": U.tokens(U.MIXED, 37, 4),
            "e": U.tokens(U.MIXED, 90, 5)}
    want = {r: U.plain_logits(U.MIXED, weights, t) for r, t in reqs.items()}
    models = {}

    def get(dtype):
        if dtype not in models:
            models[dtype] = U.load(U.MIXED, weights, dtype)
        return models[dtype]

    return weights, reqs, want, get


def check_all(got, want, dtype, what):
    for r in want:
        U.assert_close(got[r], want[r], dtype, (what, r))


def stepper_for(model, **kw):
    from mstar_b200.engine.step import make_stepper
    kw.setdefault("page_size", 4)
    kw.setdefault("num_pages", 64)
    kw.setdefault("num_slots", 3)
    return make_stepper(model, **kw)


@pytest.mark.parametrize("dtype", DTYPES)
def test_whole_prompts_and_token_by_token(mixed_model, dtype):
    """Each request alone: its prompt in one step, and every token as a step of its own (with
    and without captured graphs); the three agree with the plain model."""
    _, reqs, want, get = mixed_model
    model = get(dtype)
    whole = U.run_schedule(stepper_for(model), reqs, [[(r, len(t))] for r, t in reqs.items()])
    check_all(whole, want, dtype, "whole")
    for graphs in (False, True):
        st = stepper_for(model, cuda_graphs=graphs)
        single = U.run_schedule(st, reqs, [[(r, 1)] for r, t in reqs.items() for _ in t])
        check_all(single, want, dtype, f"token by token, graphs={graphs}")
        assert (st.graph_replays > 0) == graphs


@pytest.mark.parametrize("dtype", DTYPES)
def test_portions_of_every_size(mixed_model, dtype):
    """Prompts cut into portions of changing size, down to two tokens, ends decoded one by one:
    cuts fall inside pages, inside windows, among the kept first keys and inside the scan's
    token chunks."""
    _, reqs, want, get = mixed_model
    schedule = []
    for r, t in reqs.items():
        left, sizes, k = len(t), (2, 17, 3, 2, 16, 5, 33, 2), 0
        while left > 6:
            n = min(sizes[k % len(sizes)], left - 6)
            schedule.append([(r, n)])
            left -= n
            k += 1
        schedule += [[(r, 1)]] * left
    got = U.run_schedule(stepper_for(get(dtype)), reqs, schedule)
    check_all(got, want, dtype, "portions")


@pytest.mark.parametrize("dtype", DTYPES)
def test_mixed_batches_reuse_pages_and_slots(mixed_model, dtype):
    """Up to three live requests in a batch, portions beside single tokens, a request sitting
    out a step; five requests go through three slots and a pool of pages that holds less than
    all of them, so that slots and pages are used again; each agrees with itself alone."""
    _, reqs, want, get = mixed_model
    schedule = [
        [("a", 2), ("b", 3), ("c", 1)],               # c ends here: its slot goes to d
        [("a", 29), ("b", 1), ("d", 16)],
        [("a", 1), ("d", 2)],
        [("a", 1), ("b", 18), ("d", 1)],
        [("b", 1), ("a", 20), ("d", 17)],
        [("b", 1), ("a", 1), ("d", 1)],               # b and d end
        [("a", 1), ("e", 2)],
        [("a", 6), ("e", 64)],                        # a ends
        [("e", 1)], [("e", 21)], [("e", 1)], [("e", 1)],
    ]
    st = stepper_for(get(dtype), num_pages=40, num_slots=3)
    got = U.run_schedule(st, reqs, schedule)
    check_all(got, want, dtype, "mixed")
    assert st.manager.num_requests() == 0 and st.manager.check() == 0
    assert st.manager.free_slots() == 3


@pytest.mark.parametrize("dtype", DTYPES)
def test_long_decoding_past_many_windows(dtype):
    """A short prompt and 400 decoded tokens through captured graphs: the window passes over
    decoded tokens many times while the first keys stay, pages between them return and are
    taken again, and the scan's state is carried 400 steps."""
    cfg = U.config([U.layer(U.left(2, 1, 16, 24, size=13, keep_first=5, rot_dims=8, scale=0.4),
                            U.right(40, 8, 4, 4), U.dense(64)),
                    U.layer(U.left(2, 2, 32, 16, size=9, keep_first=0, rot_dims=32, scale=0.3),
                            U.right(24, 4, 2, 2), U.moe(4, 1, 2, 16))],
                   width=64, vocab=97)
    weights = U.random_weights(cfg, 11)
    toks = U.tokens(cfg, 410, 12)
    want = U.plain_logits(cfg, weights, toks)
    st = stepper_for(U.load(cfg, weights, dtype), page_size=4, num_pages=9, num_slots=1)
    got = U.run_schedule(st, {"r": toks}, [[("r", 10)]] + [[("r", 1)]] * 400)
    U.assert_close(got["r"], want, dtype, "long decoding")
    assert st.graph_replays == 400


@pytest.mark.parametrize("dtype", DTYPES)
def test_sizes_that_are_one_or_equal(dtype):
    """One query head on one key head, a value as wide as a key, a window of one, a kept first
    key alone, a state of one, one tap, one expert of which one is chosen, a multiplier of
    one; a second model whose layers all share the first layer's tensors; one whose first
    layer runs the second's; and one whose sizes are multiples of nothing (a width of 100,
    heads of 12 and 10, 50 channels, a vocabulary of 53)."""
    for layers, mult, width, vocab in (
            ([U.layer(U.left(1, 1, 16, 16, size=1, keep_first=1, rot_dims=16, scale=0.25),
                      U.right(16, 1, 1, 1), U.moe(1, 0, 1, 8))], 1.0, 32, 50),
            ([U.layer(U.left(2, 2, 8, 8, size=3, keep_first=2, rot_dims=4, scale=0.5),
                      U.right(8, 2, 2, 2), U.dense(16)),
              U.layer(weights_of=0), U.layer(weights_of=1)], 0.7, 32, 50),
            # a layer that runs the tensors of the layer after it
            ([U.layer(weights_of=1),
              U.layer(U.left(2, 1, 8, 16, size=4, keep_first=1, rot_dims=8, scale=0.5),
                      U.right(16, 3, 2, 3), U.moe(2, 1, 2, 8))], 0.5, 32, 50),
            ([U.layer(U.left(3, 1, 12, 10, size=6, keep_first=2, rot_dims=6, scale=0.4),
                      U.right(50, 5, 3, 3), U.dense(36)),
              U.layer(U.left(3, 3, 12, 10, size=9, keep_first=0, rot_dims=12, scale=0.4),
                      U.right(50, 5, 3, 2), U.moe(3, 1, 2, 20))], 0.6, 100, 53)):
        cfg = U.config(layers, width=width, vocab=vocab, mult=mult)
        weights = U.random_weights(cfg, 21)
        reqs = {"x": U.tokens(cfg, 33, 1), "y": U.tokens(cfg, 12, 2)}
        want = {r: U.plain_logits(cfg, weights, t) for r, t in reqs.items()}
        st = stepper_for(U.load(cfg, weights, dtype))
        got = U.run_schedule(st, reqs, [[("x", 7), ("y", 2)], [("x", 1), ("y", 10)],
                                        [("x", 25)]])
        check_all(got, want, dtype, "small sizes")


@pytest.mark.parametrize("dtype", DTYPES)
def test_greedy_generation_through_the_entry_point(mixed_model, dtype, tmp_path):
    """LLM.generate with its scheduler (portions under a small token budget, several requests
    at once) picks the tokens the plain model picks; in bfloat16 a pick may differ only where
    the plain model's own margin is small, but for one token in twenty."""
    import json

    from safetensors.torch import save_file

    from mstar_b200 import LLM, SamplingParams

    weights, reqs, _, _ = mixed_model
    (tmp_path / "config.json").write_text(json.dumps(U.MIXED))
    save_file({k: v.contiguous() for k, v in weights.items()}, str(tmp_path / "model.safetensors"))
    llm = LLM(str(tmp_path), dtype=dtype, page_size=8, max_num_pages=48,
              max_num_batched_tokens=16, max_concurrent_requests=3)
    prompts = [reqs["a"][:40], reqs["b"][:5], reqs["d"][:19], reqs["e"][:2]]
    n_new = 12
    results = llm.generate(prompts, SamplingParams(temperature=0.0, ignore_eos=True,
                                                   max_output_tokens=n_new))
    w = U.as_numpy(weights)
    far_off = 0
    for prompt, res in zip(prompts, results):
        assert len(res.token_ids) == n_new
        states = [{} for _ in U.MIXED["layers"]]
        logits = P.plain_forward(list(prompt), w, U.MIXED, states)[-1]
        for tok in res.token_ids:
            best = int(np.argmax(logits))
            margin = float(logits[best] - logits[tok])
            assert tok == best or dtype == "bfloat16", (tok, best, margin)
            far_off += tok != best and margin >= 0.25
            logits = P.plain_forward([tok], w, U.MIXED, states)[-1]
    assert far_off <= len(prompts) * n_new // 20, far_off


def test_trace_replay_of_a_model_folder(mixed_model, tmp_path):
    """bin/trace_run on a folder of this design: the registry picks the model by config.json."""
    import json
    import subprocess
    import sys
    from pathlib import Path

    from safetensors.torch import save_file

    weights, reqs, want, _ = mixed_model
    folder = tmp_path / "model"
    folder.mkdir()
    (folder / "config.json").write_text(json.dumps(U.MIXED))
    save_file({k: v.contiguous() for k, v in weights.items()}, str(folder / "model.safetensors"))
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": reqs["a"][:50], "want": [3, 49]},
                                     {"id": "b", "tokens": reqs["b"][:2], "want": []}], "end": []},
             {"step": 1, "entries": [{"id": "b", "tokens": reqs["b"][2:], "want": [0]},
                                     {"id": "a", "tokens": reqs["a"][50:51], "want": [0]}],
              "end": ["b"]}]
    exe = Path(__file__).resolve().parent.parent / "bin" / "trace_run"
    out = tmp_path / "out"
    done = subprocess.run([sys.executable, str(exe), "--model", str(folder), "--dtype", "float32",
                           "--out", str(out), "--max-tokens", "128"],
                          input="\n".join(json.dumps(s) for s in steps) + "\n", text=True,
                          capture_output=True, timeout=900)
    assert done.returncode == 0, done.stderr[-2000:]
    assert [l for l in done.stdout.splitlines() if l.startswith("done")] == ["done 0", "done 1"]
    got0 = torch.from_numpy(np.fromfile(out / "0.f32", dtype="<f4").reshape(2, -1))
    got1 = torch.from_numpy(np.fromfile(out / "1.f32", dtype="<f4").reshape(2, -1))
    U.assert_close(got0, want["a"][[3, 49]], "float32", "trace step 0")
    U.assert_close(got1, torch.stack([want["b"][2], want["a"][50]]), "float32", "trace step 1")

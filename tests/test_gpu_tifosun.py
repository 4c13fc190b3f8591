"""The Tifosun decoder in the engine against the plain implementation (tests/plain_tifosun.py):
each mechanism alone, then whole models through the step function, the cache and state
manager, the scheduler and the entry point, under every kind of schedule."""
import pytest
import torch

import plain_tifosun as P
import tifosun_util as U

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
    err = (got.double().cpu() - want.double()).abs().max().item() / want.abs().max().item()
    assert err < (f32 if dtype == "float32" else bf16), (what, dtype, err)


# ------------------------------------------------------------------ mechanisms alone
@pytest.mark.parametrize("dtype", DTYPES)
def test_norm_after_a_sublayer_joins_the_residual(dtype):
    """h += norm_b(y), then norm(h), as the one kernel that does both, and the first half alone."""
    from mstar_b200 import ops

    for width in (96, 200, 1000):
        h, y = rnd(7, width, seed=1).float(), rnd(7, width, seed=2, scale=3.0)
        wb, w = rnd(width, seed=3, scale=0.2).float(), rnd(width, seed=4, scale=0.2)
        want_h = h.double() + P.norm_around_zero(y.double(), wb.double(), 1e-5)
        want_x = P.norm_around_zero(want_h, w.double(), 1e-5)
        resid = h.clone().to(DEV)
        x = ops.add_postnorm_rmsnorm(resid, dev(y, dtype), wb.to(DEV), 1e-5, 1.0, dev(w, dtype),
                                     1e-5, 1.0, TORCH[dtype])
        close(resid, want_h, "float32", "residual")
        close(x, want_x, dtype, "normed", bf16=1e-2)
        resid = h.clone().to(DEV)
        assert ops.add_postnorm_rmsnorm(resid, dev(y, dtype), wb.to(DEV), 1e-5, 1.0) is None
        close(resid, want_h, "float32", "residual alone")


def mlstm_part(cfg_m, width, dtype, seed, gate_bias=(1.0, 2.0)):
    from mstar_b200.config.layout import MatrixMemorySpec
    from mstar_b200.parts import build_part

    cfg = U.config([{"type": "mlstm", "mixer": cfg_m, "mlp": None}], width=width)
    w = U.random_weights(cfg, seed, gate_bias=gate_bias)
    spec = MatrixMemorySpec(hidden_size=width, num_heads=cfg_m["heads"], qk_dim=cfg_m["dim"],
                            v_dim=cfg_m["vdim"], gate_cap=cfg_m["gate_cap"], norm_eps=1e-5)
    p = "l0.mix."
    params = {"in.weight": torch.cat([w[p + k] for k in "qkvg"]),
              "gates.weight": torch.cat([w[p + "i"], w[p + "f"]]),
              "gates.bias": torch.cat([w[p + "i.b"], w[p + "f.b"]]),
              "norm.weight": w[p + "norm"], "o.weight": w[p + "o"]}
    part = build_part("mixer", spec, {k: dev(v, dtype) for k, v in params.items()}, runtime(dtype))
    return part, spec, {k: v.double() for k, v in w.items()}


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("heads,dim,vdim,bias", [(3, 24, 40, (1.0, 2.0)), (2, 72, 33, (-4.0, 3.0)),
                                                 (1, 136, 64, (4.0, -1.0)), (2, 264, 32, (0.0, 5.0))])
def test_matrix_memory_alone(dtype, heads, dim, vdim, bias):
    """The recurrent mixer over a sequence cut into a portion, a two-token portion, single
    tokens and a last portion, in a slot that was used before, against the token-by-token
    recurrence.  The gate biases cover input gates far below the forget gates at the first
    tokens (the running maximum then stays near its start at zero) and the opposite."""
    from mstar_b200 import ops
    from mstar_b200.parts import LayerCache

    m = {"heads": heads, "dim": dim, "vdim": vdim, "gate_cap": 7.0}
    part, spec, w = mlstm_part(m, 96, dtype, seed=dim, gate_bias=bias)
    T = 45
    x = rnd(T, 96, seed=5)
    want, _ = P.mlstm_mixer(x.double(), w, "l0.mix.", m, 1e-5)
    size = ops.matrix_memory_state_size(heads, dim, vdim)
    state = torch.randn(4, size, device=DEV)               # leftovers of earlier requests
    slot = 2
    state[slot].zero_()
    cache = LayerCache(state=state)
    outs, at = [], 0
    for n in (19, 2, 1, 1, 1, 17, 4):
        outs.append(part.forward(dev(x[at:at + n], dtype), step_ctx([n], [at], [slot]), cache))
        at += n
    assert at == T
    close(torch.cat(outs), want, dtype, "matrix memory")
    # two sequences in one batch, in other slots, agree with each alone
    state2 = torch.zeros(4, size, device=DEV)
    both = part.forward(dev(torch.cat([x[:9], x[:30]]), dtype), step_ctx([9, 30], [0, 0], [3, 0]),
                        LayerCache(state=state2))
    close(both[:9], want[:9], dtype, "first of two")
    close(both[9:], want[:30], dtype, "second of two")


def attention_part(m, width, dtype, seed):
    from mstar_b200.config.layout import LatentAttentionSpec, PositionSpec
    from mstar_b200.parts import build_part

    cfg = U.config([{"type": "latent_attention", "mixer": m, "mlp": None}], width=width)
    w = U.random_weights(cfg, seed)
    pos = PositionSpec(kind="rope", head_dim=m["rot_dim"], rotary_dim=m["rot"]["dims"],
                       theta=m["rot"]["base"], interleaved=True)
    spec = LatentAttentionSpec(hidden_size=width, num_heads=m["heads"], qk_dim=m["dim"],
                               rot_dim=m["rot_dim"], v_dim=m["vdim"], kv_rank=m["kv_rank"],
                               position=pos, window=m.get("mask", {}).get("size"), scale=m["scale"],
                               norm_eps=1e-5)
    p = "l0.mix."
    params = {"in.weight": torch.cat([w[p + "q"], w[p + "dkv"], w[p + "g"]]),
              "kv_norm.weight": w[p + "dkv.norm"], "uk.weight": w[p + "uk"],
              "uv.weight": w[p + "uv"], "o.weight": w[p + "o"]}
    part = build_part("mixer", spec, {k: dev(v, dtype) for k, v in params.items()}, runtime(dtype))
    return part, spec, {k: v.double() for k, v in w.items()}


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("window,rot_dims,page,heads,rank,rot",
                         [(11, 8, 4, 3, 40, 8), (9, 4, 8, 3, 40, 8), (None, 8, 16, 3, 40, 8),
                          (1, 2, 4, 3, 40, 8),
                          # rows of whole k-steps and ranks of whole column tiles: in bfloat16 both
                          # products run on the tensor cores (18 heads: two blocks a token; rank 96:
                          # an odd number of column tiles a warp)
                          (13, 16, 8, 5, 64, 16), (37, 8, 16, 18, 96, 16), (None, 16, 4, 2, 32, 16),
                          # rows of 28 features: no 16-byte rows in bfloat16
                          (6, 4, 8, 2, 24, 4)])
def test_latent_attention_alone(dtype, window, rot_dims, page, heads, rank, rot):
    """The attention mixer alone with scores so sharp that one key carries a query's weight:
    a key that a window of the wrong size would take in or leave out, at page borders or far
    back, changes the output by its whole value.  Portions down to two tokens and single
    tokens; pages scattered over the pool."""
    from mstar_b200.parts import LayerCache

    m = U.attention_layer(heads=heads, dim=24, rot_dim=rot, rot_dims=rot_dims, vdim=20, rank=rank,
                          window=window, scale=1.5)["mixer"]
    part, spec, w = attention_part(m, 96, dtype, seed=7)
    T = 70
    x = rnd(T, 96, seed=8)
    want, _ = P.latent_attention_mixer(x.double(), w, "l0.mix.", m, 1e-5, torch.arange(T))
    pages = -(-T // page)
    kv = torch.full((pages + 3, 1, 1, page, rank + rot), 7.0, dtype=TORCH[dtype], device=DEV)
    table = (torch.randperm(pages + 3, generator=torch.Generator().manual_seed(1))[:pages]
             .to(torch.int32).to(DEV)[None])
    cache = LayerCache(kv=kv, page_size=page, block_table=table)
    outs, at = [], 0
    for n in (23, 2, 1, 1, 1, 1, 1, 1, 1, 1, 1, 1, 1, 29, 3, 2):
        outs.append(part.forward(dev(x[at:at + n], dtype), step_ctx([n], [at]), cache))
        at += n
    assert at == T
    close(torch.cat(outs), want, dtype, "latent attention", bf16=8e-2)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("experts,top,shared,score,renorm,on_input",
                         [(5, 2, 40, "sigmoid", False, True), (7, 3, 0, "sigmoid", False, True),
                          (4, 1, 24, "sigmoid", False, True), (6, 2, 0, "softmax", True, False),
                          (3, 3, 16, "sigmoid", True, True)])
def test_routed_experts_alone(dtype, experts, top, shared, score, renorm, on_input):
    from mstar_b200.config.layout import RoutedExpertsSpec
    from mstar_b200.parts import build_part

    width, ff, T = 96, 24, 33
    mlp = U.moe(experts=experts, top=top, ff=ff, shared=shared)
    cfg = U.config([U.mlstm_layer(mlp=mlp)], width=width)
    w = {k: v.double() for k, v in U.random_weights(cfg, experts).items()}
    p = "l0.mlp."
    spec = RoutedExpertsSpec(hidden_size=width, num_experts=experts, top=top, expert_size=ff,
                             shared_size=shared, score=score, renormalize=renorm,
                             scale_input=on_input)
    params = {"router.weight": w[p + "router"],
              "experts.gate_up.weight": torch.cat([w[f"{p}e{e}.{k}"] for e in range(experts)
                                                   for k in ("gate", "up")]),
              "experts.down.weight": torch.cat([w[f"{p}e{e}.down"] for e in range(experts)])}
    if shared:
        params["shared.gate_up.weight"] = torch.cat([w[p + "shared.gate"], w[p + "shared.up"]])
        params["shared.down.weight"] = w[p + "shared.down"]
    part = build_part("ffn", spec, {k: dev(v, dtype) for k, v in params.items()}, runtime(dtype))
    x = rnd(T, width, seed=9)
    xd = x.double()
    # the defining sums, with the options of the part that the decoder itself does not use
    z = xd @ w[p + "router"].T
    s = torch.sigmoid(z) if score == "sigmoid" else torch.softmax(z, -1)
    want = torch.zeros(T, width, dtype=torch.float64)
    for t in range(T):
        idx = torch.topk(s[t], top).indices
        wt = s[t, idx] / (s[t, idx].sum() if renorm else 1.0)
        for e, a in zip(idx.tolist(), wt.tolist()):
            args = [w[f"{p}e{e}.{k}"] for k in ("gate", "up", "down")]
            want[t] += (P.gated_ffn(a * xd[t:t + 1], *args)[0] if on_input
                        else a * P.gated_ffn(xd[t:t + 1], *args)[0])
    if shared:
        want += P.gated_ffn(xd, w[p + "shared.gate"], w[p + "shared.up"], w[p + "shared.down"])
    if (score, renorm, on_input) == ("sigmoid", False, True):
        assert (want - P.routed_ffn(xd, w, p, mlp)).abs().max() < 1e-12
    got = part.forward(dev(x, dtype), None)
    close(got, want, dtype, "routed experts")
    # a row alone gives the same numbers as the row in the batch
    alone = part.forward(dev(x[5:6], dtype), None)
    assert (alone.float() - got[5:6].float()).abs().max().item() <= (0 if dtype == "float32" else 2e-2)


def test_router_choice_and_weights():
    from mstar_b200 import ops

    z = torch.tensor([[0.1, 2.0, -1.0, 2.0, 0.5], [-3.0, -2.0, -1.0, -0.5, -4.0]], device=DEV)
    idx, wt = ops.route_topk(z, 3)
    assert idx.tolist() == [[1, 3, 4], [3, 2, 1]]           # the lower index wins a tie
    assert torch.allclose(wt.cpu(), torch.sigmoid(z.cpu()).gather(1, idx.cpu().long()), atol=1e-6)
    idx, wt = ops.route_topk(z, 2, softmax=True, renormalize=True)
    assert idx.tolist() == [[1, 3], [3, 2]]
    sm = torch.softmax(z.cpu(), -1).gather(1, idx.cpu().long())
    assert torch.allclose(wt.cpu(), sm / sm.sum(-1, keepdim=True), atol=1e-6)


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
    cuts fall inside pages, inside windows and inside the scan's token chunks."""
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
    """A short prompt and 400 decoded tokens through captured graphs: the windows pass over
    decoded tokens many times, pages of the windowed cache return and are taken again, and
    the recurrent state is carried 400 steps."""
    cfg = U.config([U.mlstm_layer(heads=2, dim=40, vdim=24, cap=5.0, mlp=U.dense(64)),
                    U.attention_layer(heads=2, dim=16, rot_dim=8, vdim=24, rank=32, window=13,
                                      scale=1.2, mlp=U.moe(experts=4, top=1, ff=16, shared=16))],
                   width=64, vocab=97)
    weights = U.random_weights(cfg, 11, gate_bias=(0.0, 4.0))
    toks = U.tokens(cfg, 410, 12)
    want = U.plain_logits(cfg, weights, toks)
    st = stepper_for(U.load(cfg, weights, dtype), page_size=4, num_pages=8, num_slots=1)
    got = U.run_schedule(st, {"r": toks}, [[("r", 10)]] + [[("r", 1)]] * 400)
    U.assert_close(got["r"], want, dtype, "long decoding")
    assert st.graph_replays == 400


@pytest.mark.parametrize("dtype", DTYPES)
def test_models_of_one_kind_of_layer(dtype):
    """A model of matrix memories only has no pages at all; one of attention layers only, with
    one window for all and none for one layer, has no state."""
    for layers in ([U.mlstm_layer(mlp=U.dense(48)), U.mlstm_layer(heads=1, dim=8, vdim=8, kind="mlstm_2")],
                   [U.attention_layer(window=5, mlp=U.dense(48)),
                    U.attention_layer(heads=1, window=None, rot_dims=2)]):
        cfg = U.config(layers, width=64, vocab=50)
        weights = U.random_weights(cfg, 21)
        reqs = {"x": U.tokens(cfg, 33, 1), "y": U.tokens(cfg, 12, 2)}
        want = {r: U.plain_logits(cfg, weights, t) for r, t in reqs.items()}
        st = stepper_for(U.load(cfg, weights, dtype))
        got = U.run_schedule(st, reqs, [[("x", 7), ("y", 2)], [("x", 1), ("y", 10)],
                                        [("x", 25)]])
        check_all(got, want, dtype, "one kind")


@pytest.mark.parametrize("dtype", DTYPES)
def test_greedy_generation_through_the_entry_point(mixed_model, dtype, tmp_path):
    """LLM.generate with its scheduler (portions under a small token budget, several requests
    at once) picks the tokens the plain model picks; in bfloat16 a pick may differ only where
    the plain model's own margin is small, but for one token in twenty (a router's close call
    that rounding turned the other way moves that token's logits by more)."""
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
    far_off = 0
    for prompt, res in zip(prompts, results):
        assert len(res.token_ids) == n_new
        ids = list(prompt)
        plain = P.PlainTifosun(U.MIXED, weights)
        logits = plain.forward(ids)[-1]
        for tok in res.token_ids:
            best = int(logits.argmax())
            margin = (logits[best] - logits[tok]).item()
            assert tok == best or dtype == "bfloat16", (tok, best, margin)
            far_off += tok != best and margin >= 0.25
            logits = plain.forward([tok])[-1]
    assert far_off <= len(prompts) * n_new // 20, far_off


@pytest.mark.parametrize("experts,top,width,ff,tokens,on_input",
                         [(5, 2, 96, 24, 200, True), (12, 1, 64, 40, 64, True),
                          (7, 3, 136, 72, 333, False), (3, 3, 96, 8, 70, True)])
def test_experts_sorted_by_expert_agree_with_rows_alone(experts, top, width, ff, tokens, on_input):
    """Many bfloat16 rows go through the experts sorted by expert, as tiles on the tensor
    cores; a few rows each stream their experts' matrices.  Both against the plain sums, and
    against each other: groups that end inside a tile, an expert nobody chose, widths and
    expert sizes that are no multiple of a tile."""
    from mstar_b200 import ops

    g = torch.Generator().manual_seed(experts)
    x = torch.randn(tokens, width, generator=g).to(torch.bfloat16)
    w_gu = (torch.randn(experts * 2 * ff, width, generator=g) / width ** 0.5).to(torch.bfloat16)
    w_dn = (torch.randn(experts * width, ff, generator=g) / ff ** 0.5).to(torch.bfloat16)
    add = torch.randn(tokens, width, generator=g).to(torch.bfloat16)
    z = torch.randn(tokens, experts, generator=g)
    z[:, 1] = -30.0                                  # nobody chooses expert 1 (unless all are)
    chosen, weight = ops.route_topk(z.to(DEV), top)
    want = add.double().clone()
    for t in range(tokens):
        for k in range(top):
            e, a = int(chosen[t, k]), float(weight[t, k])
            gate, up = w_gu[e * 2 * ff:e * 2 * ff + ff].double(), w_gu[e * 2 * ff + ff:(e + 1) * 2 * ff].double()
            down = w_dn[e * width:(e + 1) * width].double()
            xt = x[t:t + 1].double()
            want[t] += (P.gated_ffn(a * xt, gate, up, down)[0] if on_input
                        else a * P.gated_ffn(xt, gate, up, down)[0])
    args = (x.to(DEV), w_gu.to(DEV), w_dn.to(DEV), chosen, weight)
    grouped = ops.experts_grouped(*args, experts, ff, on_input, add=add.to(DEV))
    by_row = ops.experts_by_row(*args, ff, on_input, add=add.to(DEV))
    close(grouped, want, "bfloat16", "sorted by expert", bf16=2e-2)
    close(by_row, want, "bfloat16", "row by row", bf16=2e-2)
    assert ops.routed_experts(*args, experts, ff, on_input, add=add.to(DEV)).equal(grouped)

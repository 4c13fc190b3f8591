"""Configuration, layout, checkpoint map and plain implementation of the Vudivik decoder (no
GPU needed)."""
import copy

import numpy as np
import pytest

import plain_vudivik as P
import vudivik_util as U
from mstar_b200.cache.manager import CacheManager, GroupConfig
from mstar_b200.cache.storage import plan_groups
from mstar_b200.config.base import ConfigError
from mstar_b200.config.registry import config_from_dict, get_architecture, known_architectures
from mstar_b200.engine.model import cache_needs, model_param_specs
from mstar_b200.parts.rope import rope_inverse_frequencies


def test_architecture_is_registered_and_round_trips():
    assert "Vudivik" in known_architectures()
    cfg = config_from_dict(U.MIXED)
    assert cfg.architecture == "Vudivik" and cfg.to_dict()["layers"] == U.MIXED["layers"]
    assert config_from_dict(cfg.to_dict()).to_dict() == cfg.to_dict()


def test_layout_reads_every_size_and_constant_per_layer():
    lay = config_from_dict(U.MIXED).layout()
    # four sets of weights, seven runs, a cache for every run
    assert len(lay.blocks) == 4
    assert [(e.block, e.cache) for e in lay.order] == [(0, 0), (1, 1), (0, 2), (2, 3), (1, 4),
                                                       (3, 5), (0, 6)]
    assert all(b.kind == "postnorm" and b.residual_mult == 0.4 and b.norm1 is None
               for b in lay.blocks)
    a0, s0 = lay.blocks[0].mixer.branches
    assert (a0.num_heads, a0.num_kv_heads, a0.head_dim, a0.value_dim) == (4, 2, 24, 40)
    assert (a0.window, a0.keep_first, a0.scale, a0.bias, a0.qk_norm_eps) == (11, 3, 0.35, True, 1e-5)
    assert a0.position.rotary_dim == 16 and not a0.position.interleaved
    assert a0.position.scaling.factor == 8.0 and not a0.plain
    assert (s0.inner, s0.state, s0.dt_rank, s0.conv) == (48, 6, 5, 3)
    a2 = lay.blocks[2].mixer.branches[0]
    assert a2.position.kind == "none" and (a2.window, a2.keep_first) == (5, 18)
    a3 = lay.blocks[3].mixer.branches[0]
    assert a3.window is None and a3.keep_first == 0
    assert lay.blocks[2].ffn is None and lay.blocks[2].norm2_post is None
    f0, f1, f3 = lay.blocks[0].ffn, lay.blocks[1].ffn, lay.blocks[3].ffn
    assert (f0.kind, f0.intermediate_size, f0.activation) == ("mlp", 72, "relu2")
    assert (f1.num_experts, f1.identity_experts, f1.top, f1.expert_size) == (5, 2, 3, 24)
    assert (f1.score, f1.renormalize, f1.gated, f1.choice_bias, f1.scale_input) == (
        "softmax", False, False, True, False)
    assert f3.identity_experts == 0
    needs = cache_needs(lay)
    assert needs[0].kv.keep_first == 3 and needs[0].kv.v_head_dim == 40
    assert needs[3].kv.v_head_dim is None and needs[5].kv.window is None
    assert needs[0].state.shape == ((3 - 1) * 48 + 48 * 6,)
    assert needs[2] == needs[0] and needs[6] == needs[0]       # runs of one block
    windows, group_of = plan_groups(needs)
    assert windows == [(11, 3), 21, (5, 18), None] and group_of == [0, 1, 0, 2, 1, 3, 0]


def test_a_layer_may_borrow_from_a_later_one_and_through_another():
    raw = U.config([U.layer(weights_of=2), U.layer(weights_of=0), U.layer(mlp=U.dense(16)),
                    U.layer(U.left(size=None), mlp=None)], width=32, vocab=50)
    raw["layers"][0] = dict(raw["layers"][2], weights_of=2)
    raw["layers"][1] = dict(raw["layers"][2], weights_of=0)
    cfg = config_from_dict(raw)
    lay = cfg.layout()
    assert [(e.block, e.cache) for e in lay.order] == [(0, 0), (0, 1), (0, 2), (1, 3)]
    assert cfg.block_owners() == [2, 3]
    names = {s.name.split(".")[0] for s in get_architecture("Vudivik").checkpoint_map(cfg, lay).sources}
    assert names == {"embed", "final", "head", "l2", "l3"}
    # the plain implementation follows the same chain
    w = U.as_numpy(U.random_weights(raw, 5))
    assert set(k.split(".")[0] for k in w) == names
    assert P.plain_forward(U.tokens(raw, 6, 1), w, raw).shape == (6, 50)
    raw["layers"][2] = dict(raw["layers"][2], weights_of=0)        # a circle
    with pytest.raises(ConfigError, match="weights_of"):
        config_from_dict(raw)


def test_checkpoint_names_cover_the_parameters():
    cfg = config_from_dict(U.MIXED)
    lay = cfg.layout()
    specs = model_param_specs(lay)
    cmap = get_architecture("Vudivik").checkpoint_map(cfg, lay)
    weights = U.random_weights(U.MIXED, 1)
    assert {s.name for s in cmap.sources} == set(weights)
    assert {s.param for s in cmap.sources} == set(specs)
    assert not any(n.startswith(("l2.", "l4.", "l6.")) for n in weights)   # borrowed layers
    rows: dict = {}
    for s in cmap.sources:
        rows[s.param] = rows.get(s.param, 0) + s.rows
        assert tuple(weights[s.name].shape) == (s.rows,) + tuple(specs[s.param].shape[1:]), s.name
    assert all(rows[p] == specs[p].shape[0] for p in specs)


def test_missing_and_unusable_keys_are_named_together():
    raw = copy.deepcopy(U.MIXED)
    del raw["residual_mult"]
    del raw["layers"][0]["mixer"]["left"]["scale"]
    raw["layers"][1]["mixer"]["right"]["conv"] = 0
    raw["layers"][3]["type"] = "serial"
    raw["layers"][4]["weights_of"] = 19
    with pytest.raises(ConfigError) as err:
        config_from_dict(raw)
    text = str(err.value)
    for piece in ("residual_mult", "layers[0].mixer.left.scale", "layers[1].mixer.right.conv",
                  "'serial'", "layers[4].weights_of"):
        assert piece in text, piece


def test_frequency_scaling_has_all_three_bands():
    lay = config_from_dict(U.MIXED).layout()
    pos = lay.blocks[0].mixer.branches[0].position
    got = np.asarray(rope_inverse_frequencies(pos))
    want = P.plain_rotary_frequencies(16, 10000.0, U.SCALING)
    plain = P.plain_rotary_frequencies(16, 10000.0, None)
    assert np.allclose(got, want, rtol=1e-12)
    ratio = want / plain
    assert ratio[0] == 1.0 and abs(ratio[-1] - 1 / 8.0) < 1e-12
    assert any(1 / 8.0 + 1e-6 < r < 1 - 1e-6 for r in ratio)
    # by hand: wavelength 2 pi / f against 32 / 4 and 32 / 1
    f = 10000.0 ** (-2.0 * 1 / 16)
    wl = 2 * np.pi / f
    assert 8 < wl < 32
    s = (32 / wl - 1.0) / (4.0 - 1.0)
    assert abs(want[1] - ((1 - s) * f / 8.0 + s * f)) < 1e-15


def test_plain_mask_rotation_and_router_by_hand():
    assert [j for j in range(10) if P.plain_visible(9, j, 3, 2)] == [0, 1, 7, 8, 9]
    assert [j for j in range(10) if P.plain_visible(9, j, None, 0)] == list(range(10))
    assert [j for j in range(4) if P.plain_visible(2, j, 8, 1)] == [0, 1, 2]
    x = np.array([[[1.0, 2.0, 3.0, 4.0, 5.0]]])
    out = P.plain_rotate(x, [2], np.array([0.5, 0.25]))            # 4 of 5 features rotated
    c0, s0, c1, s1 = np.cos(1.0), np.sin(1.0), np.cos(0.5), np.sin(0.5)
    assert np.allclose(out[0, 0], [1 * c0 - 3 * s0, 2 * c1 - 4 * s1, 3 * c0 + 1 * s0,
                                   4 * c1 + 2 * s1, 5.0])
    # the correction moves the choice, not the weights
    h = np.eye(3)[:1]
    router = np.array([[2.0, 0, 0], [1.0, 0, 0], [0.0, 0, 0]])
    chosen, weights = P.plain_route(h, router, np.array([0.0, 0.0, 1.0]), 2)
    s = np.exp([2.0, 1.0, 0.0]) / np.exp([2.0, 1.0, 0.0]).sum()
    assert chosen.tolist() == [[2, 0]] and np.allclose(weights, [[s[2], s[0]]])
    # an identity expert hands its input on, times its weight
    p = {"router": router, "correction": np.array([0.0, 0.0, 5.0]),
         "e0.up": np.ones((2, 3)), "e0.down": np.ones((3, 2)),
         "e1.up": np.zeros((2, 3)), "e1.down": np.zeros((3, 2))}
    y = P.plain_moe(h, p, {"router": {"experts": 2, "identity": 1, "top": 1}})
    assert np.allclose(y, s[2] * h)


def test_plain_portions_equal_the_whole():
    """The plain implementation itself: a sequence fed whole, in portions and token by token."""
    cfg = U.config([U.layer(U.left(size=4, keep_first=2), U.right(conv=4), U.dense(16)),
                    U.layer(weights_of=0)], width=32, vocab=50)
    w = U.as_numpy(U.random_weights(cfg, 3))
    toks = U.tokens(cfg, 17, 4)
    whole = P.plain_forward(toks, w, cfg)
    for cuts in ([5, 2, 1, 9], [1] * 17):
        states, rows, at = [{} for _ in cfg["layers"]], [], 0
        for n in cuts:
            rows.append(P.plain_forward(toks[at:at + n], w, cfg, states))
            at += n
        assert np.allclose(np.concatenate(rows), whole, atol=1e-9)


def test_kept_first_pages_stay_with_the_request():
    """A window of 6 over pages of 4 that keeps the first 5 keys: the two pages that hold them
    never return while the request runs; the pages between them and the window do."""
    cm = CacheManager([GroupConfig(4, 12, window=6, keep_first=5)], num_slots=1)
    cm.add_request("a")
    held = []
    for n in range(40):
        cm.reserve(["a"], [1])
        cm.commit("a", 1)
        table = cm.block_table("a")
        first_needed = max(n + 1 - 6 + 1, 0) // 4
        for p, page in enumerate(table):
            assert (page >= 0) == (p < 2 or p >= first_needed), (n, table)
        held.append(sum(page >= 0 for page in table))
        assert cm.check() == 0
    assert max(held) <= 2 + 3
    cm.free_request("a")
    assert cm.free_pages(0) == 12 and cm.check() == 0
    # without kept keys the same window gives its first pages back
    cm = CacheManager([GroupConfig(4, 12, window=6)], num_slots=1)
    cm.add_request("a")
    cm.reserve(["a"], [20])
    cm.commit("a", 20)
    assert cm.block_table("a")[:3] == [-1, -1, -1]


def test_command_line_writes_a_random_model_of_this_design(tmp_path, capsys):
    """``mstar random-model`` with a Vudivik configuration: the folder holds the design's
    tensor names (none for a layer that borrows), and its configuration reads back."""
    import json

    from safetensors import safe_open

    from mstar_b200.cli import main as cli
    from mstar_b200.config.registry import load_config

    src = tmp_path / "config.json"
    src.write_text(json.dumps(U.MIXED))
    out = tmp_path / "model"
    cli.main(["random-model", str(src), str(out), "--seed", "5", "--std", "0.05"])
    assert str(out) in capsys.readouterr().out
    assert load_config(out).to_dict() == config_from_dict(U.MIXED).to_dict()
    with safe_open(str(out / "model.safetensors"), framework="pt") as f:
        assert set(f.keys()) == set(U.random_weights(U.MIXED, 1))
        assert tuple(f.get_tensor("l0.mix.right.A_log").shape) == (48, 6)
        assert tuple(f.get_tensor("l1.mlp.correction").shape) == (7,)

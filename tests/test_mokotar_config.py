"""Configuration, layout, checkpoint map and plain implementation of the Mokotar decoder (no
GPU needed)."""
import copy

import numpy as np
import pytest

import mokotar_util as U
import plain_mokotar as P
from mstar_b200.cache.storage import plan_groups
from mstar_b200.config.base import ConfigError
from mstar_b200.config.registry import config_from_dict, get_architecture, known_architectures
from mstar_b200.engine.model import cache_needs, model_param_specs
from mstar_b200.weights.loader import checkpoint_shapes


def shaped(raw, weights=None):
    """The typed configuration with the ranks that only the tensors give."""
    cfg = config_from_dict(raw)
    return cfg.with_shapes(checkpoint_shapes(weights if weights is not None
                                             else U.random_weights(raw, 1)))


def test_architecture_is_registered_and_round_trips():
    assert "Mokotar" in known_architectures()
    cfg = config_from_dict(U.MIXED)
    assert cfg.architecture == "Mokotar" and cfg.to_dict()["layers"] == U.MIXED["layers"]
    assert cfg.to_dict()["loop"] == U.MIXED["loop"] and cfg.to_dict()["streams"] == 3
    assert config_from_dict(cfg.to_dict()).to_dict() == cfg.to_dict()


def test_layout_reads_every_size_and_constant_per_layer():
    lay = shaped(U.MIXED).layout()
    # five sets of weights; the stretch 1..3 runs twice; a cache for every run
    assert len(lay.blocks) == 5
    assert [(e.block, e.cache) for e in lay.order] == [(0, 0), (1, 1), (2, 2), (3, 3), (1, 4),
                                                       (2, 5), (3, 6), (4, 7)]
    assert all(b.kind == "hyper" and b.residual_mult == 0.4 and b.streams == 3 for b in lay.blocks)
    a0 = lay.blocks[0].mixer
    assert (a0.num_heads, a0.num_kv_heads, a0.head_dim, a0.value_dim) == (4, 2, 24, 40)
    assert (a0.scale, a0.softcap, a0.q_temp, a0.sink) == (0.3, 8.0, (0.4, 7), "learned")
    assert a0.feature_gate and not a0.qk_norm_whole and a0.position.kind == "none"
    assert a0.window is None and not a0.plain
    a2 = lay.blocks[2].mixer
    assert a2.qk_norm_whole and a2.position.interleaved and a2.position.rotary_dim == 12
    assert a2.position.theta == 300.0 and a2.softcap is None and a2.q_temp is None
    assert a2.sink == "learned" and a2.feature_gate
    assert lay.blocks[2].ffn is None and lay.blocks[2].norm2 is None
    p1 = lay.blocks[1].mixer
    assert p1.merge == "weighted_sum" and p1.scales == (1.3, 0.8)
    l1, r1 = p1.branches
    assert (l1.sink, l1.feature_gate, l1.qk_norm_whole, l1.softcap) == ("zero", False, False, None)
    assert l1.position.interleaved and l1.position.rotary_dim == 16
    assert (r1.num_heads, r1.num_kv_heads, r1.qk_dim, r1.v_dim, r1.conv) == (4, 2, 24, 20, 3)
    assert (r1.decay_rank, r1.gate_rank) == U.RANKS
    r3 = lay.blocks[3].mixer.branches[1]
    assert (r3.num_heads, r3.num_kv_heads, r3.qk_dim, r3.v_dim, r3.conv) == (3, 3, 10, 36, 4)
    f0 = lay.blocks[0].ffn
    assert (f0.kind, f0.intermediate_size, f0.activation, f0.bias) == ("gated_mlp", 72, "silu", True)
    needs = cache_needs(lay)
    assert needs[0].kv.v_head_dim == 40 and needs[0].state is None and needs[0].kv.window is None
    assert needs[1].state.shape == ((3 - 1) * (2 * 48 + 80) + 4 * 24 * 20,)
    assert needs[4] == needs[1] and needs[6] == needs[3]          # the passes of one block
    windows, group_of = plan_groups(needs)
    assert windows == [None] and group_of == [0] * 8


def test_no_loop_no_copies_and_a_loop_at_either_end():
    layers = U.MIXED["layers"]
    plain = shaped(U.config(layers, streams=0)).layout()
    assert [e.block for e in plain.order] == [0, 1, 2, 3, 4]
    assert all(b.streams == 0 for b in plain.blocks)
    specs = model_param_specs(plain)
    assert not any(".hc" in k for k in specs)
    for loop, want in (((0, 2, 3), [0, 1, 0, 1, 0, 1, 2, 3, 4]), ((3, 5, 2), [0, 1, 2, 3, 4, 3, 4]),
                       ((2, 2, 4), [0, 1, 2, 3, 4]), ((0, 5, 1), [0, 1, 2, 3, 4])):
        raw = U.config(layers, loop=loop)
        assert [e.block for e in shaped(raw).layout().order] == want == P.plain_run_order(raw)


def test_checkpoint_names_cover_the_parameters():
    weights = U.random_weights(U.MIXED, 2)
    cfg = shaped(U.MIXED, weights)
    lay = cfg.layout()
    specs = model_param_specs(lay)
    cmap = get_architecture("Mokotar").checkpoint_map(cfg, lay)
    assert {s.name for s in cmap.sources} == set(weights)
    filled = {}
    for s in cmap.sources:
        assert tuple(weights[s.name].shape) == (s.rows,) + tuple(specs[s.param].shape[1:]), s.name
        filled[s.param] = filled.get(s.param, 0) + s.rows
    assert {k: v.shape[0] for k, v in specs.items()} == filled
    assert specs["blocks.2.mixer.q_norm.weight"].shape == (3 * 40,)       # over the projection
    assert specs["blocks.0.mixer.q_norm.weight"].shape == (24,)           # a head
    assert specs["blocks.0.mixer.qkv.weight"].shape == (4 * 24 + 2 * 24 + 2 * 40 + 4 * 40, 64)
    assert "blocks.1.mixer.branch0.sink" not in specs and "blocks.0.mixer.sink" in specs
    assert specs["blocks.1.hc2.mix"].shape == (3, 3)


def test_ranks_come_from_the_tensors_or_the_configuration():
    raw = copy.deepcopy(U.MIXED)
    bare = config_from_dict(raw).layout().blocks[1].mixer.branches[1]
    assert (bare.decay_rank, bare.gate_rank) == (0, 0)              # not known yet
    weights = U.random_weights(raw, 3, ranks=(9, 2))
    got = shaped(raw, weights).layout().blocks[3].mixer.branches[1]
    assert (got.decay_rank, got.gate_rank) == (9, 2)
    raw["layers"][1]["mixer"]["right"].update(decay_rank=11, gate_rank=4)
    said = config_from_dict(raw).layout().blocks[1].mixer.branches[1]
    assert (said.decay_rank, said.gate_rank) == (11, 4)


def test_unusable_configurations_name_everything():
    raw = copy.deepcopy(U.MIXED)
    del raw["layers"][0]["mixer"]["softcap"]
    del raw["layers"][2]["mixer"]["rot"]
    raw["layers"][1]["mixer"]["right"]["heads"] = 5
    raw["layers"][3]["type"] = "attention_3"
    raw["layers"][4]["mlp"] = {"kind": "moe"}
    raw["loop"] = {"start": 3, "stop": 2, "times": 2}
    del raw["vocab"]
    with pytest.raises(ConfigError) as err:
        config_from_dict(raw)
    text = str(err.value)
    for part in ("softcap", "layers[2].mixer.rot", "layers[1].mixer.right.heads", "attention_3",
                 "layers[4].mlp.kind", "config.loop", "vocab"):
        assert part in text, part


def test_plain_mechanisms_on_hand_computed_cases():
    # pairs of neighbours, angle p * base^(-2i/dims); features beyond dims pass
    x = np.array([[[1.0, 0.0, 0.0, 2.0, 5.0, 6.0]]])
    y = P.plain_rotate_pairs(x, [3], 4, 100.0)
    a0, a1 = 3.0, 3.0 * 100.0 ** -0.5
    assert np.allclose(y[0, 0], [np.cos(a0), np.sin(a0), -2 * np.sin(a1), 2 * np.cos(a1), 5, 6])
    # the sink takes its share and gives nothing back
    p = P.plain_sink_softmax(np.array([0.0, 0.0]), sink=np.log(2.0))
    assert np.allclose(p, [0.25, 0.25])
    assert np.allclose(P.plain_sink_softmax(np.array([1.0, 1.0]), None), [0.5, 0.5])
    assert np.allclose(P.plain_sink_softmax(np.array([0.0]), 0.0), [0.5])     # one added
    # temperature: steps at multiples of `every`
    t = P.plain_query_temperature([0, 5, 6, 13, 20], 0.5, 7)
    assert np.allclose(t, 1 + 0.5 * np.log([1, 1, 2, 3, 4]))
    # the delta rule: a key written once is read back exactly when beta is one; a second
    # write along the same key replaces the value; the decay fades the rows
    k = np.array([[1.0, 0.0], [1.0, 0.0], [0.0, 1.0]])
    v = np.array([[3.0], [5.0], [7.0]])
    S = np.zeros((2, 1))
    o = P.plain_delta_rule(k.copy(), k, v, np.ones(3), np.ones((3, 2)), S)
    assert np.allclose(o[:, 0], [3.0, 5.0, 7.0]) and np.allclose(S[:, 0], [5.0, 7.0])
    S = np.zeros((2, 1))
    o = P.plain_delta_rule(k.copy(), k, v, np.full(3, 0.5), np.full((3, 2), 0.5), S)
    # S0 = 1.5; then decayed 0.75, u = .5 (5 - .75) = 2.125 -> 2.875
    assert np.allclose(o[:2, 0], [1.5, 2.875])
    # hyper-connections with one copy and unit tables are the plain residual
    xs = np.arange(6.0).reshape(1, 2, 3)
    y = np.ones((2, 3))
    assert np.allclose(P.plain_hyper_write(xs, y, [[1.0]], [1.0], 0.5)[0], xs[0] + 0.5)
    assert np.allclose(P.plain_hyper_read(np.stack([xs[0], 2 * xs[0]]), [0.5, 0.25]), xs[0])
    # the convolution's last column meets the token itself, zeros before the start
    st = {}
    c = P.plain_short_conv(np.array([[1.0], [2.0], [3.0]]), np.array([[10.0, 1.0]]), st, "c")
    assert np.allclose(c[:, 0], [1.0, 12.0, 23.0]) and np.allclose(st["c"], [[3.0]])
    c2 = P.plain_short_conv(np.array([[4.0]]), np.array([[10.0, 1.0]]), st, "c")
    assert np.allclose(c2, [[34.0]])


def test_plain_model_in_portions_equals_whole():
    w = U.as_numpy(U.random_weights(U.MIXED, 4))
    toks = U.tokens(U.MIXED, 19, 1)
    whole = P.plain_forward(toks, w, U.MIXED)
    states = [{} for _ in range(U.runs(U.MIXED))]
    parts = [P.plain_forward(toks[a:b], w, U.MIXED, states) for a, b in ((0, 7), (7, 9), (9, 10), (10, 19))]
    assert np.abs(np.concatenate(parts) - whole).max() < 1e-9
    # the copies matter, the loop matters, the sink matters
    other = P.plain_forward(toks, w, dict(U.MIXED, loop={"start": 1, "stop": 4, "times": 1}))
    assert np.abs(other - whole).max() > 1e-2
    w2 = dict(w)
    w2["l0.mix.sink"] = w["l0.mix.sink"] + 2.0
    assert np.abs(P.plain_forward(toks, w2, U.MIXED) - whole).max() > 1e-3

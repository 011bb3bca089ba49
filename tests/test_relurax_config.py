"""Configuration, layout, checkpoint map and plain implementation of the Relurax decoder (no
GPU needed)."""
import copy

import numpy as np
import pytest

import plain_relurax as P
import relurax_util as U
from mstar_b200.cache.storage import plan_groups
from mstar_b200.config.base import ConfigError
from mstar_b200.config.registry import config_from_dict, get_architecture, known_architectures
from mstar_b200.engine.model import cache_needs, model_param_specs


def test_architecture_is_registered_and_round_trips():
    assert "Relurax" in known_architectures()
    cfg = config_from_dict(U.MIXED)
    assert cfg.architecture == "Relurax" and cfg.to_dict()["layers"] == U.MIXED["layers"]
    assert config_from_dict(cfg.to_dict()).to_dict() == cfg.to_dict()


def test_layout_reads_every_size_and_constant_per_layer():
    lay = config_from_dict(U.MIXED).layout()
    assert len(lay.blocks) == 8
    # a layer that reads another's rows runs on that layer's cache; the others count on
    assert [(e.block, e.cache) for e in lay.order] == [(0, 0), (1, 1), (2, 2), (3, 1), (4, 3),
                                                       (5, 4), (6, 5), (7, 4)]
    assert all(b.kind == "sandwich" and b.norm1.weight_offset == 0.0 and b.norm1.eps == 1e-5
               for b in lay.blocks)
    a0 = lay.blocks[0].mixer
    assert (a0.num_heads, a0.num_kv_heads, a0.head_dim, a0.value_dim) == (4, 2, 24, 24)
    assert (a0.window, a0.conv_taps, a0.value_from_key, a0.head_gate) == (11, 3, True, True)
    assert a0.scale == 4.0 / 24 and a0.qk_norm_eps == 1e-5 and a0.position.kind == "none"
    assert not a0.plain and not a0.bias and a0.keep_first == 0
    a2, a6 = lay.blocks[2].mixer, lay.blocks[6].mixer
    assert (a2.conv_taps, a2.scale, a2.window) == (1, 0.3, 21) and a6.window is None
    l1, l3, l5 = (lay.blocks[i].mixer for i in (1, 3, 5))
    assert (l1.num_heads, l1.qk_dim, l1.rot_dim, l1.v_dim, l1.kv_rank, l1.q_rank) == (3, 16, 8, 24,
                                                                                     40, 20)
    assert l1.window is None and l1.gated and l1.gate_per_head and not l1.shares_kv
    assert not l1.position.interleaved and l1.position.rotary_dim == 8
    assert l3.shares_kv and (l3.num_heads, l3.qk_dim, l3.v_dim, l3.q_rank) == (2, 8, 12, 28)
    assert (l5.position.theta, l5.position.rotary_dim, l5.rot_dim) == (50.0, 8, 12)
    assert lay.blocks[2].ffn is None and lay.blocks[2].norm2_post is None
    f0 = lay.blocks[0].ffn
    assert (f0.kind, f0.intermediate_size, f0.activation) == ("gated_mlp", 72, "gelu_tanh")
    needs = cache_needs(lay)
    assert len(needs) == 6
    assert needs[0].kv.window == 11 and needs[0].kv.planes == 2 and needs[0].kv.v_head_dim is None
    assert needs[0].state.shape == ((3 - 1) * (4 + 2) * 24,)
    assert needs[2].state is None                      # one tap keeps nothing
    assert needs[1].kv.planes == 1 and needs[1].kv.head_dim == 48 and needs[1].state is None
    windows, group_of = plan_groups(needs)
    assert windows == [11, None, 21, 5] and group_of == [0, 1, 2, 3, 1, 1]


def test_checkpoint_names_cover_the_parameters():
    cfg = config_from_dict(U.MIXED)
    lay = cfg.layout()
    specs = model_param_specs(lay)
    cmap = get_architecture("Relurax").checkpoint_map(cfg, lay)
    weights = U.random_weights(U.MIXED, 1)
    assert {s.name for s in cmap.sources} == set(weights)
    filled = {}
    for s in cmap.sources:
        assert tuple(weights[s.name].shape) == (s.rows,) + tuple(specs[s.param].shape[1:]), s.name
        filled[s.param] = filled.get(s.param, 0) + s.rows
    assert filled == {name: spec.shape[0] for name, spec in specs.items()}
    # a layer that reads another's rows has no down-projection, the others have
    assert "l3.mix.dkv" not in weights and "l1.mix.dkv" in weights
    assert specs["blocks.3.mixer.in.weight"].shape == (28 + 2, 64)
    assert specs["blocks.1.mixer.in.weight"].shape == (20 + 40 + 8 + 3, 64)
    assert specs["blocks.0.mixer.qkv.weight"].shape == (4 * 24 + 2 * 24 + 4, 64)
    assert specs["blocks.4.mixer.k_conv.weight"].shape == (2 * 20, 5)


@pytest.mark.parametrize("change,word", [
    (lambda c: c["layers"][0]["mixer"].pop("conv"), "conv is missing"),
    (lambda c: c["layers"][0]["mixer"].update(vdim=8), "vdim"),
    (lambda c: c["layers"][0]["mixer"].update(heads=5), "multiple of kv_heads"),
    (lambda c: c["layers"][1]["mixer"].pop("q_rank"), "q_rank is missing"),
    (lambda c: c["layers"][1]["mixer"]["rot"].update(dims=7), "rot.dims"),
    (lambda c: c["layers"][3]["mixer"].update(kv_from=5), "kv_from"),       # a later layer
    (lambda c: c["layers"][3]["mixer"].update(kv_from=0), "kv_from"),       # not a latent layer
    (lambda c: c["layers"][7]["mixer"].update(kv_from=3), "kv_from"),       # itself a reader
    (lambda c: c["layers"][3]["mixer"].update(kv_rank=24), "kv_rank must equal"),
    (lambda c: c["layers"][0].update(type="mamba"), "not known"),
    (lambda c: c["layers"][0]["mlp"].update(kind="moe"), "not known"),
    (lambda c: c.pop("width"), "width is missing"),
    (lambda c: c["norm"].pop("eps"), "eps is missing"),
])
def test_unusable_configurations_are_named(change, word):
    raw = copy.deepcopy(U.MIXED)
    change(raw)
    with pytest.raises(ConfigError, match=word):
        config_from_dict(raw)


def test_plain_pieces_on_hand_computed_values():
    # a convolution of three taps over a sequence fed in two parts
    w = np.array([[1.0, 10.0, 100.0]])
    u = np.array([[1.0], [2.0], [3.0], [4.0]])
    y, last = P.plain_causal_conv(u, w, np.zeros((2, 1)))
    assert y[:, 0].tolist() == [100.0, 210.0, 321.0, 432.0] and last[:, 0].tolist() == [3.0, 4.0]
    y1, mid = P.plain_causal_conv(u[:1], w, np.zeros((2, 1)))
    y2, last2 = P.plain_causal_conv(u[1:], w, mid)
    assert np.concatenate([y1, y2])[:, 0].tolist() == y[:, 0].tolist()
    assert mid[:, 0].tolist() == [0.0, 1.0] and last2[:, 0].tolist() == [3.0, 4.0]
    # the window: a token and the size - 1 before it
    assert [j for j in range(10) if P.plain_window_visible(7, j, 3)] == [5, 6, 7]
    assert [j for j in range(10) if P.plain_window_visible(1, j, 3)] == [0, 1]
    assert [j for j in range(4) if P.plain_window_visible(2, j)] == [0, 1, 2]
    # rotate-half pairs: feature i with i + half; what lies beyond passes
    x = np.array([[[1.0, 0.0, 0.0, 1.0, 5.0]]])
    r = P.plain_rotate_half(x, [1], np.array([np.pi / 2, np.pi]))
    assert np.allclose(r[0, 0], [0.0, 0.0, 1.0, -1.0, 5.0])
    assert np.allclose(P.plain_rotary_frequencies(4, 100.0), [1.0, 0.1])
    assert abs(float(P.plain_gelu_tanh(1.0)) - 0.8411919906) < 1e-9
    assert np.allclose(P.plain_rms_norm([3.0, 4.0], [1.0, 2.0], 0.0), [3 / 12.5 ** 0.5, 8 / 12.5 ** 0.5])


def test_plain_model_is_the_same_whole_and_in_parts():
    w = U.as_numpy(U.random_weights(U.MIXED, 2))
    toks = U.tokens(U.MIXED, 40, 3)
    model = P.PlainRelurax(U.MIXED, w)
    whole, after = model.forward(toks)
    assert whole.shape == (40, 157) and after.shape == (8, 40, 64)
    model.reset()
    parts = [model.forward(toks[a:b])[0] for a, b in ((0, 13), (13, 15), (15, 16), (16, 40))]
    assert np.abs(np.concatenate(parts) - whole).max() < 1e-9
    # the layers that read another's rows depend on them: other rows, other logits
    other = dict(w)
    other["l1.mix.dkv"] = w["l1.mix.dkv"][::-1].copy()
    assert np.abs(P.PlainRelurax(U.MIXED, other).forward(toks)[0] - whole).max() > 1e-3


def test_norms_of_an_absent_feed_forward_are_not_read():
    """A checkpoint may carry norm2 / norm2b for a layer without a feed-forward; the map
    leaves them alone, and still names any other tensor it has no place for."""
    lay = config_from_dict(U.MIXED).layout()
    cmap = get_architecture("Relurax").checkpoint_map(config_from_dict(U.MIXED), lay)
    assert cmap.ignore("l2.norm2") and cmap.ignore("l2.norm2b")
    assert not cmap.ignore("l0.norm2") and not cmap.ignore("l2.norm1") and not cmap.ignore("l2.mlp.up")

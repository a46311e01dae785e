"""Pofazen without a GPU: configuration and refusals, tensor names against a drawn model file, what each layer
keeps between steps and how the cache manager groups, sizes and gives it back, the mask's definition, the
frequency table, and properties of the plain mechanisms that the GPU tests lean on."""

import copy
import math

import pytest
import torch

from pofazen_helpers import CONFIGS, PP, draw_weights, layer, left, model, parallel, right, wkv


def build(raw, shapes=None):
    from prism_b200.model_registry import build_model
    return build_model(copy.deepcopy(raw), shapes)


def test_the_registry_finds_the_design_and_every_tensor_has_a_taker():
    from prism_b200.model_registry import registered_architectures
    assert "Pofazen" in registered_architectures()
    for name, (raw, seed, _) in CONFIGS.items():
        w = draw_weights(raw, seed)
        cfg, mdl = build(raw, {k: tuple(v.shape) for k, v in w.items()})
        asked = {s.name: tuple(s.shape) for _, spec in mdl.named_params() for s in spec.sources if not spec.optional}
        assert asked == {k: tuple(v.shape) for k, v in w.items()}, name


def test_sizes_come_from_the_file_where_only_the_file_has_them():
    raw = copy.deepcopy(CONFIGS["T"][0])
    for l in raw["layers"]:
        del l["mixer"]["decay_rank"]
    from prism_b200.config.model_config import ConfigError
    with pytest.raises(ConfigError, match="decay_rank"):
        build(raw)
    cfg, _ = build(raw, {"l0.mix.w1": (5, 48), "l1.mix.w1": (9, 48)})
    assert [l.mixer.decay_rank for l in cfg.layers] == [5, 9]
    with pytest.raises(ConfigError, match="l1.mix.w1"):
        build(raw, {"l0.mix.w1": (5, 48)})


@pytest.mark.parametrize("edit, text", [
    (lambda r: r.pop("postln_alpha"), "postln_alpha"),
    (lambda r: r["layers"][0].update(type="conv"), "parallel"),
    (lambda r: r["layers"][0]["mixer"]["left"].update(kv_heads=4), "divisible"),
    (lambda r: r["layers"][0]["mixer"]["left"]["rot"].update(dims=7), "even"),
    (lambda r: r["layers"][0]["mixer"]["right"].pop("conv"), "conv"),
    (lambda r: r["layers"][0]["mixer"].pop("left_scale"), "left_scale"),
    (lambda r: r["layers"][0]["mlp"].update(kind="experts"), "dense"),
    (lambda r: r["layers"][0]["mixer"]["left"]["rot"]["scaling"].pop("low"), "low"),
])
def test_refusals_name_the_key(edit, text):
    from prism_b200.config.model_config import ConfigError
    raw = copy.deepcopy(CONFIGS["P"][0])
    edit(raw)
    with pytest.raises(ConfigError, match=text):
        build(raw)


def test_what_the_layers_keep_between_steps():
    from prism_b200.engine.runner import cache_groups
    _, mdl = build(CONFIGS["P"][0])
    needs = mdl.cache_needs()
    kinds = [tuple(n.kind for n in need) for need in needs]
    assert kinds == [("paged", "state", "state"), ("state", "state"), ("state", "state"), ("paged", "state", "state")]
    first = needs[0]
    assert (first[0].window, first[0].keep_first, first[0].num_kv_heads, first[0].head_dim, first[0].value_dim) == (13, 3, 2, 16, 24)
    assert first[1].state_shape == (4, 20, 12) and first[2].state_shape == (2, 2 * 2 * 12 + 4 * 20)
    assert needs[1][0].state_shape == (3, 20, 20) and needs[1][1].state_shape == (1, 72)
    groups, where = cache_groups(mdl)
    assert all(isinstance(w, list) and len(w) == len(n) for w, n in zip(where, needs))
    # a layer's views come in the order of its needs, every plane is owned once
    for w, need in zip(where, needs):
        assert [groups[gi].need.group_key() for gi, _, _ in w] == [n.group_key() for n in need]
    planes = [(gi, pi) for w in where for gi, pi, _ in w]
    assert len(planes) == len(set(planes)) == sum(g.num_planes for g in groups)
    # recurrent layers only: nothing is paged
    groups_t, _ = cache_groups(build(CONFIGS["T"][0])[1])
    assert [g.kind for g in groups_t] == ["state"] * len(groups_t)


def test_a_layer_with_several_needs_neither_lends_nor_borrows_a_cache():
    from prism_b200.models.decoder import DecoderModel, ScheduleEntry
    from prism_b200.models.pofazen import PofazenConfig, pofazen_spec
    spec = pofazen_spec(PofazenConfig.from_dict(copy.deepcopy(CONFIGS["P"][0])))
    spec.schedule = [ScheduleEntry(0), ScheduleEntry(1), ScheduleEntry(2), ScheduleEntry(3, reads_cache_of=0)]
    with pytest.raises(ValueError, match="several"):
        DecoderModel(spec)


def test_pages_behind_the_window_come_back_and_the_kept_ones_stay():
    from prism_b200.cache.manager import CacheGroup, CacheManager, pool_sizes
    from prism_b200.parts.base import CacheNeed
    P = 8
    need = CacheNeed("paged", 2, 16, window=13, keep_first=10)
    groups = [CacheGroup(0, need, [0]), CacheGroup(1, CacheNeed("state", state_shape=(3, 4)), [0])]
    cm = CacheManager(groups, P, [12, 0], 2, 400)
    cm.add_request("a")
    held = []
    for n in (5, 20, 1, 1, 30, 2, 40, 7):
        cm.append("a", n)
        cm.commit("a", n)
        cm.check_invariants()
        row = cm.block_table_row("a", 0)
        length = cm.length("a")
        for idx, page in enumerate(row):
            lo, hi = idx * P, (idx + 1) * P
            if lo < 10:
                assert page >= 0, "a page that holds kept first positions was given back"
            elif hi <= length - 13 + 1:
                assert page == -1, "a page wholly behind the window is still held"
            else:
                assert page >= 0
        held.append(cm.pages_in_use())
    assert max(held) <= 2 + 3 + 5 + 1          # kept pages, the window's, one portion's, one more
    freed = cm.num_free_pages(0)
    cm.free_request("a")
    assert cm.num_free_pages(0) == 12 and freed < 12
    cm.add_request("b")
    cm.append("b", 3)
    assert cm.block_table_row("b", 0)[0] in range(12)
    # the pool of a windowed group: window + portion + kept pages per slot
    sizes = pool_sizes(groups, P, 2, 400, 2, 16, None, 1e9)
    assert sizes[0] == 2 * ((13 + 16 + P - 1) // P + 1 + 2) and sizes[1] == 0


def test_the_mask_on_the_host_is_the_plain_mask():
    from prism_b200 import ops
    for size, keep in ((13, 3), (5, 9), (1, 1), (64, 0), (7, 1)):
        m = ops.KeyMask.window(size, keep)
        ref = PP.window_keep_mask(90, size, keep)
        for pos in (0, 1, 4, 12, 13, 14, 40, 89):
            assert [m.sees(pos, j) for j in range(90)] == ref[pos].tolist(), (size, keep, pos)
        assert m.most_keys(1000) == size + keep
    with pytest.raises(ValueError):
        ops.KeyMask(ops.MASK_CHUNK, 8, 2)
    assert ops.KeyMask.window(None, 5).kind == ops.MASK_CAUSAL


def test_rescaled_frequencies_have_three_bands():
    from prism_b200.parts.positions import ScaledRotaryEmbedding
    sc = dict(factor=8.0, low=1.0, high=4.0, original=128)
    f = ScaledRotaryEmbedding(32, 10000.0, sc).frequencies()
    plain = ScaledRotaryEmbedding(32, 10000.0, None).frequencies()
    assert torch.allclose(f, PP.scaled_frequencies(10000.0, 32, sc, torch.float32), rtol=1e-6, atol=0)
    wl = 2 * math.pi / plain
    short, long_ = wl < 128 / 4.0, wl > 128 / 1.0
    assert short.any() and long_.any() and (~short & ~long_).any()
    assert torch.equal(f[short], plain[short]) and torch.allclose(f[long_], plain[long_] / 8.0)
    mid = ~short & ~long_
    assert ((f[mid] < plain[mid]) & (f[mid] > plain[mid] / 8.0)).all()
    assert ScaledRotaryEmbedding(0, 10.0, None).frequencies().numel() == 0


def test_plain_recurrences_do_not_depend_on_where_a_sequence_is_cut():
    """The plain delta rule and wkv loops carry nothing but S (and the inputs before the cut): running a prefix
    and comparing its rows with the whole sequence's rows settles causality of the oracle itself."""
    raw = CONFIGS["P"][0]
    w = {k: v.float() for k, v in draw_weights(raw, 3).items()}
    g = torch.Generator().manual_seed(0)
    h = torch.randn(30, raw["width"], generator=g)
    mx = raw["layers"][0]["mixer"]
    whole = PP.gated_delta(h, w, "l0.mix.right.", mx["right"], 1e-5)
    assert torch.allclose(PP.gated_delta(h[:17], w, "l0.mix.right.", mx["right"], 1e-5), whole[:17], atol=1e-5)
    whole = PP.wkv(h, w, "l1.mix.", raw["layers"][1]["mixer"], 1e-5)
    assert torch.allclose(PP.wkv(h[:9], w, "l1.mix.", raw["layers"][1]["mixer"], 1e-5), whole[:9], atol=1e-5)
    whole = PP.gated_window_attention(h, w, "l0.mix.left.", mx["left"], 1e-5)
    assert torch.allclose(PP.gated_window_attention(h[:20], w, "l0.mix.left.", mx["left"], 1e-5), whole[:20], atol=1e-5)
    # a kept first token matters to a query far behind the window: moving it changes that query's row
    h2 = h.clone()
    h2[1] += 1.0
    far = PP.gated_window_attention(h2, w, "l0.mix.left.", mx["left"], 1e-5)[29]
    assert float((far - whole[29]).abs().max()) > 1e-4
    h3 = h.clone()
    h3[5] += 1.0                   # neither kept (3) nor inside the window (13) of position 29
    assert torch.allclose(PP.gated_window_attention(h3, w, "l0.mix.left.", mx["left"], 1e-5)[29], whole[29], atol=1e-6)


def test_random_weights_mode_draws_a_model_of_the_design(tmp_path):
    from prism_b200.weights.loader import read_safetensors_header
    from prism_b200.weights.random_init import write_model_folder
    raw = model(50, 32, [layer("parallel", parallel(left(2, 1, 8, 16, 6, 2), right(2, 1, 8, 8, 3)), 48),
                         layer("wkv", wkv(2, 8, 4), None)])
    d = write_model_folder(raw, 5, str(tmp_path / "m"))
    names = set(read_safetensors_header(str(tmp_path / "m" / "model.safetensors")))
    assert {"embed.norm", "l0.mix.left.q.norm", "l0.mix.right.q.conv", "l0.mix.right.A_log", "l1.mix.mu.w", "l1.mix.w1",
            "l0.norm2"} <= names
    assert "l1.norm2" not in names           # no feed-forward, no second norm
    assert d

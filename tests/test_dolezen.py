"""Dolezen on the CPU: its configuration and layer plan, what its layers ask of the cache manager, the key
masks, and the plain implementation's mechanisms against properties that follow from their definitions."""

import copy
import math

import pytest
import torch

from dolezen_helpers import CONFIG_X, CONFIG_Y, CONFIG_Z, CONFIGS, DP, draw_weights
from prism_b200 import ops
from prism_b200.cache.manager import CacheManager, plan_groups, pool_sizes
from prism_b200.config.model_config import ConfigError
from prism_b200.model_registry import build_model, resolve
from prism_b200.parts.base import CacheNeed


# ---- configuration and layer plan ---------------------------------------------------------------------

def test_architecture_is_found_by_its_name_string():
    assert resolve(dict(architecture="Dolezen")).name == "Dolezen"
    assert resolve(dict(architectures=["Dolezen"])).name == "Dolezen"
    with pytest.raises(ConfigError):
        resolve(dict(architecture="NoSuchDesign"))


@pytest.mark.parametrize("name", ["X", "Y", "Z"])
def test_the_plan_asks_for_exactly_the_tensors_of_the_file(name):
    raw, seed, _ = CONFIGS[name]
    _, model = build_model(raw)
    asked = {s.name: tuple(s.shape) for _, p in model.named_params() for s in p.sources}
    drawn = {k: tuple(v.shape) for k, v in draw_weights(raw, seed).items()}
    assert asked == drawn


def test_layers_that_use_another_layers_keys_have_no_projections_and_read_its_plane():
    _, model = build_model(CONFIG_X)
    names = {s.name for _, p in model.named_params() for s in p.sources}
    assert "l1.mix.k" in names and "l2.mix.k" not in names and "l3.mix.v.b" not in names and "l2.mix.q" in names
    assert [e.reads_cache_of for e in model.schedule] == [None, None, 1, 1, None]
    assert "l2.mlp.up" not in names            # a layer without feed-forward
    needs = model.cache_needs()
    assert needs[2] is None and needs[3] is None
    # the plane's readers have other masks than its owner: pages are never given back by block
    assert needs[1] == CacheNeed("paged", 2, 16, None, v_head_dim=24, chunk=None)
    # latent layers: one head of rank + rotated entries, no value plane, release by window
    assert needs[0] == CacheNeed("paged", 1, 40, 11, v_head_dim=0)
    assert needs[4] == CacheNeed("paged", 1, 64, 5, v_head_dim=0)


def test_equal_masks_let_a_shared_plane_release_by_block():
    _, model = build_model(CONFIG_Y)
    needs = model.cache_needs()
    assert needs[0] == CacheNeed("paged", 1, 32, None, chunk=70) and needs[1] is None
    assert needs[3] == CacheNeed("paged", 2, 64, None, v_head_dim=16)           # no mask: every key is kept
    assert needs[4] == CacheNeed("paged", 1, 96, None, v_head_dim=0)


def test_constants_come_from_the_file():
    cfg, model = build_model(CONFIG_X)
    assert model.embedding.scale == 3.5 and model.final_norm.eps == 1e-5
    m = model.layers[3].mixer
    assert (m.scale, m.chunk, m.nh, m.nkv, m.hd, m.vhd, m.sink, m.own_kv) == (0.3, 13, 6, 2, 16, 24, True, False)
    lat = model.layers[4].mixer
    assert (lat.rope_dims, lat.rd, lat.kv_rank, lat.q_rank, lat.window, lat.rope_base) == (8, 16, 48, 24, 5, 10000.0)
    assert model.layers[0].mixer.rope_base == 500.0
    assert model.layers[2].feed_forward is None and model.layers[1].feed_forward.activation == "relu2"


@pytest.mark.parametrize("edit, text", [
    (lambda c: c["layers"][2]["mixer"].update(kv_from=2), "kv_from"),
    (lambda c: c["layers"][2]["mixer"].update(kv_from=0), "kv_from"),              # a latent layer has no such plane
    (lambda c: c["layers"][3]["mixer"].update(kv_from=2), "kv_from"),              # layer 2 has no projections itself
    (lambda c: c["layers"][2]["mixer"].update(vdim=16), "equal those of layer 1"),
    (lambda c: c["layers"][1]["mixer"].update(kv_heads=4), "not divisible"),
    (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=10), "rot.dims"),
    (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=3), "rot.dims"),
    (lambda c: c["layers"][0].update(type="recurrent"), "type"),
    (lambda c: c["layers"][1]["mlp"].update(kind="experts"), "dense"),
    (lambda c: c["layers"][1]["mixer"].pop("scale"), "scale"),
    (lambda c: c.pop("norm"), "norm"),
    (lambda c: c["layers"][1]["mixer"]["mask"].update(size=0), "positive"),
])
def test_bad_configurations_are_refused_with_the_key_named(edit, text):
    raw = copy.deepcopy(CONFIG_X)
    edit(raw)
    with pytest.raises(ConfigError, match=text):
        build_model(raw)


# ---- cache manager ------------------------------------------------------------------------------------------

def test_pages_before_the_current_block_are_given_back_and_used_again():
    groups, _ = plan_groups([CacheNeed("paged", 1, 8, None, chunk=20)], [None])
    cm = CacheManager(groups, page_size=8, num_pages=[4], max_seqs=2, max_seq_len=200)
    cm.add_request("a")
    held = []
    for step in range(60):
        cm.append("a", 1)
        cm.commit("a", 1)
        cm.check_invariants()
        n = step + 1
        first = n // 20 * 20                      # the next query sits at position n
        pages = cm.block_table_row("a", 0)
        assert all((p >= 0) == ((i + 1) * 8 > first) for i, p in enumerate(pages)), (n, pages)
        held.append(sum(p >= 0 for p in pages))
    assert max(held) <= 4                          # 60 tokens went through a pool of 4 pages of 8
    assert len({p for p in cm.block_table_row("a", 0)}) <= 5
    cm.free_request("a")
    assert cm.pages_in_use() == 0


def test_a_window_and_a_block_keep_what_the_next_query_sees():
    assert CacheNeed("paged", 1, 8, 5).first_kept(12) == 8
    assert CacheNeed("paged", 1, 8, None, chunk=5).first_kept(12) == 10
    assert CacheNeed("paged", 1, 8, None, chunk=5).first_kept(10) == 10
    assert CacheNeed("paged", 1, 8, None).first_kept(12) == 0


def test_groups_differ_by_value_size_and_release_rule_and_pools_follow():
    a, b = CacheNeed("paged", 2, 16, None, v_head_dim=24), CacheNeed("paged", 2, 16, None)
    c, d = CacheNeed("paged", 1, 40, 11, v_head_dim=0), CacheNeed("paged", 2, 16, None, chunk=32)
    groups, where = plan_groups([a, b, c, a, d], [None] * 5)
    assert [g.entries for g in groups] == [[0, 3], [1], [2], [4]]
    assert where[3] == (0, 1, True)
    sizes = pool_sizes(groups, page_size=16, elem_bytes=2, max_seq_len=4096, max_seqs=4, max_portion=64, num_pages=100)
    assert sizes[0] == 100 and sizes[1] == 100
    assert sizes[2] == 4 * ((11 + 64 + 15) // 16 + 1) and sizes[3] == 4 * ((32 + 64 + 15) // 16 + 1)


# ---- key masks ----------------------------------------------------------------------------------------------------

def test_first_key_of_every_mask_kind():
    w, c, all_ = ops.KeyMask.window(5), ops.KeyMask.chunk(5), ops.KeyMask.causal()
    assert [w.first_key(p) for p in (0, 3, 4, 5, 11)] == [0, 0, 0, 1, 7]
    assert [c.first_key(p) for p in (0, 4, 5, 9, 10, 11)] == [0, 0, 5, 5, 10, 10]
    assert [all_.first_key(p) for p in (0, 7)] == [0, 0]
    assert ops.KeyMask.window(None).kind == ops.MASK_CAUSAL and ops.KeyMask.chunk(1).first_key(9) == 9
    with pytest.raises(ValueError):
        ops.KeyMask(ops.MASK_WINDOW, 0)
    for mask, plain in ((w, DP.sliding_mask(23, 5)), (c, DP.chunk_mask(23, 5))):
        for i in range(23):
            seen = [j for j in range(23) if plain[i, j]]
            assert seen == list(range(mask.first_key(i), i + 1))


# ---- the plain implementation's mechanisms ------------------------------------------------------------------

def test_plain_rotation_turns_pairs_and_passes_the_rest():
    x = torch.randn(7, 3, 12)
    pos = torch.tensor([0, 1, 2, 50, 51, 1000, 7])
    y = DP.rotate(x, pos, 100.0, 8)
    assert torch.equal(y[..., 8:], x[..., 8:]) and torch.allclose(y[0], x[0])
    assert torch.allclose(y[..., :8].norm(dim=-1), x[..., :8].norm(dim=-1), atol=1e-5)
    # the product of a rotated query and a rotated key depends on the distance only
    q, k = torch.randn(1, 8), torch.randn(1, 8)
    a = (DP.rotate(q, torch.tensor([9]), 100.0, 8) * DP.rotate(k, torch.tensor([4]), 100.0, 8)).sum()
    b = (DP.rotate(q, torch.tensor([105]), 100.0, 8) * DP.rotate(k, torch.tensor([100]), 100.0, 8)).sum()
    assert abs(float(a - b)) < 1e-4
    # dimension i turns with frequency base^(-2i/dims): entry 1 of 8 at position 1, base 100
    e = torch.zeros(1, 8)
    e[0, 1] = 1.0
    r = DP.rotate(e, torch.tensor([1]), 100.0, 8)
    ang = 100.0 ** (-2.0 / 8)
    assert torch.allclose(r[0, [1, 5]], torch.tensor([math.cos(ang), math.sin(ang)]), atol=1e-6)


def test_plain_sink_takes_weight_without_a_value():
    s = torch.zeros(2, 3, 3)
    p = DP.masked_softmax(s, DP.chunk_mask(3, 8), torch.tensor([0.0, -1e9]))
    assert torch.allclose(p[0, 2].sum(), torch.tensor(3 / 4)) and torch.allclose(p[1, 2].sum(), torch.tensor(1.0))
    assert torch.allclose(p[0, 0, 0], torch.tensor(0.5))


def test_plain_forward_ignores_what_the_masks_hide():
    """Changing a token changes the logits of exactly the positions that can see it through some chain of
    layers; with a chunked model of one block size and no latent layer, never across a block's edge."""
    raw = dict(architecture="Dolezen", vocab=50, width=24, norm=dict(eps=1e-6), embedding=dict(scale=2.0), layers=[
        dict(type="attention", mixer=dict(heads=2, kv_heads=1, dim=8, vdim=4, scale=0.4, mask=dict(size=6)), mlp=None),
        dict(type="attention", mixer=dict(heads=2, kv_heads=1, dim=8, vdim=4, scale=0.4, mask=dict(size=6), kv_from=0),
             mlp=dict(kind="dense", ff=16))])
    w = {k: v.float() for k, v in draw_weights(raw, 3).items()}
    a = list(range(20))
    b = list(a)
    b[7] = 33
    la, lb = DP.forward(raw, w, a)[0], DP.forward(raw, w, b)[0]
    changed = [i for i in range(20) if not torch.equal(la[i], lb[i])]
    assert changed == [7, 8, 9, 10, 11]


def test_key_splits_of_a_masked_decode_step():
    """As many CTAs per (request, kv head) as fill one wave, each keeping two tiles or more; a mask bounds
    the keys whatever the context."""
    assert ops.masked_decode_splits(8, 4, 1024, sms=148) == 8               # 17 tiles: 8 CTAs of 2 or 3 tiles
    assert ops.masked_decode_splits(8, 4, ops.KeyMask.window(512).most_keys(100000), sms=148) == 4
    assert ops.masked_decode_splits(64, 8, 4096, sms=148) == 1              # 512 CTAs fill the GPU by themselves
    assert ops.masked_decode_splits(1, 1, 40, sms=148) == 1                 # one tile
    assert ops.masked_decode_splits(1, 1, 100000, sms=148) == 64
    assert ops.KeyMask.causal().most_keys(777) == 777 and ops.KeyMask.chunk(200).most_keys(777) == 200

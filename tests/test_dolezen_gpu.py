"""Dolezen on the GPU against the plain implementation (tests/plain/dolezen_plain.py): each kernel alone,
each mixer alone, whole prompts against token-by-token decoding, portions down to two tokens, mixed batches
with pages and slots that are used again, keys at the edges of windows, blocks and pages, and greedy
generation through the engine's scheduler."""

import math
import types

import pytest
import torch

from dolezen_helpers import CONFIGS, DP, attn, compare, latent, layer, model_folder, plain_logits, write_folder, draw_weights
from helpers import random_tokens, run_trace, trace_budget, trace_mixed, trace_portions, trace_tail, trace_whole

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


# ---------------------------------------------------------------------------------------------------------
# kernels alone
# ---------------------------------------------------------------------------------------------------------

def paged_case(segs, nkv, dk, dv, page_size, dtype, seed, values_in_keys=False):
    """Random keys and values for segments ``[(cached, new), ...]`` in a pool whose pages are handed out in a
    scrambled order.  Returns the step's arrays, the planes, and per segment the dense keys and values."""
    g = torch.Generator().manual_seed(seed)
    total_pages = sum((c + n + page_size - 1) // page_size for c, n in segs)
    order = torch.randperm(total_pages + 3, generator=g).tolist()
    W = max((c + n + page_size - 1) // page_size for c, n in segs) + 1
    kp = torch.zeros(total_pages + 4, page_size, nkv, dk)
    vp = kp[..., :dv] if values_in_keys else torch.zeros(total_pages + 4, page_size, nkv, dv)
    bt = torch.full((len(segs), W), total_pages + 3, dtype=torch.int32)
    dense, pos, tok_seg, seg_start, cached = [], [], [], [0], []
    for s, (c, n) in enumerate(segs):
        k = torch.randn(c + n, nkv, dk, generator=g)
        v = k[..., :dv] if values_in_keys else torch.randn(c + n, nkv, dv, generator=g)
        k, v = k.to(dtype).float(), v.to(dtype).float()
        for p in range(c + n):
            if p % page_size == 0:
                bt[s, p // page_size] = order.pop()
            kp[bt[s, p // page_size], p % page_size] = k[p]
            if not values_in_keys:
                vp[bt[s, p // page_size], p % page_size] = v[p]
        dense.append((k, v))
        pos += list(range(c, c + n))
        tok_seg += [s] * n
        seg_start.append(seg_start[-1] + n)
        cached.append(c)
    i32 = lambda x: torch.tensor(x, dtype=torch.int32, device=DEV)
    kp = kp.to(dtype).to(DEV)
    vp = kp[..., :dv] if values_in_keys else vp.to(dtype).to(DEV)
    ctx = types.SimpleNamespace(positions=i32(pos), tok_seg=i32(tok_seg), seg_start=i32(seg_start), cached_len=i32(cached),
                                S=len(segs), max_q_len=max(n for _, n in segs), decode_only=all(n == 1 for _, n in segs),
                                max_kv_len=max(c + n for c, n in segs),
                                err=torch.zeros(1, dtype=torch.int32, device=DEV))
    return ctx, kp, vp, bt.to(DEV), total_pages + 4, dense


def plain_attention(q, dense, segs, nh, nkv, mask_fn, size, scale, sink):
    """``q [T, nh, dk]`` float32 -> ``[T, nh * dv]`` with the plain masks and softmax, segment by segment."""
    out, t0 = [], 0
    for (c, n), (k, v) in zip(segs, dense):
        L = c + n
        qq = torch.zeros(L, nh, q.shape[2])
        qq[c:] = q[t0:t0 + n]
        rep = nh // nkv
        s = torch.einsum("iad,jad->aij", qq, k.repeat_interleave(rep, 1)) * scale
        mask = mask_fn(L, size) if size else DP.chunk_mask(L, L)
        p = DP.masked_softmax(s, mask, sink)
        o = torch.einsum("aij,jad->iad", p, v.repeat_interleave(rep, 1))
        out.append(o[c:].reshape(n, -1))
        t0 += n
    return torch.cat(out)


SHAPES = [  # nh, nkv, dk, dv, values in keys
    (6, 3, 64, 48, False), (6, 2, 16, 24, False), (8, 1, 160, 128, True), (3, 1, 40, 32, True),
    (4, 4, 32, 32, False), (20, 1, 96, 96, True), (4, 1, 320, 288, True), (2, 1, 24, 8, False), (5, 5, 8, 6, False), (70, 1, 48, 16, True),
]
MASKS = [("window", 44), ("chunk", 50), ("window", 1), ("chunk", 7), ("causal", 0), ("window", 230)]


@pytest.mark.parametrize("shape", SHAPES, ids=lambda s: "h%d_g%d_k%d_v%d_%s" % s)
@pytest.mark.parametrize("mask", MASKS, ids=lambda m: "%s%d" % m)
@pytest.mark.parametrize("kernel", ["generic_f32", "generic_bf16", "tc_portions", "tc_decode"])
def test_attention_under_a_mask_with_sink(shape, mask, kernel):
    from prism_b200 import ops
    nh, nkv, dk, dv, vin = shape
    kind, size = mask
    dtype = torch.float32 if kernel == "generic_f32" else torch.bfloat16
    if kernel == "tc_decode":
        segs = [(130, 1), (0, 1), (63, 1), (64, 1), (199, 1), (39, 1)]
    else:
        segs = [(0, 150), (37, 2), (100, 1), (64, 64), (5, 97), (0, 1)]
    page = 16 if kernel.startswith("generic") else 64
    ctx, kp, vp, bt, npages, dense = paged_case(segs, nkv, dk, dv, page, dtype, seed=dk * 7 + size, values_in_keys=vin)
    g = torch.Generator().manual_seed(5)
    T = sum(n for _, n in segs)
    q = (torch.randn(T, nh, dk, generator=g) * 1.5).to(dtype)
    sink = torch.randn(nh, generator=g) * 2 if kind != "causal" else None
    m = {"window": ops.KeyMask.window, "chunk": ops.KeyMask.chunk, "causal": lambda n: ops.KeyMask.causal()}[kind](size)
    scale = 0.7 / math.sqrt(dk)
    out = torch.empty(T, nh * dv, dtype=dtype, device=DEV)
    qd, sd = q.to(DEV), None if sink is None else sink.to(DEV)
    if kernel.startswith("generic"):
        ops.attention_masked_generic(qd, out, kp, vp, bt, ctx.positions, ctx.tok_seg, npages, m, scale, sd, ctx.err)
    else:
        if not ops.attention_masked_tc_ok(qd, kp, vp, nh, nkv, dk, dv):
            pytest.skip("sizes that go to the shape-generic kernel")
        few = kernel == "tc_decode"
        ops.attention_masked_bf16(qd, out, kp, vp, bt, ctx.seg_start, ctx.cached_len, ctx.S, ctx.max_q_len, npages, m,
                                  scale, sd, few, ctx.err)
    assert int(ctx.err.item()) == 0
    ref = plain_attention(q.float(), dense, segs, nh, nkv, DP.sliding_mask if kind == "window" else DP.chunk_mask, size,
                          scale, sink)
    err = float((out.float().cpu() - ref).abs().max())
    assert err <= (3e-5 if dtype == torch.float32 else 2.5e-2), err
    if kernel == "tc_decode" and few:
        # the same with a request's key tiles shared among CTAs (more CTAs than some requests have tiles)
        for ns in (2, 5):
            out2 = torch.zeros_like(out)
            ops.attention_masked_bf16(qd, out2, kp, vp, bt, ctx.seg_start, ctx.cached_len, ctx.S, ctx.max_q_len, npages, m,
                                      scale, sd, True, ctx.err, nsplit=ns)
            assert float((out2.float().cpu() - ref).abs().max()) <= 2.5e-2, ns


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("vin", [False, True], ids=["own_values", "values_in_keys"])
@pytest.mark.parametrize("kind, size", [("window", 37), ("chunk", 64), ("chunk", 50), ("window", 65), ("causal", 0)])
def test_one_key_that_stands_out_is_seen_exactly_when_the_mask_lets_it(dtype, kind, size, vin):
    """Among hundreds of keys one is aligned with the query and carries a value of its own.  The query's
    output holds that value when the key is far away but visible, at a page's border, just inside a window
    or block - and none of it just outside - in a prompt's portion and in a decoded token, on every kernel."""
    from prism_b200 import ops
    nh, nkv, dk, dv, page = (4, 1, 32, 16, 64) if vin else (4, 2, 32, 16, 64)
    m = {"window": ops.KeyMask.window, "chunk": ops.KeyMask.chunk, "causal": lambda n: ops.KeyMask.causal()}[kind](size)
    L = 330
    for qpos in (329, 320, 256, 200, 192, 128, 127, 65, 64, 63, 1, 0):
        lo = m.first_key(qpos)
        keys = sorted({lo, lo + 1, qpos, qpos - 1, lo - 1, lo - 2, qpos // 64 * 64, qpos // 64 * 64 - 1, 0} & set(range(L)))
        for key in keys:
            if key > qpos:
                continue
            visible = key >= lo
            for n_new in ((1, 7) if qpos >= 6 else (1,)):           # decoded alone, or last of a portion
                c = qpos - n_new + 1
                ctx, kp, vp, bt, npages, dense = paged_case([(c, n_new)], nkv, dk, dv, page, dtype, seed=1, values_in_keys=vin)
                # overwrite: the chosen key lies along the key rows' last entry; its value is the all-ones vector
                # times 8 (with the values inside the key rows: the row's leading entries)
                row = bt[0, key // page].item(), key % page
                kp[row[0], row[1]] = 0
                vp[row[0], row[1]] = 8.0
                kp[row[0], row[1], :, dk - 1] = 30.0
                q = torch.zeros(n_new, nh, dk, dtype=dtype, device=DEV)
                q[-1, :, dk - 1] = 30.0
                out = torch.empty(n_new, nh * dv, dtype=dtype, device=DEV)
                variants = ["generic"] + (["tc"] if dtype == torch.bfloat16 else [])
                for variant in variants:
                    if variant == "generic":
                        ops.attention_masked_generic(q, out, kp, vp, bt, ctx.positions, ctx.tok_seg, npages, m, 1.0,
                                                     None, ctx.err)
                    else:
                        ops.attention_masked_bf16(q, out, kp, vp, bt, ctx.seg_start, ctx.cached_len, 1, n_new, npages,
                                                  m, 1.0, None, n_new == 1, ctx.err)
                    got = float(out[-1].float().mean())
                    if visible:
                        assert got > 7.9, (variant, qpos, key, n_new, got)
                    else:
                        assert got < 4.0, (variant, qpos, key, n_new, got)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_a_large_sink_takes_the_weight(dtype):
    from prism_b200 import ops
    ctx, kp, vp, bt, npages, dense = paged_case([(20, 3)], 1, 16, 16, 64, dtype, seed=2)
    vp.fill_(1.0)
    q = torch.zeros(3, 2, 16, dtype=dtype, device=DEV)
    sink = torch.tensor([math.log(23.0 * 3), -50.0], device=DEV)         # head 0: 3/4 of the weight at position 22
    out = torch.empty(3, 32, dtype=dtype, device=DEV)
    for tc in ([False, True] if dtype == torch.bfloat16 else [False]):
        if tc:
            ops.attention_masked_bf16(q, out, kp, vp, bt, ctx.seg_start, ctx.cached_len, 1, 3, npages, ops.KeyMask.causal(),
                                      0.3, sink, False, ctx.err)
        else:
            ops.attention_masked_generic(q, out, kp, vp, bt, ctx.positions, ctx.tok_seg, npages, ops.KeyMask.causal(), 0.3,
                                         sink, ctx.err)
        o = out.float().cpu()
        assert torch.allclose(o[2, :16], torch.full((16,), 0.25), atol=4e-3) and torch.allclose(o[2, 16:], torch.ones(16), atol=4e-3)
        assert torch.allclose(o[0, :16], torch.full((16,), 21 / (21 + 69.0)), atol=4e-3)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("R, r, dims", [(32, 8, 8), (48, 16, 8), (8, 0, 0), (130, 6, 2)])
def test_latent_cache_row_and_query_rotation(dtype, R, r, dims):
    from prism_b200 import ops
    T, page = 9, 4
    g = torch.Generator().manual_seed(R)
    x = torch.randn(T, 5 + R + r, generator=g) * 3
    w = (torch.randn(R, generator=g) * 0.2 + 1).to(dtype)
    pos = [0, 1, 2, 3, 1000, 5, 77, 7, 12345]                 # pages 0, 250, 1, 19, 3086 of the request
    bt = torch.full((1, 3087), 7, dtype=torch.int32)
    for logical, physical in ((0, 2), (1, 0), (19, 1), (250, 5), (3086, 6)):
        bt[0, logical] = physical
    bt = bt.to(DEV)
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=DEV)
    plane = torch.zeros(8, page, 1, R + r, dtype=dtype, device=DEV)
    inv = (50.0 ** (-2.0 * torch.arange(dims // 2, dtype=torch.float64) / max(dims, 1))).float().to(DEV)
    err = torch.zeros(1, dtype=torch.int32, device=DEV)
    wq = (torch.randn(5, generator=g) * 0.2 + 1).to(dtype)
    cq = torch.zeros(T, 7, dtype=dtype, device=DEV)
    xd = x.to(DEV)
    ops.latent_kv_store(xd[:, 5:], w.to(DEV), 1e-5, R, dims, inv, plane, bt, i32(pos), i32([0] * T), 8, 1 << 20, err,
                        xq=xd[:, :5], q_weight=wq.to(DEV), q_out=cq[:, 1:6])
    assert int(err.item()) == 0
    # the query latent (the matrix's first columns), normed by the same launch into a strided output
    assert torch.allclose(cq[:, 1:6].float().cpu(), DP.rms_norm(x[:, :5], wq.float(), 1e-5), atol=1e-5 if dtype == torch.float32 else 3e-2)
    assert float(cq[:, 0].abs().max()) == 0 and float(cq[:, 6].abs().max()) == 0
    c = DP.rms_norm(x[:, 5:5 + R], w.float(), 1e-5)
    kr = DP.rotate(x[:, 5 + R:], torch.tensor(pos), 50.0, dims) if r else x[:, 5 + R:]
    tol = 1e-5 if dtype == torch.float32 else 2e-2
    for t, p in enumerate(pos):
        row = plane[bt[0, p // page].item(), p % page, 0].float().cpu()
        assert torch.allclose(row[:R], c[t], atol=tol * 4), (t, (row[:R] - c[t]).abs().max())
        # the kernel forms the angle position * frequency in float32, the plain code in float64: at position p the
        # two differ by up to p * 2^-24 radians, times entries of up to about 10
        assert torch.allclose(row[R:], kr[t], atol=tol * 60 + p * 1.2e-6), (t, (row[R:] - kr[t]).abs().max())
    assert int((plane[7] != 0).sum()) == 0 and int((plane[3:5] != 0).sum()) == 0
    if r:
        src = (torch.randn(T, 3, 7 + r, generator=g)).to(dtype).to(DEV)
        dst = torch.zeros(T, 3, 11 + r, dtype=dtype, device=DEV)
        ops.rotate_slice(src[:, :, 7:], dst[:, :, 11:], dims, inv, i32(pos))
        ref = DP.rotate(src[:, :, 7:].float().cpu(), torch.tensor(pos), 50.0, dims)
        assert torch.allclose(dst[:, :, 11:].float().cpu(), ref, atol=4e-3 if dtype == torch.float32 else 3e-2)
        assert float(dst[:, :, :11].abs().max()) == 0


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_small_kernels(dtype):
    from prism_b200 import ops
    g = torch.Generator().manual_seed(1)
    x = (torch.randn(5, 40, generator=g) * 2).to(dtype)
    z = x.float()
    want = {"relu2": torch.clamp(z, min=0) ** 2, "relu": torch.clamp(z, min=0), "silu": z / (1 + torch.exp(-z)),
            "gelu_tanh": 0.5 * z * (1 + torch.tanh(math.sqrt(2 / math.pi) * (z + 0.044715 * z ** 3)))}
    for kind, ref in want.items():
        for cols in (40, 37):
            wide = torch.zeros(5, 64, dtype=dtype, device=DEV)
            ops.activation(x.to(DEV)[:, :cols], wide[:, 8:8 + cols], kind)
            assert torch.allclose(wide[:, 8:8 + cols].float().cpu(), ref[:, :cols], atol=1e-5 if dtype == torch.float32 else 5e-2)
            assert float(wide[:, :8].abs().max()) == 0 and float(wide[:, 8 + cols:].abs().max()) == 0
    # rows of a float32 matrix normed into a strided output
    xf = torch.randn(6, 50, generator=g)
    w = (torch.rand(24, generator=g) + 0.5).to(dtype)
    out = torch.zeros(6, 30, dtype=dtype, device=DEV)
    ops.rms_rows(xf.to(DEV)[:, 3:27], w.to(DEV), 1e-3, out[:, 2:26])
    assert torch.allclose(out[:, 2:26].float().cpu(), DP.rms_norm(xf[:, 3:27], w.float(), 1e-3), atol=1e-5 if dtype == torch.float32 else 3e-2)
    # embedding rows times a scale, in float32
    table = torch.randn(11, 24, generator=g).to(dtype)
    ids = torch.tensor([3, 0, 10], dtype=torch.int32, device=DEV)
    res = torch.empty(3, 24, device=DEV)
    ops.embed(ids, table.to(DEV), res, torch.zeros(1, dtype=torch.int32, device=DEV), 7.25)
    assert torch.equal(res.cpu(), table.float()[[3, 0, 10]] * 7.25)
    # rows into a paged plane
    src = torch.randn(4, 30, generator=g).to(dtype).to(DEV)
    plane = torch.zeros(5, 8, 2, 6, dtype=dtype, device=DEV)
    bt = torch.tensor([[4, 1], [0, 2]], dtype=torch.int32, device=DEV)
    e = torch.zeros(1, dtype=torch.int32, device=DEV)
    ops.cache_store(src[:, 9:21], plane, bt, torch.tensor([7, 8, 0, 15], dtype=torch.int32, device=DEV),
                    torch.tensor([0, 0, 1, 1], dtype=torch.int32, device=DEV), 5, 100, e)
    for t, (pg, sl) in enumerate([(4, 7), (1, 0), (0, 0), (2, 7)]):
        assert torch.equal(plane[pg, sl].reshape(-1), src[t, 9:21])
    assert int((plane != 0).sum()) <= 48 and int(e.item()) == 0
    # two planes of different widths in one launch
    plane.zero_()
    plane2 = torch.zeros(5, 8, 2, 4, dtype=dtype, device=DEV)
    ops.cache_store(src[:, 9:21], plane, bt, torch.tensor([7, 8, 0, 15], dtype=torch.int32, device=DEV),
                    torch.tensor([0, 0, 1, 1], dtype=torch.int32, device=DEV), 5, 100, e, src2=src[:, 21:29], plane2=plane2)
    for t, (pg, sl) in enumerate([(4, 7), (1, 0), (0, 0), (2, 7)]):
        assert torch.equal(plane[pg, sl].reshape(-1), src[t, 9:21]) and torch.equal(plane2[pg, sl].reshape(-1), src[t, 21:29])
    assert int((plane2 != 0).sum()) <= 32 and int(e.item()) == 0


# ---------------------------------------------------------------------------------------------------------
# models
# ---------------------------------------------------------------------------------------------------------

LIMIT = {"float32": 2e-5, "bfloat16": 3e-2}
LENGTHS = {"X": [1, 9, 40, 71, 130], "Y": [2, 65, 128, 200, 333], "Z": [1, 5, 33], "W": [3, 26, 61]}


def runner_for(folder, dtype, max_tokens, page_size, max_live=4):
    from prism_b200.engine.replay import build_runner
    return build_runner(folder, dtype, max_tokens, page_size, max_live)[3]


def sequences(name):
    vocab = CONFIGS[name][0]["vocab"]
    return {f"r{i}": random_tokens(vocab, n, 300 + i) for i, n in enumerate(LENGTHS[name])}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["X", "Y", "Z", "W"])
@pytest.mark.parametrize("mode", ["whole", "tail", "portions", "small_portions", "mixed"])
def test_cutting(name, dtype, mode):
    """Whole prompts, a decoded tail, portions (one schedule of twos and threes only), and mixed batches of up
    to four live requests in a pool that holds no more than the schedule needs, so that pages and slots come
    back and are used again."""
    seqs = sequences(name)
    steps = {"whole": trace_whole, "tail": lambda s: trace_tail(s, 48), "portions": trace_portions,
             "small_portions": lambda s: trace_portions(s, (2, 3, 2, 2, 5, 2)),
             "mixed": lambda s: trace_mixed(s, seed=3)}[mode](seqs)
    ps = CONFIGS[name][2]
    unit = max(ps, 64)
    runner = runner_for(model_folder(name), dtype, trace_budget(steps, unit), ps)
    got = run_trace(runner, steps)
    assert len(got) == sum(len(s) for s in seqs.values())
    compare(name, seqs, got, LIMIT[dtype])
    assert runner.cache.pages_in_use() == 0


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding_across_windows_blocks_and_pages(dtype):
    seq = random_tokens(CONFIGS["Y"][0]["vocab"], 420, 9)
    steps = trace_tail({"a": seq}, 300)
    runner = runner_for(model_folder("Y"), dtype, 448, 64)
    got = run_trace(runner, steps)
    compare("Y", {"a": seq}, got, LIMIT[dtype])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_batches_of_unequal_requests_against_each_alone(dtype):
    seqs = sequences("X")
    ps = CONFIGS["X"][2]
    alone = run_trace(runner_for(model_folder("X"), dtype, 4096, ps), trace_portions(seqs, (5, 2, 9)))
    together = run_trace(runner_for(model_folder("X"), dtype, 4096, ps, max_live=5), trace_mixed(seqs, seed=11, max_live=5))
    tol = 2e-5 if dtype == "float32" else 6e-2
    for key, row in alone.items():
        assert float((row - together[key]).abs().max()) <= tol * max(1.0, float(row.abs().max())), key


def one_layer(kind, mixer, ff=None, width=48, vocab=97, scale=2.0):
    return dict(architecture="Dolezen", vocab=vocab, width=width, norm=dict(eps=1e-6), embedding=dict(scale=scale),
                layers=[layer(kind, mixer, ff)])


ONE_LAYER = {
    "chunked_sink": one_layer("attention", attn(4, 2, 16, 8, 9)),
    "chunked_sink_one_group": one_layer("attention", attn(3, 1, 32, 32, 21, scale=0.11)),
    "latent": one_layer("latent_attention", latent(4, 16, 16, 16, 24, 32, 12, base=300.0)),
    "latent_part_rotated": one_layer("latent_attention", latent(2, 8, 24, 40, 16, 16, 30, dims=4)),
    "feed_forward": one_layer("attention", attn(1, 1, 8, 8, 1), ff=112),
    "odd_sizes": one_layer("attention", attn(2, 1, 7, 5, 6), ff=33, width=37, vocab=51),
    "wide_heads": one_layer("attention", attn(2, 2, 272, 264, 40), width=64),
    "latent_odd": one_layer("latent_attention", latent(3, 5, 6, 7, 9, 11, 4, dims=2), width=29, vocab=40),
}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("which", sorted(ONE_LAYER))
def test_each_mixer_alone(which, dtype):
    raw = ONE_LAYER[which]
    w = draw_weights(raw, 21)
    folder = write_folder(raw, w)
    seq = random_tokens(raw["vocab"], 75, 4)
    ref = DP.forward(raw, {k: v.float() for k, v in w.items()}, seq)[0]
    runner = runner_for(folder, dtype, 128, 16)
    got = run_trace(runner, trace_portions({"a": seq}, (20, 1, 1, 30, 2, 1)))
    scale = float((ref - ref.mean(-1, keepdim=True)).pow(2).mean().sqrt())
    worst = max(float((got[("a", p)] - ref[p] - (got[("a", p)] - ref[p]).mean()).pow(2).mean().sqrt()) / scale for p in range(75))
    assert worst <= LIMIT[dtype], worst


def test_greedy_generation_through_the_scheduler():
    """Engine.generate (scheduler, batching, sampling, CUDA graphs for the decode steps) picks the plain
    model's greedy tokens."""
    from prism_b200.config.engine_config import EngineConfig, SchedulerConfig
    from prism_b200.engine.llm import Engine
    from prism_b200.sampling.sampler import SamplingParams
    raw = CONFIGS["X"][0]
    w = {k: v.float() for k, v in draw_weights(raw, CONFIGS["X"][1]).items()}
    prompts = [random_tokens(raw["vocab"], n, 40 + n) for n in (3, 17, 30, 8, 1)]
    n_new = 24
    for graphs in (False, True):
        eng = Engine(model_folder("X"), EngineConfig(kv_page_size=8, num_pages=40, max_seq_len=128, use_cuda_graph=graphs,
                                                      graph_batch_sizes=(1, 2, 4, 8),
                                                      scheduler=SchedulerConfig(max_batch_tokens=48, max_num_seqs=4, prefill_chunk=16)),
                     dtype="float32")
        res = eng.generate(prompts, SamplingParams(max_new_tokens=n_new, ignore_eos=True))
        for p, r in zip(prompts, res):
            seq = list(p)
            for tok in r.token_ids:
                logits = DP.forward(raw, w, seq)[0][-1]
                top = torch.topk(logits, 2).values
                if float(top[0] - top[1]) > 1e-3:          # a near tie may fall either way
                    assert tok == int(logits.argmax()), (graphs, len(p), len(seq))
                seq.append(tok)
            assert len(r.token_ids) == n_new
        assert eng.cache.pages_in_use() == 0


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_the_replay_program_serves_the_design(tmp_path, dtype):
    """bin/trace_run as a user runs it, on a Dolezen folder: the model class is found by config.json, the pool
    holds what --max-tokens says, steps come as JSON lines and logits leave as <step>.f32 files."""
    import json
    import os
    import subprocess
    import sys
    import numpy as np
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    name = "X"
    vocab = CONFIGS[name][0]["vocab"]
    seqs = {f"q{i}": random_tokens(vocab, n, 500 + i) for i, n in enumerate([70, 33, 90, 12, 64, 5])}
    steps = trace_mixed(seqs, seed=17)
    out = tmp_path / "out"
    proc = subprocess.run([sys.executable, os.path.join(root, "bin", "trace_run"), "--model", model_folder(name), "--dtype", dtype,
                           "--out", str(out), "--max-tokens", str(trace_budget(steps, 64))],
                          input="\n".join(json.dumps(s) for s in steps) + "\n", capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    assert [l for l in proc.stdout.split("\n") if l.startswith("done")] == [f"done {s['step']}" for s in steps]
    got, fed = {}, {}
    for s in steps:
        n_want = sum(len(e["want"]) for e in s["entries"])
        data = np.fromfile(out / f"{s['step']}.f32", dtype="<f4").reshape(n_want, vocab)
        r = 0
        for e in s["entries"]:
            for w in e["want"]:
                got[(e["id"], fed.get(e["id"], 0) + w)] = torch.from_numpy(data[r].copy())
                r += 1
            fed[e["id"]] = fed.get(e["id"], 0) + len(e["tokens"])
    assert len(got) == sum(len(s) for s in seqs.values())
    compare(name, seqs, got, LIMIT[dtype])

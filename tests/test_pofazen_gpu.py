"""Pofazen on the GPU against the plain implementation (tests/plain/pofazen_plain.py): each kernel alone, each
mixer alone, whole prompts against token-by-token decoding, portions down to two tokens, mixed batches with
pages and state slots that are used again, keys at the edges of windows, kept tokens and pages, long decoding,
and greedy generation through the engine's scheduler."""

import math
import types

import pytest
import torch

from pofazen_helpers import (CONFIGS, PP, compare, draw_weights, layer, left, model, model_folder, parallel, right,
                             wkv, write_folder)
from helpers import random_tokens, run_trace, trace_budget, trace_mixed, trace_portions, trace_tail, trace_whole

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


# ---------------------------------------------------------------------------------------------------------
# kernels alone
# ---------------------------------------------------------------------------------------------------------

def paged_case(segs, nkv, dk, dv, page_size, dtype, seed):
    """``segs``: (cached, new) per request.  Keys and values of every position in pages handed out in a scrambled
    order; returns the step's descriptor arrays, the planes, and the dense keys/values per request."""
    from prism_b200 import ops  # noqa: F401
    g = torch.Generator().manual_seed(seed)
    pages_per = [(-(-(c + n) // page_size)) for c, n in segs]
    total = sum(pages_per)
    order = torch.randperm(total + 3, generator=g).tolist()
    W = max(pages_per)
    bt = torch.full((len(segs), W), total + 3, dtype=torch.int32)
    kc = torch.randn(total + 4, page_size, nkv, dk, generator=g)
    vc = torch.randn(total + 4, page_size, nkv, dv, generator=g)
    dense, o = [], 0
    for s, (c, n) in enumerate(segs):
        ids = order[o:o + pages_per[s]]
        o += pages_per[s]
        bt[s, :len(ids)] = torch.tensor(ids, dtype=torch.int32)
        dense.append((kc[ids].reshape(-1, nkv, dk)[:c + n], vc[ids].reshape(-1, nkv, dv)[:c + n]))
    pos = torch.cat([torch.arange(c, c + n) for c, n in segs]).to(torch.int32)
    tok_seg = torch.cat([torch.full((n,), s) for s, (c, n) in enumerate(segs)]).to(torch.int32)
    seg_start = torch.tensor([0] + list(torch.tensor([n for _, n in segs]).cumsum(0)), dtype=torch.int32)
    ctx = types.SimpleNamespace(
        positions=pos.to(DEV), tok_seg=tok_seg.to(DEV), seg_start=seg_start.to(DEV),
        cached_len=torch.tensor([c for c, _ in segs], dtype=torch.int32, device=DEV), S=len(segs),
        max_q_len=max(n for _, n in segs), max_kv_len=max(c + n for c, n in segs),
        decode_only=all(n == 1 for _, n in segs), err=torch.zeros(1, dtype=torch.int32, device=DEV))
    return ctx, kc.to(dtype).to(DEV), vc.to(dtype).to(DEV), bt.to(DEV), total + 4, dense


def plain_window_attention(q, dense, segs, nh, nkv, window, keep, scale):
    outs, t = [], 0
    for (c, n), (k, v) in zip(segs, dense):
        vis = PP.window_keep_mask(c + n, window if window else c + n + 1, keep)[c:]
        o = torch.empty(n, nh, v.shape[-1])
        for h in range(nh):
            g = h // (nh // nkv)
            s = (q[t:t + n, h] @ k[:, g].T) * scale
            o[:, h] = torch.softmax(s.masked_fill(~vis, -math.inf), -1) @ v[:, g]
        outs.append(o.reshape(n, -1))
        t += n
    return torch.cat(outs)


SHAPES = [(4, 2, 16, 24), (3, 1, 32, 32), (6, 6, 64, 16), (2, 1, 7, 5), (16, 4, 128, 128)]      # nh, nkv, dk, dv
MASKS = [(13, 3), (64, 4), (70, 40), (5, 9), (1, 1), (0, 0), (100, 0)]                            # window (0: none), keep


def run_attention(kernel, segs, shape, window, keep, page_size, seed, q=None, boost=None):
    from prism_b200 import ops
    nh, nkv, dk, dv = shape
    dtype = torch.float32 if kernel == "generic_f32" else torch.bfloat16
    ctx, kc, vc, bt, npages, dense = paged_case(segs, nkv, dk, dv, page_size, dtype, seed)
    T = int(ctx.positions.shape[0])
    g = torch.Generator().manual_seed(seed + 1)
    q = torch.randn(T, nh, dk, generator=g) if q is None else q
    if boost is not None:
        boost(q, kc, vc, bt, dense)
    dense = [(k.to(dtype).float(), v.to(dtype).float()) for k, v in dense]
    qd = q.to(dtype).to(DEV)
    out = torch.empty(T, nh * dv, dtype=dtype, device=DEV)
    mask = ops.KeyMask.window(window, keep) if window else ops.KeyMask.causal()
    scale = dk ** -0.5
    if kernel.startswith("generic"):
        ops.attention_masked_generic(qd, out, kc, vc, bt, ctx.positions, ctx.tok_seg, npages, mask, scale, None, ctx.err)
    else:
        few = kernel.startswith("tc_decode")
        ns = int(kernel.split(":")[1]) if ":" in kernel else 1
        ops.attention_masked_bf16(qd, out, kc, vc, bt, ctx.seg_start, ctx.cached_len, ctx.S, ctx.max_q_len, npages, mask,
                                  scale, None, few, ctx.err, nsplit=ns)
    assert int(ctx.err.item()) == 0
    ref = plain_window_attention(qd.float().cpu(), dense, segs, nh, nkv, window, keep, scale)
    return out.float().cpu(), ref


@pytest.mark.parametrize("shape", SHAPES, ids=lambda s: "h%d_g%d_k%d_v%d" % s)
@pytest.mark.parametrize("mask", MASKS, ids=lambda m: "w%d_keep%d" % m)
@pytest.mark.parametrize("kernel", ["generic_f32", "generic_bf16", "tc_portions", "tc_decode", "tc_decode:3"])
def test_attention_under_a_window_that_keeps_first_tokens(shape, mask, kernel):
    from prism_b200 import ops
    nh, nkv, dk, dv = shape
    if kernel.startswith("tc") and not ops.lib().prism_attention_masked_supported(dk, dv, nh, nkv):
        pytest.skip("the tensor-core kernel leaves this shape to the generic one")
    if kernel.startswith("tc") and dv % 8:
        pytest.skip("values in whole 16-byte pieces only")
    window, keep = mask
    if kernel.startswith("tc_decode"):
        segs = [(0, 1), (3, 1), (12, 1), (63, 1), (64, 1), (130, 1), (257, 1)]
    else:
        segs = [(0, 1), (0, 37), (5, 2), (60, 9), (100, 80), (199, 1), (3, 130)]
    got, ref = run_attention(kernel, segs, shape, window, keep, 16 if dk < 64 else 64, 5)
    tol = 2e-5 if kernel == "generic_f32" else 2e-2
    assert float((got - ref).abs().max()) <= tol


@pytest.mark.parametrize("kernel", ["generic_f32", "generic_bf16", "tc_portions", "tc_decode", "tc_decode:4"])
@pytest.mark.parametrize("window, keep", [(37, 4), (64, 1), (65, 70), (200, 3)])
def test_one_key_that_stands_out_is_seen_exactly_when_the_mask_lets_it(kernel, window, keep):
    """One key of a long context gets a score far above all others and a value of its own.  The output is that
    value when the query sees the key - far back among hundreds but a kept first token, at a page border, the
    last one inside the window - and shows nothing of it when it does not: just outside the window, the first
    token that is not kept."""
    nh, nkv, dk, dv = 4, 2, 32, 32
    ctx_len = 700
    decode = kernel.startswith("tc_decode")
    cases = []
    for qpos in (ctx_len - 1, ctx_len - 40):
        lo = qpos - window + 1
        for key in (0, keep - 1, keep, lo - 1, lo, lo + 1, qpos, 63, 64, 640, 639):
            if 0 <= key <= qpos:
                cases.append((qpos, key))
    for qpos, key in cases:
        segs = [(qpos, 1)] if decode else [(qpos - 5, 9)]
        row = 0 if decode else 5

        def boost(q, kc, vc, bt, dense, key=key):
            k, v = dense[0]
            k[key] = 0.0
            k[key, :, 0] = 30.0
            v[key] = 7.0
            q[row, :, 0] = 30.0
            page, at = int(bt[0, key // 64]), key % 64
            kc[page, at] = k[key].to(kc.dtype)
            vc[page, at] = v[key].to(vc.dtype)
        got, ref = run_attention(kernel, segs, (nh, nkv, dk, dv), window, keep, 64, 9, boost=boost)
        seen = key <= qpos and (qpos - key < window or key < keep)
        val = got[row].view(nh, dv)
        if seen:
            assert float((val - 7.0).abs().max()) < 0.05, (qpos, key, "should be seen")
        else:
            assert float(val.abs().max()) < 4.0, (qpos, key, "should not be seen")
        assert float((got - ref).abs().max()) <= (2e-5 if kernel == "generic_f32" else 3e-2), (qpos, key)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("nh, nkv, dk, dv, rot", [(4, 2, 16, 24, 8), (3, 3, 10, 14, 6), (1, 1, 8, 8, 0), (2, 1, 64, 32, 64)])
def test_query_key_norm_rotation_and_store(dtype, nh, nkv, dk, dv, rot):
    from prism_b200 import ops
    from prism_b200.parts.positions import ScaledRotaryEmbedding
    segs = [(0, 3), (12340, 6), (63, 2)]
    ctx, kc, vc, bt, npages, _ = paged_case(segs, nkv, dk, dv, 64, dtype, 2)
    T = 11
    g = torch.Generator().manual_seed(3)
    proj = torch.randn(T, nh * dk + nkv * dk + nkv * dv + 5, generator=g)
    wq, wk = torch.randn(dk, generator=g) * 0.3 + 1, torch.randn(dk, generator=g) * 0.3 + 1
    scaling = dict(factor=4.0, low=1.0, high=4.0, original=64)
    part = ScaledRotaryEmbedding(rot, 300.0, scaling)
    freq = part.frequencies()
    assert torch.allclose(freq, PP.scaled_frequencies(300.0, rot, scaling, torch.float32), rtol=1e-6, atol=0)
    pd = proj.to(DEV)
    a, b, c = nh * dk, nh * dk + nkv * dk, nh * dk + nkv * dk + nkv * dv
    q_out = torch.empty(T, nh, dk, dtype=dtype, device=DEV)
    ops.qk_norm_rope_store(pd[:, :a], pd[:, a:b], pd[:, b:c], wq.to(DEV), wk.to(DEV), 1e-5, freq.to(DEV) if rot else None,
                           rot, q_out, kc, vc, bt, ctx.positions, ctx.tok_seg, npages, 1 << 20, ctx.err)
    assert int(ctx.err.item()) == 0
    pos = ctx.positions.cpu().long()
    f64 = PP.scaled_frequencies(300.0, rot, scaling, torch.float32)
    q_ref = PP.rotate_interleaved(PP.rms_norm(proj[:, :a].view(T, nh, dk), wq, 1e-5), pos, f64) if rot else \
        PP.rms_norm(proj[:, :a].view(T, nh, dk), wq, 1e-5)
    k_ref = PP.rms_norm(proj[:, a:b].view(T, nkv, dk), wk, 1e-5)
    if rot:
        k_ref = PP.rotate_interleaved(k_ref, pos, f64)
    tol = 2e-3 if dtype == torch.float32 else 4e-2          # float32 sin/cos of angles up to 12,345 radians
    assert float((q_out.float().cpu() - q_ref).abs().max()) <= tol
    seg_of = ctx.tok_seg.cpu().tolist()
    for t in range(T):
        p = int(pos[t])
        page = int(bt[seg_of[t], p // 64])
        assert float((kc[page, p % 64].float().cpu() - k_ref[t]).abs().max()) <= tol
        assert float((vc[page, p % 64].float().cpu() - proj[t, b:c].view(nkv, dv)).abs().max()) <= (1e-6 if dtype == torch.float32 else 2e-2)


def step_ctx(qlens, slots):
    seg_start = torch.tensor([0] + list(torch.tensor(qlens).cumsum(0)), dtype=torch.int32, device=DEV)
    tok_seg = torch.cat([torch.full((n,), s) for s, n in enumerate(qlens)]).to(torch.int32).to(DEV)
    return types.SimpleNamespace(seg_start=seg_start, tok_seg=tok_seg, S=len(qlens),
                                 state_slots=torch.tensor(slots, dtype=torch.int32, device=DEV))


def cut(total, sizes):
    out, at, k = [], 0, 0
    while at < total:
        n = min(sizes[k % len(sizes)], total - at)
        out.append((at, n))
        at, k = at + n, k + 1
    return out


@pytest.mark.parametrize("G, rep, dk, dv", [(1, 2, 32, 64), (2, 2, 12, 20), (1, 1, 1, 1), (1, 3, 7, 5), (2, 1, 40, 8), (1, 1, 300, 16),
                                            (1, 2, 128, 128), (1, 1, 64, 200)])
def test_delta_rule_scan_in_pieces_against_the_plain_loop(G, rep, dk, dv):
    """Two requests of unequal length, cut into portions down to one token and run through the scan with their
    states in slots 2 and 0; the plain loop runs each whole."""
    from prism_b200 import ops
    H = G * rep
    g = torch.Generator().manual_seed(dk * 100 + dv)
    lens = [150, 37]
    data = []
    for n in lens:
        q = torch.nn.functional.normalize(torch.randn(n, G, dk, generator=g), dim=-1) * dk ** -0.5
        k = torch.nn.functional.normalize(torch.randn(n, G, dk, generator=g), dim=-1)
        v = torch.randn(n, H, dv, generator=g)
        beta, dec = torch.rand(n, H, generator=g), torch.rand(n, H, generator=g) * 0.6 + 0.4
        ref = torch.empty(n, H, dv)
        for h in range(H):
            S = torch.zeros(dk, dv)
            for t in range(n):
                S = dec[t, h] * S
                u = beta[t, h] * (v[t, h] - S.T @ k[t, h // rep])
                S = S + torch.outer(k[t, h // rep], u)
                ref[t, h] = S.T @ q[t, h // rep]
        data.append((torch.cat([q.reshape(n, -1), k.reshape(n, -1), v.reshape(n, -1)], 1), torch.cat([beta, dec], 1), ref))
    state = torch.zeros(4, H, dv, dk, device=DEV)
    state[1] = 9.0                                     # a neighbour's state: must stay as it is
    cuts = [cut(lens[0], (40, 1, 1, 17, 2, 64)), cut(lens[1], (5, 2, 1, 30))]
    got = [torch.empty(n, H, dv) for n in lens]
    for step in range(max(len(c) for c in cuts)):
        act = [(r, cuts[r][step]) for r in range(2) if step < len(cuts[r])]
        x = torch.cat([data[r][0][a:a + n] for r, (a, n) in act]).to(DEV)
        bg = torch.cat([data[r][1][a:a + n] for r, (a, n) in act]).to(DEV).contiguous()
        ctx = step_ctx([n for _, (_, n) in act], [(2, 0)[r] for r, _ in act])
        o = torch.empty(x.shape[0], H, dv, device=DEV)
        ops.recurrent_scan(ops.SCAN_DELTA, x[:, :G * dk], x[:, G * dk:2 * G * dk], x[:, 2 * G * dk:], state, ctx, H, rep, dk, dv, o, bg=bg)
        at = 0
        for r, (a, n) in act:
            got[r][a:a + n] = o[at:at + n].cpu()
            at += n
    for r in range(2):
        assert float((got[r] - data[r][2]).abs().max()) <= 2e-5 * max(1.0, float(data[r][2].abs().max())), r
    assert float((state[1] - 9.0).abs().max()) == 0.0


@pytest.mark.parametrize("H, d", [(2, 32), (3, 20), (1, 1), (1, 7), (2, 64), (1, 300)])
def test_bonus_scan_in_pieces_against_the_plain_loop(H, d):
    from prism_b200 import ops
    g = torch.Generator().manual_seed(d)
    lens = [90, 41]
    w0, u = torch.randn(H * d, generator=g) * 0.5 - 1.0, torch.randn(H * d, generator=g) * 0.5
    data = []
    for n in lens:
        r, k, v = (torch.randn(n, H, d, generator=g) * 0.5 for _ in range(3))
        ww = torch.randn(n, H * d, generator=g)
        w = torch.exp(-torch.exp(ww + w0)).view(n, H, d)
        ref = torch.empty(n, H, d)
        for h in range(H):
            S = torch.zeros(d, d)
            for t in range(n):
                kv = torch.outer(k[t, h], v[t, h])
                ref[t, h] = (S + u.view(H, d)[h][:, None] * kv).T @ r[t, h]
                S = w[t, h][:, None] * S + kv
        data.append((torch.cat([r.reshape(n, -1), k.reshape(n, -1), v.reshape(n, -1)], 1), ww, ref))
    state = torch.zeros(3, H, d, d, device=DEV)
    cuts = [cut(lens[0], (33, 1, 2, 1, 20)), cut(lens[1], (2, 2, 17, 1))]
    got = [torch.empty(n, H, d) for n in lens]
    A = H * d
    for step in range(max(len(c) for c in cuts)):
        act = [(r, cuts[r][step]) for r in range(2) if step < len(cuts[r])]
        x = torch.cat([data[r][0][a:a + n] for r, (a, n) in act]).to(DEV)
        ww = torch.cat([data[r][1][a:a + n] for r, (a, n) in act]).to(DEV)
        ctx = step_ctx([n for _, (_, n) in act], [(1, 2)[r] for r, _ in act])
        o = torch.empty(x.shape[0], H, d, device=DEV)
        if step % 2:      # r, k, v as three products of their own (separate allocations) ...
            r_, k_, v_ = (x[:, i * A:(i + 1) * A].clone() for i in range(3))
        else:             # ... or as column blocks of one
            r_, k_, v_ = (x[:, i * A:(i + 1) * A] for i in range(3))
        ops.recurrent_scan(ops.SCAN_BONUS, r_, k_, v_, state, ctx, H, 1, d, d, o, ww=ww, w0=w0.to(DEV), u=u.to(DEV))
        at = 0
        for r, (a, n) in act:
            got[r][a:a + n] = o[at:at + n].cpu()
            at += n
    for r in range(2):
        assert float((got[r] - data[r][2]).abs().max()) <= 2e-5 * max(1.0, float(data[r][2].abs().max())), r


@pytest.mark.parametrize("G, H, dk, dv, K", [(1, 2, 8, 16, 4), (2, 4, 6, 5, 3), (1, 1, 4, 4, 1), (1, 1, 3, 2, 6)])
def test_convolution_with_its_tail_unit_vectors_and_gates(G, H, dk, dv, K):
    """Portions shorter than the convolution's reach, so that the tail is partly moved up and partly refilled."""
    from prism_b200 import ops
    g = torch.Generator().manual_seed(K)
    C = 2 * G * dk + H * dv
    n = 23
    proj = torch.randn(n, C + 2 * H + 3, generator=g)
    taps = torch.randn(C, K, generator=g) * 0.6
    a_log, dt = torch.randn(H, generator=g) * 0.5, torch.randn(H, generator=g)
    y = PP.silu(PP.causal_conv(proj[:, :C], taps))
    q = PP.unit(y[:, :G * dk].view(n, G, dk)) * dk ** -0.5
    k = PP.unit(y[:, G * dk:2 * G * dk].view(n, G, dk))
    ref = torch.cat([q.reshape(n, -1), k.reshape(n, -1), y[:, 2 * G * dk:]], 1)
    ref_b = torch.sigmoid(proj[:, C:C + H])
    ref_g = torch.exp(-torch.exp(a_log) * PP.softplus(proj[:, C + H:C + 2 * H] + dt))
    tail = torch.zeros(3, max(K - 1, 0), C, device=DEV)
    got, got_bg = torch.empty(n, C), torch.empty(n, 2 * H)
    pd = proj.to(DEV)
    for a, m in cut(n, (1, 2, 1, 1, 7, 3)):
        ctx = step_ctx([m], [1])
        qkv, bg = torch.empty(m, C, device=DEV), torch.empty(m, 2 * H, device=DEV)
        ops.conv_unit_gates(pd[a:a + m], C, C + H, taps.to(DEV), tail, a_log.to(DEV), dt.to(DEV), ctx, G, H, dk, dv, 1e-6, qkv, bg)
        ops.state_tail(pd[a:a + m], tail, ctx)
        got[a:a + m], got_bg[a:a + m] = qkv.cpu(), bg.cpu()
    assert float((got - ref).abs().max()) <= 1e-5
    assert float((got_bg - torch.cat([ref_b, ref_g], 1)).abs().max()) <= 1e-5
    if K > 1:
        assert float((tail[1].cpu() - proj[n - (K - 1):, :C]).abs().max()) == 0.0
        assert float(tail[0].abs().max()) == 0.0 and float(tail[2].abs().max()) == 0.0
    # token by token, the kernel moving the tail up itself (two requests side by side, the second one step behind)
    tail.zero_()
    got2 = torch.empty(n, C)
    for a in range(n + 1):
        rows = [r for r in (a, a - 1) if 0 <= r < n]
        ctx = step_ctx([1] * len(rows), [2 if r == a else 0 for r in rows])
        qkv, bg = torch.empty(len(rows), C, device=DEV), torch.empty(len(rows), 2 * H, device=DEV)
        ops.conv_unit_gates(pd[rows], C, C + H, taps.to(DEV), tail, a_log.to(DEV), dt.to(DEV), ctx, G, H, dk, dv, 1e-6, qkv, bg,
                            move_tail=True)
        if a < n:
            got2[a] = qkv[0].cpu()
        if a >= 1:
            assert float((qkv[-1].cpu() - ref[a - 1]).abs().max()) <= 1e-5
    assert float((got2 - ref).abs().max()) <= 1e-5


@pytest.mark.parametrize("T, R, N", [(1, 16, 64), (9, 5, 60), (70, 64, 300), (8, 1, 1), (3, 100, 130)])
def test_decay_from_the_low_rank_product(T, R, N):
    from prism_b200 import ops
    g = torch.Generator().manual_seed(T * R)
    low, w2, w0 = torch.randn(T, R + 3, generator=g), torch.randn(N, R, generator=g) / R ** 0.5, torch.randn(N, generator=g) - 1.0
    out = torch.empty(T, N, device=DEV)
    ops.lowrank_decay(low.to(DEV)[:, 3:], w2.t().contiguous().to(DEV), w0.to(DEV), out)
    ref = torch.exp(-torch.exp(torch.tanh(low[:, 3:]) @ w2.T + w0))
    assert float((out.cpu() - ref).abs().max()) <= 2e-6
    ww = (torch.tanh(low[:, 3:]) @ w2.T).to(DEV)
    ops.decay_from_exponent(ww, w0.to(DEV))
    assert float((ww.cpu() - ref).abs().max()) <= 2e-6


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_small_kernels(dtype):
    from prism_b200 import ops
    g = torch.Generator().manual_seed(1)
    tol = 1e-5 if dtype == torch.float32 else 2e-2
    # norm after the sum, with a stack of partial sums
    x, d, w = torch.randn(9, 52, generator=g), torch.randn(3, 9, 52, generator=g), torch.randn(52, generator=g) * 0.1 + 1
    xd, copy = x.to(DEV), torch.empty(9, 52, dtype=dtype, device=DEV)
    ops.scale_add_rmsnorm(xd, 2.5, d.to(DEV), w.to(DEV), 1e-5, copy)
    ref = PP.rms_norm(2.5 * x + d.sum(0), w, 1e-5)
    assert float((xd.cpu() - ref).abs().max()) <= 1e-5 and float((copy.float().cpu() - ref).abs().max()) <= tol
    xd = x.to(DEV)
    ops.scale_add_rmsnorm(xd, 1.0, None, w.to(DEV), 1e-5, None)
    assert float((xd.cpu() - PP.rms_norm(x, w, 1e-5)).abs().max()) <= 1e-5
    # gate on a column block of a wider buffer
    a, gate = torch.randn(7, 40, generator=g), torch.randn(7, 90, generator=g)
    out = torch.zeros(7, 64, dtype=dtype, device=DEV)
    ops.gated_product(a.to(dtype).to(DEV), gate.to(DEV)[:, 50:], out[:, 8:48], "sigmoid", 1.2)
    assert float((out[:, 8:48].float().cpu() - a.to(dtype).float() * torch.sigmoid(gate[:, 50:]) * 1.2).abs().max()) <= tol
    assert float(out[:, :8].abs().max()) == 0.0 and float(out[:, 48:].abs().max()) == 0.0
    # token-shift mixes: the first token of a step takes the request's previous input from its slot
    xs, mu = torch.randn(6, 20, generator=g), torch.rand(5, 20, generator=g)
    prev = torch.randn(3, 1, 20, generator=g)
    ctx = step_ctx([4, 2], [2, 0])
    mixes = torch.empty(5, 6, 20, dtype=dtype, device=DEV)
    pd = prev.to(DEV)
    ops.shift_mix(xs.to(DEV), pd, mu.to(DEV), ctx, mixes)
    before = torch.cat([prev[2], xs[:3], prev[0], xs[4:5]])
    ref = xs[None] + (before - xs)[None] * mu[:, None]
    assert float((mixes.float().cpu() - ref).abs().max()) <= tol
    ops.state_tail(xs.to(DEV), pd, ctx)
    assert torch.equal(pd[2, 0].cpu(), xs[3]) and torch.equal(pd[0, 0].cpu(), xs[5]) and torch.equal(pd[1].cpu(), prev[1])
    # single tokens: the mix kernel keeps each token as its request's previous one itself
    pd = prev.to(DEV)
    ctx1 = step_ctx([1, 1], [1, 0])
    m1 = torch.empty(5, 2, 20, dtype=dtype, device=DEV)
    ops.shift_mix(xs[:2].to(DEV), pd, mu.to(DEV), ctx1, m1, keep_prev=True)
    ref1 = xs[None, :2] + (torch.cat([prev[1], prev[0]]) - xs[:2])[None] * mu[:, None]
    assert float((m1.float().cpu() - ref1).abs().max()) <= tol
    assert torch.equal(pd[1, 0].cpu(), xs[0]) and torch.equal(pd[0, 0].cpu(), xs[1]) and torch.equal(pd[2].cpu(), prev[2])
    # head norm with one weight for all heads and with a weight per head, gate, constant
    o, gt = torch.randn(5, 3, 14, generator=g), torch.randn(5, 42, generator=g)
    for wt in (torch.randn(14, generator=g), torch.randn(42, generator=g)):
        out = torch.empty(5, 42, dtype=dtype, device=DEV)
        ops.headnorm_gate(o.to(DEV), gt.to(DEV), wt.to(DEV), 1e-5, 0.7, out)
        wfull = wt if wt.numel() == 42 else wt.repeat(3)
        ref = (PP.rms_norm(o, None, 1e-5).reshape(5, 42) * wfull * PP.silu(gt)) * 0.7
        assert float((out.float().cpu() - ref).abs().max()) <= tol * max(1.0, float(ref.abs().max()))


@pytest.mark.parametrize("T, A, R, K", [(8, 128, 16, 256), (1, 256, 40, 512), (16, 128, 128, 136), (5, 64, 8, 64), (70, 128, 8, 128),
                                        (4, 8, 64, 32), (3, 128, 200, 64)])
def test_projections_that_each_read_their_own_input_as_one_product(T, A, R, K):
    """Four blocks of A weight rows and one of R, each applied to its own [T, K] input: the grouped launch of the
    weight-streaming kernel (A a multiple of 128, up to 16 tokens) and the product-per-group path give the plain
    products."""
    from prism_b200 import ops
    g = torch.Generator().manual_seed(T + A)
    xs = torch.randn(5, T, K, generator=g).to(torch.bfloat16)
    w = (torch.randn(4 * A + R, K, generator=g) / K ** 0.5).to(torch.bfloat16)
    out = torch.cat(ops.linear_grouped(xs.to(DEV), w.to(DEV), (A, A, A, A, R), torch.float32), 1).cpu()
    ref = torch.cat([xs[i].float() @ w[i * A:(i * A + R if i == 4 else (i + 1) * A)].float().T for i in range(5)], 1)
    assert out.shape == (T, 4 * A + R)
    assert float((out - ref).abs().max()) <= 2e-3 * max(1.0, float(ref.abs().max()))
    xs32, w32 = xs.float().to(DEV), w.float().to(DEV)
    out32 = torch.cat(ops.linear_grouped(xs32, w32, (A, A, A, A, R), torch.float32), 1).cpu()
    assert float((out32 - ref).abs().max()) <= 1e-4 * max(1.0, float(ref.abs().max()))


# ---------------------------------------------------------------------------------------------------------
# the model through the engine's step function
# ---------------------------------------------------------------------------------------------------------

LIMIT = {"float32": 3e-5, "bfloat16": 4e-2}
ILL = {"float32": 0.0, "bfloat16": 0.05}        # see pofazen_helpers.compare
LENGTHS = {"P": [1, 9, 40, 71, 130], "Q": [2, 65, 128, 200, 333], "R": [1, 5, 33], "S": [3, 26, 61], "T": [1, 20, 70]}


def runner_for(folder, dtype, max_tokens, page_size, max_live=4):
    from prism_b200.engine.replay import build_runner
    return build_runner(folder, dtype, max_tokens, page_size, max_live)[3]


def sequences(name):
    vocab = CONFIGS[name][0]["vocab"]
    return {f"r{i}": random_tokens(vocab, n, 300 + i) for i, n in enumerate(LENGTHS[name])}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", sorted(CONFIGS))
@pytest.mark.parametrize("mode", ["whole", "tail", "portions", "small_portions", "mixed"])
def test_cutting(name, dtype, mode):
    """Whole prompts, a decoded tail, portions (one schedule of twos and threes only), and mixed batches of up
    to four live requests in a pool that holds no more than the schedule needs, so that pages and state slots
    come back and are used again."""
    seqs = sequences(name)
    steps = {"whole": trace_whole, "tail": lambda s: trace_tail(s, 48), "portions": trace_portions,
             "small_portions": lambda s: trace_portions(s, (2, 3, 2, 2, 5, 2)),
             "mixed": lambda s: trace_mixed(s, seed=3)}[mode](seqs)
    ps = CONFIGS[name][2]
    runner = runner_for(model_folder(name), dtype, trace_budget(steps, max(ps, 64)), ps)
    got = run_trace(runner, steps)
    assert len(got) == sum(len(s) for s in seqs.values())
    compare(name, seqs, got, LIMIT[dtype], ILL[dtype])
    assert runner.cache.pages_in_use() == 0 and len(runner.cache.requests) == 0


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding_across_windows_and_pages(dtype):
    seq = random_tokens(CONFIGS["Q"][0]["vocab"], 420, 9)
    runner = runner_for(model_folder("Q"), dtype, 448, 64)
    got = run_trace(runner, trace_tail({"a": seq}, 300))
    compare("Q", {"a": seq}, got, LIMIT[dtype], ILL[dtype])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_batches_of_unequal_requests_against_each_alone(dtype):
    seqs = sequences("P")
    ps = CONFIGS["P"][2]
    alone = run_trace(runner_for(model_folder("P"), dtype, 4096, ps), trace_portions(seqs, (5, 2, 9)))
    together = run_trace(runner_for(model_folder("P"), dtype, 4096, ps, max_live=5), trace_mixed(seqs, seed=11, max_live=5))
    tol = 2e-5 if dtype == "float32" else 8e-2
    for key, row in alone.items():
        assert float((row - together[key]).abs().max()) <= tol * max(1.0, float(row.abs().max())), key


def test_a_state_slot_that_is_used_again_starts_from_zero():
    """One slot only: the second request gets the slot the first one left, and must not inherit its state."""
    seqs = {"a": random_tokens(90, 40, 1), "b": random_tokens(90, 25, 2)}
    runner = runner_for(model_folder("T"), "float32", 64, 16, max_live=1)
    got = run_trace(runner, trace_portions(seqs, (7, 1, 3)))
    compare("T", seqs, got, LIMIT["float32"])


ONE_LAYER = {
    "parallel": [layer("parallel", parallel(left(4, 2, 16, 8, 9, 2, rot_dims=8, base=300.0, scaling=(2.0, 1.0, 2.0, 32)),
                                            right(2, 1, 16, 24, 4), 1.25, 0.85), None)],
    "attention_side_mostly": [layer("parallel", parallel(left(3, 1, 32, 32, 21, 5, scale=0.11), right(1, 1, 8, 8, 2), 1.5, 0.01), None)],
    "delta_side_mostly": [layer("parallel", parallel(left(1, 1, 8, 8, 4), right(4, 2, 24, 12, 5), 0.01, 1.5), None)],
    "wkv": [layer("wkv", wkv(3, 16, 6), None)],
    "feed_forward": [layer("wkv", wkv(1, 8, 2), 112)],
    "odd_sizes": [layer("parallel", parallel(left(2, 1, 7, 5, 6, 1, rot_dims=4), right(3, 3, 5, 3, 2)), 33)],
}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("which", sorted(ONE_LAYER))
def test_each_mixer_alone(which, dtype):
    odd = which == "odd_sizes"
    raw = model(51 if odd else 97, 37 if odd else 48, ONE_LAYER[which], alpha=1.5)
    w = draw_weights(raw, 21)
    folder = write_folder(raw, w)
    seq = random_tokens(raw["vocab"], 75, 4)
    ref = PP.forward(raw, {k: v.float() for k, v in w.items()}, seq)
    runner = runner_for(folder, dtype, 128, 16)
    got = run_trace(runner, trace_portions({"a": seq}, (20, 1, 1, 30, 2, 1)))
    scale = float((ref - ref.mean(-1, keepdim=True)).pow(2).mean().sqrt())
    errs = sorted(float((got[("a", p)] - ref[p] - (got[("a", p)] - ref[p]).mean()).pow(2).mean().sqrt()) / scale for p in range(75))
    assert errs[-1] <= LIMIT[dtype] * (8 if ILL[dtype] else 1) and errs[int(len(errs) * (1 - ILL[dtype])) - 1] <= LIMIT[dtype], errs[-4:]


def test_side_by_side_mixers_fused_and_each_on_its_own():
    """The sum of mixers as one joint input product and one joint output product against every mixer with its own
    projections, results added in float32: the same numbers up to rounding."""
    from prism_b200.model_registry import build_model
    from prism_b200.weights.loader import load_weights
    from prism_b200.engine.runner import ModelRunner
    from prism_b200.engine.batch import Segment
    raw = CONFIGS["P"][0]
    folder = model_folder("P")
    seq = random_tokens(raw["vocab"], 50, 8)
    outs = []
    for fuse in (True, False):
        cfg, mdl = build_model(raw, {k: tuple(v.shape) for k, v in draw_weights(raw, CONFIGS["P"][1]).items()})
        if not fuse:
            from prism_b200.models.pofazen import pofazen_spec
            from prism_b200.models.decoder import DecoderModel
            spec = pofazen_spec(cfg)
            for blk in spec.layers:
                if blk.args["mixer"].kind == "sum":
                    blk.args["mixer"].args["fuse"] = False
            mdl = DecoderModel(spec)
        load_weights(mdl, folder, DEV, torch.float32)
        runner = ModelRunner(mdl, DEV, torch.float32, 8, 16, 2, 128)
        runner.begin_request("a")
        outs.append(runner.step([Segment("a", seq, list(range(50)))]).cpu())
        runner.check_errors()
    assert float((outs[0] - outs[1]).abs().max()) <= 2e-4 * float(outs[1].abs().max())
    ref = PP.forward(raw, {k: v.float() for k, v in draw_weights(raw, CONFIGS["P"][1]).items()}, seq)
    assert float((outs[1] - ref).abs().max()) <= 2e-4 * float(ref.abs().max())


def test_greedy_generation_through_the_scheduler():
    """Engine.generate (scheduler, batching, sampling, CUDA graphs for the decode steps) picks the plain
    model's greedy tokens; more prompts than request slots, so that state slots are used again."""
    from prism_b200.config.engine_config import EngineConfig, SchedulerConfig
    from prism_b200.engine.llm import Engine
    from prism_b200.sampling.sampler import SamplingParams
    raw = CONFIGS["P"][0]
    w = {k: v.float() for k, v in draw_weights(raw, CONFIGS["P"][1]).items()}
    prompts = [random_tokens(raw["vocab"], n, 40 + n) for n in (3, 17, 30, 8, 1, 12)]
    n_new = 24
    # a folder as an exporter writes it: the decay's rank is in no key of config.json, the model file has it
    bare = dict(raw, layers=[dict(l, mixer={k: v for k, v in l["mixer"].items() if k != "decay_rank"}) for l in raw["layers"]])
    folder = write_folder(bare, draw_weights(raw, CONFIGS["P"][1]))
    for graphs in (False, True):
        eng = Engine(folder, EngineConfig(kv_page_size=8, num_pages=40, max_seq_len=128, use_cuda_graph=graphs,
                                                      graph_batch_sizes=(1, 2, 4, 8),
                                                      scheduler=SchedulerConfig(max_batch_tokens=48, max_num_seqs=4, prefill_chunk=16)),
                     dtype="float32")
        assert eng.runner.use_cuda_graph == graphs
        res = eng.generate(prompts, SamplingParams(max_new_tokens=n_new, ignore_eos=True))
        for p, r in zip(prompts, res):
            seq = list(p)
            for tok in r.token_ids:
                logits = PP.forward(raw, w, seq)[-1]
                top = torch.topk(logits, 2).values
                if float(top[0] - top[1]) > 1e-3:          # a near tie may fall either way
                    assert tok == int(logits.argmax()), (graphs, len(p), len(seq))
                seq.append(tok)
            assert len(r.token_ids) == n_new
        assert eng.cache.pages_in_use() == 0


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_the_replay_program_serves_the_design(tmp_path, dtype):
    """bin/trace_run as a user runs it, on a Pofazen folder: the model class is found by config.json, the decay's
    rank by the model file, the pool holds what --max-tokens says and there are four state slots."""
    import json
    import os
    import subprocess
    import sys
    import numpy as np
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    name = "P"
    raw = dict(CONFIGS[name][0])
    raw["layers"] = [dict(l, mixer={k: v for k, v in l["mixer"].items() if k != "decay_rank"}) for l in raw["layers"]]
    folder = write_folder(raw, draw_weights(CONFIGS[name][0], CONFIGS[name][1]))
    vocab = raw["vocab"]
    seqs = {f"q{i}": random_tokens(vocab, n, 500 + i) for i, n in enumerate([70, 33, 90, 12, 64, 5])}
    steps = trace_mixed(seqs, seed=17)
    out = tmp_path / "out"
    proc = subprocess.run([sys.executable, os.path.join(root, "bin", "trace_run"), "--model", folder, "--dtype", dtype,
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
    compare(name, seqs, got, LIMIT[dtype], ILL[dtype])

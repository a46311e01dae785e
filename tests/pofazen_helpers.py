"""Shared pieces of the Pofazen tests: small configurations that differ from one another in every size and
option, model folders with weights drawn here (larger than the framework's random-weights recipe, so that
attention is far from uniform, decays are neither 0 nor 1 and a wrong key or a lost state shows), and the
comparison with the plain implementation."""

from __future__ import annotations

import json
import math
import os
import sys
import tempfile

import torch

HERE = os.path.dirname(os.path.abspath(__file__))
if HERE not in sys.path:
    sys.path.insert(0, HERE)

from plain import pofazen_plain as PP  # noqa: E402


def left(heads, kv_heads, dim, vdim, window, keep_first=0, scale=None, rot_dims=None, base=10000.0, scaling=None):
    m = dict(heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim, scale=scale if scale is not None else dim ** -0.5)
    if window is not None:
        m["mask"] = dict(size=window, keep_first=keep_first)
    if rot_dims is None:
        rot_dims = dim // 2 * 2
    if rot_dims:
        m["rot"] = dict(base=base, dims=rot_dims)
        if scaling is not None:
            m["rot"]["scaling"] = dict(zip(("factor", "low", "high", "original"), scaling))
    return m


def right(heads, kv_heads, dim, vdim, conv):
    return dict(heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim, conv=conv)


def parallel(l, r, left_scale=1.0, right_scale=1.0):
    return dict(left=l, right=r, left_scale=left_scale, right_scale=right_scale)


def wkv(heads, dim, rank):
    return dict(heads=heads, dim=dim, decay_rank=rank)


def layer(kind, mixer, ff):
    return dict(type=kind, mixer=mixer, mlp=None if ff is None else dict(kind="dense", ff=ff))


def model(vocab, width, layers, eps=1e-6, alpha=2.0):
    return dict(architecture="Pofazen", vocab=vocab, width=width, norm=dict(eps=eps), postln_alpha=alpha, layers=layers)


# P: three query heads per kv head, values larger than keys, a window that is no multiple of anything and keeps
# three tokens, part of a head rotated with rescaled frequencies in all three bands, two value heads per q/k head
# in the delta rule, a convolution of three taps, wkv heads that do not fill the width, a layer without feed-forward
CONFIG_P = model(211, 72, eps=1e-5, alpha=2.5, layers=[
    layer("parallel", parallel(left(6, 2, 16, 24, 13, 3, scale=0.3, rot_dims=8, base=50.0, scaling=(4.0, 1.0, 3.0, 64)),
                               right(4, 2, 12, 20, 3), 1.3, 0.8), 96),
    layer("wkv", wkv(3, 20, 5), 80),
    layer("wkv", wkv(2, 24, 7), None),
    layer("parallel", parallel(left(3, 3, 8, 8, 5, 7, rot_dims=8, base=1000.0), right(2, 2, 8, 16, 2), 0.7, 1.1), 64),
])
# Q: sizes the tensor-core kernels take (multiples of 16), pages of 64, a window larger than a page, more kept
# tokens than a tile's worth of a few, one kv head; heads and sizes of the two sides differ everywhere
CONFIG_Q = model(300, 128, alpha=2.2, layers=[
    layer("wkv", wkv(4, 32, 16), 160),
    layer("parallel", parallel(left(4, 1, 32, 64, 70, 5, scale=0.25, rot_dims=16, base=30000.0, scaling=(8.0, 1.0, 4.0, 128)),
                               right(2, 1, 64, 32, 4), 1.4, 0.9), 192),
    layer("parallel", parallel(left(2, 2, 64, 16, 100, 40, rot_dims=64), right(4, 4, 16, 16, 4), 1.0, 1.0), 96),
    layer("wkv", wkv(8, 16, 4), 128),
])
# R: everything 1 that can be: one head everywhere, a window of one position, one kept token, a convolution of
# one tap (no tail), rank 1, no rotation in one layer and no mask in another
CONFIG_R = model(64, 32, alpha=1.0, layers=[
    layer("parallel", parallel(left(1, 1, 8, 8, 1, 1, rot_dims=0), right(1, 1, 4, 4, 1), 1.0, 1.0), 32),
    layer("wkv", wkv(1, 8, 1), 32),
    layer("parallel", parallel(left(1, 1, 8, 8, None, rot_dims=2), right(1, 1, 1, 1, 2), 2.0, 0.5), 32),
])
# S: sizes that are multiples of nothing (no 16-byte piece anywhere): every kernel's scalar path, and the library
# products on unaligned rows; recurrent layers only at the start, so that a model without pages is covered by T
CONFIG_S = model(77, 52, alpha=1.7, layers=[
    layer("parallel", parallel(left(3, 3, 10, 14, 9, 2, rot_dims=6, base=100.0), right(3, 1, 7, 5, 3), 0.9, 1.4), 44),
    layer("wkv", wkv(3, 11, 3), 30),
])
# T: recurrent layers only: the model has no paged cache group at all
CONFIG_T = model(90, 48, alpha=2.0, layers=[layer("wkv", wkv(3, 16, 8), 64), layer("wkv", wkv(6, 8, 2), None)])
CONFIGS = {"P": (CONFIG_P, 11, 8), "Q": (CONFIG_Q, 12, 64), "R": (CONFIG_R, 13, 16), "S": (CONFIG_S, 14, 8),
           "T": (CONFIG_T, 15, 16)}      # config, seed, page size


def draw_weights(raw: dict, seed: int) -> dict:
    """bf16 tensors keyed by the model file's names.  Matrices ``normal(0, 1 / sqrt(in))`` times a gain, so that
    activations stay of order one through the layers, attention scores spread over several units, decays lie
    well inside (0, 1) and the gates are neither shut nor open."""
    g = torch.Generator().manual_seed(seed)
    W = raw["width"]

    def mat(o, i, gain=1.0):
        return torch.randn(o, i, generator=g) * (gain / math.sqrt(i))

    def vec(n, std, mean=0.0):
        return torch.randn(n, generator=g) * std + mean

    t = {"embed": torch.randn(raw["vocab"], W, generator=g) * 0.5, "embed.norm": vec(W, 0.1, 1.0),
         "final.norm": vec(W, 0.1, 1.0), "head": mat(raw["vocab"], W)}
    for i, lr in enumerate(raw["layers"]):
        p, m = f"l{i}.", lr["mixer"]
        t[p + "norm1"] = vec(W, 0.1, 1.0)
        if lr["type"] == "parallel":
            l, r = m["left"], m["right"]
            q = p + "mix.left."
            H, G, d, dv = l["heads"], l["kv_heads"], l["dim"], l["vdim"]
            t[q + "q"], t[q + "k"], t[q + "v"] = mat(H * d, W, 2.0), mat(G * d, W, 2.0), mat(G * dv, W)
            t[q + "q.norm"], t[q + "k.norm"] = vec(d, 0.3, 2.0), vec(d, 0.3, 2.0)
            t[q + "g"], t[q + "o"] = mat(H * dv, W, 2.0), mat(W, H * dv, 0.7)
            q = p + "mix.right."
            H, G, d, dv, K = r["heads"], r["kv_heads"], r["dim"], r["vdim"], r["conv"]
            t[q + "q"], t[q + "k"], t[q + "v"] = mat(G * d, W, 2.0), mat(G * d, W, 2.0), mat(H * dv, W, 1.5)
            t[q + "q.conv"], t[q + "k.conv"], t[q + "v.conv"] = (torch.randn(G * d, K, generator=g) * 0.6,
                                                                torch.randn(G * d, K, generator=g) * 0.6,
                                                                torch.randn(H * dv, K, generator=g) * 0.6)
            t[q + "b"], t[q + "a"] = mat(H, W, 2.0), mat(H, W, 1.5)
            t[q + "A_log"], t[q + "dt_bias"] = vec(H, 0.5, -0.5), vec(H, 0.7)
            t[q + "norm"], t[q + "g"], t[q + "o"] = vec(dv, 0.1, 1.0), mat(H * dv, W, 2.0), mat(W, H * dv, 0.7)
        else:
            q = p + "mix."
            H, d, R = m["heads"], m["dim"], m["decay_rank"]
            A = H * d
            for s_ in "rkvgw":
                t[q + "mu." + s_] = torch.rand(W, generator=g)
            t[q + "r"], t[q + "k"], t[q + "v"], t[q + "g"] = mat(A, W, 1.5), mat(A, W, 1.5), mat(A, W, 1.5), mat(A, W, 2.0)
            t[q + "w1"], t[q + "w2"], t[q + "w0"] = mat(R, W, 2.0), mat(A, R, 1.5), vec(A, 0.8, -1.0)
            t[q + "u"] = torch.randn(H, d, generator=g) * 0.5
            t[q + "norm"], t[q + "o"] = vec(A, 0.1, 1.0), mat(W, A, 0.7)
        if lr.get("mlp") is not None:
            F = lr["mlp"]["ff"]
            t[p + "norm2"] = vec(W, 0.1, 1.0)
            t[p + "mlp.gate"], t[p + "mlp.up"], t[p + "mlp.down"] = mat(F, W, 1.5), mat(F, W), mat(W, F, 0.7)
    return {k: v.to(torch.bfloat16).contiguous() for k, v in t.items()}


_folders = {}


def write_folder(raw: dict, weights: dict, d: str = None) -> str:
    from safetensors.torch import save_file
    d = d or tempfile.mkdtemp(prefix="prism_pofazen_")
    with open(os.path.join(d, "config.json"), "w") as f:
        json.dump(raw, f)
    save_file(weights, os.path.join(d, "model.safetensors"))
    return d


def model_folder(name: str) -> str:
    if name not in _folders:
        raw, seed, _ = CONFIGS[name]
        _folders[name] = write_folder(raw, draw_weights(raw, seed))
    return _folders[name]


_plain = {}


def plain_weights(name: str):
    if name not in _plain:
        raw, seed, _ = CONFIGS[name]
        _plain[name] = {k: v.float() for k, v in draw_weights(raw, seed).items()}
    return _plain[name]


_logits = {}


def plain_logits(name: str, seq) -> torch.Tensor:
    key = (name, tuple(seq))
    if key not in _logits:
        _logits[key] = PP.forward(CONFIGS[name][0], plain_weights(name), list(seq))
    return _logits[key]


def row_error(got: torch.Tensor, ref: torch.Tensor, scale: float) -> float:
    """Root mean square over the vocabulary of the difference with its mean taken off, over ``scale``."""
    d = got.double() - ref.double()
    d = d - d.mean()
    return float(torch.sqrt((d * d).mean())) / scale


def compare(name: str, seqs: dict, got: dict, limit: float, ill: float = 0.0):
    """Every row the trace produced against the plain model on the whole sequence; the error of a row is
    ``row_error`` with the root mean square of the sequence's centred logits as scale.  ``ill``: the share of
    rows that may lie over ``limit``, up to eight times.  (In bfloat16 only: a head's read-out is divided by
    its root mean square, so where it is close to zero - the first token of a sequence, whose read-out is its
    value times one dot product - rounding decides its sign.  A wrong key or a lost state moves most rows that
    follow it, and moves them in float32 too, where no row may differ.)"""
    errs = []
    for rid, seq in seqs.items():
        ref = plain_logits(name, seq)
        scale = float((ref - ref.mean(-1, keepdim=True)).pow(2).mean().sqrt())
        for pos in range(len(seq)):
            if (rid, pos) in got:
                e = row_error(got[(rid, pos)], ref[pos], scale)
                errs.append((e if e == e else math.inf, rid, pos))
    errs.sort(reverse=True)
    over = [x for x in errs if not x[0] <= limit]
    assert len(over) <= ill * len(errs) and (not over or over[0][0] <= 8 * limit), \
        f"{len(over)} of {len(errs)} rows over {limit:.1e}; worst {over[0][0]:.3e} at {over[0][1:]}"
    return errs[0] if errs else None

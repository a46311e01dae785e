"""Shared pieces of the Dolezen tests: small configurations that differ from one another in every size and
option, model folders with weights drawn here (larger than the framework's random-weights recipe, so that
attention is far from uniform and a wrong key shows), and the comparison with the plain implementation."""

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

from plain import dolezen_plain as DP  # noqa: E402


def attn(heads, kv_heads, dim, vdim, mask, scale=None, kv_from=None):
    m = dict(heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim, scale=scale if scale is not None else dim ** -0.5)
    if mask is not None:
        m["mask"] = dict(size=mask)
    if kv_from is not None:
        m["kv_from"] = kv_from
    return m


def latent(heads, dim, rot_dim, vdim, q_rank, kv_rank, window, base=10000.0, dims=None, scale=None):
    m = dict(heads=heads, dim=dim, rot_dim=rot_dim, vdim=vdim, q_rank=q_rank, kv_rank=kv_rank,
             rot=dict(base=base, dims=rot_dim if dims is None else dims),
             scale=scale if scale is not None else (dim + rot_dim) ** -0.5)
    if window is not None:
        m["mask"] = dict(size=window)
    return m


def layer(kind, mixer, ff):
    return dict(type=kind, mixer=mixer, mlp=None if ff is None else dict(kind="dense", ff=ff))


# X: grouped heads (3 query heads per kv head), values larger than keys, two readers of one plane with masks
# that differ from the owner's, a layer without feed-forward, a window that is no multiple of anything
CONFIG_X = dict(architecture="Dolezen", vocab=211, width=72, norm=dict(eps=1e-5), embedding=dict(scale=3.5), layers=[
    layer("latent_attention", latent(3, 16, 8, 24, 40, 32, 11, base=500.0), 96),
    layer("attention", attn(6, 2, 16, 24, 13), 80),
    layer("attention", attn(6, 2, 16, 24, 7, kv_from=1), None),
    layer("attention", attn(6, 2, 16, 24, 13, scale=0.3, kv_from=1), 64),
    layer("latent_attention", latent(5, 8, 16, 8, 24, 48, 5, dims=8), 88),
])
# Y: one kv head, sizes the tensor-core kernels take (multiples of 16), equal key and value sizes, pages of 64,
# masks larger than a page, an unmasked layer of each kind
CONFIG_Y = dict(architecture="Dolezen", vocab=300, width=128, norm=dict(eps=1e-6), embedding=dict(scale=1.0), layers=[
    layer("attention", attn(4, 1, 32, 32, 70), 160),
    layer("attention", attn(4, 1, 32, 32, 70, kv_from=0), 160),
    layer("latent_attention", latent(4, 32, 16, 32, 48, 64, 90), 192),
    layer("attention", attn(2, 2, 64, 16, None), 96),
    layer("latent_attention", latent(20, 16, 0, 16, 32, 96, None), 64),
])
# Z: everything 1 that can be: one head, a window and a chunk of one position, rank 8
CONFIG_Z = dict(architecture="Dolezen", vocab=64, width=32, norm=dict(eps=1e-6), embedding=dict(scale=0.5), layers=[
    layer("attention", attn(1, 1, 8, 8, 1), 32),
    layer("latent_attention", latent(1, 8, 8, 8, 8, 8, 1), 32),
    layer("attention", attn(1, 1, 8, 8, 3, kv_from=0), 32),
])
# W: sizes that are multiples of nothing (no 16-byte piece anywhere): every kernel's scalar path, and the library
# products on unaligned rows
CONFIG_W = dict(architecture="Dolezen", vocab=77, width=52, norm=dict(eps=1e-6), embedding=dict(scale=1.7), layers=[
    layer("attention", attn(3, 3, 12, 20, 10), 44),
    layer("latent_attention", latent(3, 10, 6, 14, 10, 20, 9, dims=6), 44),
    layer("attention", attn(3, 3, 12, 20, 10, kv_from=0), 30),
    layer("latent_attention", latent(2, 6, 2, 5, 7, 9, None, dims=2), None),
])
CONFIGS = {"X": (CONFIG_X, 11, 8), "Y": (CONFIG_Y, 12, 64), "Z": (CONFIG_Z, 13, 16), "W": (CONFIG_W, 14, 8)}      # config, seed, page size


def draw_weights(raw: dict, seed: int) -> dict:
    """bf16 tensors keyed by the model file's names.  Matrices ``normal(0, 1 / sqrt(in))`` times a gain, so
    that activations stay of order one through the layers and attention scores spread over several units."""
    g = torch.Generator().manual_seed(seed)
    W = raw["width"]

    def mat(o, i, gain=1.0):
        return torch.randn(o, i, generator=g) * (gain / math.sqrt(i))

    def vec(n, std, mean=0.0):
        return torch.randn(n, generator=g) * std + mean

    t = {"embed": torch.randn(raw["vocab"], W, generator=g) * 0.5, "final.norm": vec(W, 0.1, 1.0), "head": mat(raw["vocab"], W)}
    for i, lr in enumerate(raw["layers"]):
        p, m = f"l{i}.", lr["mixer"]
        t[p + "norm1"] = vec(W, 0.1, 1.0)
        if lr["type"] == "attention":
            H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
            t[p + "mix.q"], t[p + "mix.q.b"] = mat(H * d, W, 2.0), vec(H * d, 0.3)
            if m.get("kv_from") is None:
                t[p + "mix.k"], t[p + "mix.k.b"] = mat(G * d, W, 2.0), vec(G * d, 0.3)
                t[p + "mix.v"], t[p + "mix.v.b"] = mat(G * dv, W), vec(G * dv, 0.1)
            t[p + "mix.sink"] = vec(H, 1.5)
            t[p + "mix.o"], t[p + "mix.o.b"] = mat(W, H * dv, 0.5), vec(W, 0.1)
        else:
            H, d, r, dv, qr, R = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["q_rank"], m["kv_rank"]
            t[p + "mix.dq"], t[p + "mix.dq.norm"] = mat(qr, W), vec(qr, 0.1, 1.0)
            t[p + "mix.uq"] = mat(H * (d + r), qr, 2.0)
            t[p + "mix.dkv"], t[p + "mix.dkv.norm"] = mat(R + r, W, 1.5), vec(R, 0.1, 1.0)
            t[p + "mix.uk"], t[p + "mix.uv"] = mat(H * d, R, 2.0), mat(H * dv, R)
            t[p + "mix.o"] = mat(W, H * dv, 0.5)
        if lr.get("mlp") is not None:
            t[p + "mlp.up"], t[p + "mlp.down"] = mat(lr["mlp"]["ff"], W), mat(W, lr["mlp"]["ff"], 0.5)
    return {k: v.to(torch.bfloat16).contiguous() for k, v in t.items()}


_folders = {}


def write_folder(raw: dict, weights: dict, d: str = None) -> str:
    from safetensors.torch import save_file
    d = d or tempfile.mkdtemp(prefix="prism_dolezen_")
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
        _logits[key] = DP.forward(CONFIGS[name][0], plain_weights(name), list(seq))[0]
    return _logits[key]


def row_error(got: torch.Tensor, ref: torch.Tensor, scale: float) -> float:
    """Root mean square over the vocabulary of the difference with its mean taken off, over ``scale``."""
    d = got.double() - ref.double()
    d = d - d.mean()
    return float(torch.sqrt((d * d).mean())) / scale


def compare(name: str, seqs: dict, got: dict, limit: float):
    """Every row the trace produced against the plain model on the whole sequence; the error of a row is
    ``row_error`` with the root mean square of the sequence's centred logits as scale."""
    worst, where = 0.0, None
    for rid, seq in seqs.items():
        ref = plain_logits(name, seq)
        scale = float((ref - ref.mean(-1, keepdim=True)).pow(2).mean().sqrt())
        for pos in range(len(seq)):
            if (rid, pos) not in got:
                continue
            e = row_error(got[(rid, pos)], ref[pos], scale)
            if e > worst:
                worst, where = e, (rid, pos)
    assert worst <= limit, f"worst row error {worst:.3e} at {where} > {limit:.1e}"
    return worst, where

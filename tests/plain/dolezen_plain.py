"""Plain, slow float32 implementation of the Dolezen decoder, one function per
mechanism, for whole sequences on the CPU.  It shares no code with
``prism_b200``: weights come in as a dict of float32 tensors keyed by the
model file's tensor names, the configuration as the raw ``config.json`` dict.

Notation: ``x [T, D]`` is one sequence, positions are ``0 .. T-1``.
"""

from __future__ import annotations

import math

import torch


# ---- norms and activations --------------------------------------------------

def rms_norm(x, weight, eps):
    """``x / sqrt(mean(x^2) + eps) * weight`` over the last axis."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps) * weight


def relu_squared(z):
    r = torch.clamp(z, min=0.0)
    return r * r


# ---- positions ----------------------------------------------------------------

def rotate(x, positions, base, dims):
    """Rotary encoding of the first ``dims`` entries of the last axis of
    ``x [T, ..., d]``: entry i is paired with entry i + dims/2, the pair (u, v)
    at position p becomes (u cos a - v sin a, v cos a + u sin a), a = p *
    base^(-2i/dims).  The other entries are returned as they are."""
    half = dims // 2
    i = torch.arange(half, dtype=torch.float64)
    freq = base ** (-2.0 * i / dims)
    ang = positions.to(torch.float64)[:, None] * freq[None, :]          # [T, half]
    shape = [x.shape[0]] + [1] * (x.dim() - 2) + [half]
    c, s = torch.cos(ang).to(x.dtype).view(shape), torch.sin(ang).to(x.dtype).view(shape)
    u, v = x[..., :half], x[..., half:dims]
    return torch.cat([u * c - v * s, v * c + u * s, x[..., dims:]], dim=-1)


# ---- masks ----------------------------------------------------------------------

def sliding_mask(T, size):
    """``[T, T]`` bool: query i sees key j iff 0 <= i - j < size."""
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    return (i - j >= 0) & (i - j < size)


def chunk_mask(T, size):
    """Query i sees key j iff j <= i and both lie in the same block of
    ``size`` positions counted from 0."""
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    return (j <= i) & (i // size == j // size)


def layer_mask(T, mx, kind):
    """The mask of a mixer: ``kind`` ('sliding' or 'chunk') with the size the configuration gives; a mixer
    without a mask sees every earlier key."""
    size = (mx.get("mask") or {}).get("size")
    if size is None:
        return chunk_mask(T, max(T, 1))
    return sliding_mask(T, size) if kind == "sliding" else chunk_mask(T, size)


# ---- softmax ----------------------------------------------------------------------

def masked_softmax(scores, mask, sink=None):
    """Softmax over the visible keys of ``scores [H, T, T]``.  ``sink [H]``:
    one more term exp(sink_h) in the denominator of head h, with no value."""
    s = scores.masked_fill(~mask[None], -math.inf)
    m = s.max(-1, keepdim=True).values
    if sink is not None:
        m = torch.maximum(m, sink.view(-1, 1, 1))
    e = torch.exp(s - m)
    den = e.sum(-1, keepdim=True)
    if sink is not None:
        den = den + torch.exp(sink.view(-1, 1, 1) - m)
    return e / den


# ---- mixers -------------------------------------------------------------------------

def sink_attention_kv(h, w, pre, mx):
    """Keys ``[T, G, dim]`` and values ``[T, G, vdim]`` of a chunked attention layer."""
    T = h.shape[0]
    G, d, dv = mx["kv_heads"], mx["dim"], mx["vdim"]
    k = (h @ w[pre + "k"].T + w[pre + "k.b"]).view(T, G, d)
    v = (h @ w[pre + "v"].T + w[pre + "v.b"]).view(T, G, dv)
    return k, v


def sink_attention(h, w, pre, mx, kv):
    """Grouped-query attention with biases, no positions, a chunked mask and a
    sink in the softmax.  ``kv``: keys and values (this layer's or another's)."""
    T = h.shape[0]
    H, G, d, dv = mx["heads"], mx["kv_heads"], mx["dim"], mx["vdim"]
    q = (h @ w[pre + "q"].T + w[pre + "q.b"]).view(T, H, d)
    k, v = kv
    rep = H // G
    kk = k.repeat_interleave(rep, dim=1)                      # query head a uses kv head a // rep
    vv = v.repeat_interleave(rep, dim=1)
    scores = torch.einsum("iad,jad->aij", q, kk) * mx["scale"]
    p = masked_softmax(scores, layer_mask(T, mx, "chunk"), w[pre + "sink"])
    o = torch.einsum("aij,jad->iad", p, vv).reshape(T, H * dv)
    return o @ w[pre + "o"].T + w[pre + "o.b"]


def latent_attention(h, w, pre, mx, eps):
    """Attention through low-rank latents with a shared rotated key part and a
    sliding window."""
    T = h.shape[0]
    H, d, r, dv, R = mx["heads"], mx["dim"], mx["rot_dim"], mx["vdim"], mx["kv_rank"]
    pos = torch.arange(T)
    cq = rms_norm(h @ w[pre + "dq"].T, w[pre + "dq.norm"], eps)
    q = (cq @ w[pre + "uq"].T).view(T, H, d + r)
    q_plain, q_rot = q[..., :d], rotate(q[..., d:], pos, mx["rot"]["base"], mx["rot"]["dims"])
    dkv = h @ w[pre + "dkv"].T
    c = rms_norm(dkv[:, :R], w[pre + "dkv.norm"], eps)
    k_rot = rotate(dkv[:, R:], pos, mx["rot"]["base"], mx["rot"]["dims"])      # [T, r], one for all heads
    k_plain = (c @ w[pre + "uk"].T).view(T, H, d)
    v = (c @ w[pre + "uv"].T).view(T, H, dv)
    scores = (torch.einsum("iad,jad->aij", q_plain, k_plain) +
              torch.einsum("iad,jd->aij", q_rot, k_rot)) * mx["scale"]
    p = masked_softmax(scores, layer_mask(T, mx, "sliding"))
    o = torch.einsum("aij,jad->iad", p, v).reshape(T, H * dv)
    return o @ w[pre + "o"].T


# ---- feed-forward -------------------------------------------------------------------

def dense_ff(h, w, pre):
    return relu_squared(h @ w[pre + "up"].T) @ w[pre + "down"].T


# ---- the model ------------------------------------------------------------------------

def forward(cfg, w, tokens):
    """``(logits [T, V], residual stream after every layer [L, T, D])``."""
    eps = cfg["norm"]["eps"]
    tokens = torch.as_tensor(tokens, dtype=torch.long)
    x = w["embed"][tokens] * cfg["embedding"]["scale"]
    kept = {}                                  # layer -> its keys and values
    after = []
    for i, layer in enumerate(cfg["layers"]):
        pre, mx = f"l{i}.mix.", layer["mixer"]
        h = rms_norm(x, w[f"l{i}.norm1"], eps)
        if layer["type"] == "attention":
            if "kv_from" in mx and mx["kv_from"] is not None:
                kv = kept[mx["kv_from"]]
            else:
                kv = kept[i] = sink_attention_kv(h, w, pre, mx)
            delta = sink_attention(h, w, pre, mx, kv)
        elif layer["type"] == "latent_attention":
            delta = latent_attention(h, w, pre, mx, eps)
        else:
            raise ValueError(layer["type"])
        if layer.get("mlp") is not None:
            delta = delta + dense_ff(h, w, f"l{i}.mlp.")
        x = x + delta
        after.append(x)
    logits = rms_norm(x, w["final.norm"], eps) @ w["head"].T
    return logits, torch.stack(after)

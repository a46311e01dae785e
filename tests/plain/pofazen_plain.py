"""Plain, slow implementation of the Pofazen decoder, one function per
mechanism, for whole sequences on the CPU.  It shares no code with
``prism_b200``: weights come in as a dict of tensors keyed by the model file's
tensor names, the configuration as the raw ``config.json`` dict.  Everything
runs in the dtype of the weights handed in (float32 or float64).

Notation: ``x [T, D]`` is one sequence, positions are ``0 .. T-1``; ``W`` are
stored ``[out, in]`` and applied as ``x @ W.T``.
"""

from __future__ import annotations

import math

import torch


# ---- norms and activations --------------------------------------------------

def rms_norm(x, weight, eps):
    """``x / sqrt(mean(x^2) + eps) * weight`` over the last axis (``weight`` None: no weight)."""
    y = x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)
    return y if weight is None else y * weight


def unit(x, eps=1e-6):
    """``x / sqrt(sum(x^2) + eps)`` over the last axis."""
    return x / torch.sqrt((x * x).sum(-1, keepdim=True) + eps)


def silu(z):
    return z * torch.sigmoid(z)


def softplus(z):
    return torch.where(z > 30, z, torch.log1p(torch.exp(torch.clamp(z, max=30))))


# ---- positions ----------------------------------------------------------------

def scaled_frequencies(base, dims, scaling, dtype):
    """``f_i = base^(-2i/dims)`` for i < dims/2, then the three-band rule: with wavelength ``l = 2 pi / f``
    a frequency stays as it is where ``l < original / high``, is divided by ``factor`` where ``l > original
    / low``, and in between is ``(1 - s) f / factor + s f`` with ``s = (original / l - low) / (high - low)``."""
    i = torch.arange(dims // 2, dtype=dtype)
    f = base ** (-2.0 * i / dims)
    if not scaling:
        return f
    factor, low, high, orig = (float(scaling[k]) for k in ("factor", "low", "high", "original"))
    out = f.clone()
    for n in range(f.numel()):
        l = 2.0 * math.pi / float(f[n])
        if l < orig / high:
            continue
        if l > orig / low:
            out[n] = f[n] / factor
        else:
            s = (orig / l - low) / (high - low)
            out[n] = (1.0 - s) * f[n] / factor + s * f[n]
    return out


def rotate_interleaved(x, positions, freqs):
    """Entries ``2i`` and ``2i + 1`` of the last axis of ``x [T, heads, d]`` form pair i (i < len(freqs));
    the pair (u, v) at position p becomes (u cos a - v sin a, v cos a + u sin a), a = p f_i.  Entries from
    ``2 len(freqs)`` on pass unchanged."""
    n = freqs.numel()
    ang = positions.to(freqs.dtype)[:, None] * freqs[None, :]
    c, s = torch.cos(ang).to(x.dtype)[:, None, :], torch.sin(ang).to(x.dtype)[:, None, :]
    u, v = x[..., 0:2 * n:2], x[..., 1:2 * n:2]
    out = x.clone()
    out[..., 0:2 * n:2] = u * c - v * s
    out[..., 1:2 * n:2] = v * c + u * s
    return out


# ---- the left mixer: attention under a window that keeps the first tokens -------

def window_keep_mask(T, size, keep_first):
    """``[T, T]`` bool: query i sees key j iff j <= i and (i - j < size or j < keep_first)."""
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    return (j <= i) & ((i - j < size) | (j < keep_first))


def gated_window_attention(h, w, p, mx, eps):
    """``w``: the weights, ``p``: the prefix of this mixer's tensors, ``mx``: its configuration."""
    T = h.shape[0]
    H, G, d, dv = mx["heads"], mx["kv_heads"], mx["dim"], mx["vdim"]
    q = (h @ w[p + "q"].T).view(T, H, d)
    k = (h @ w[p + "k"].T).view(T, G, d)
    v = (h @ w[p + "v"].T).view(T, G, dv)
    q = rms_norm(q, w[p + "q.norm"], eps)
    k = rms_norm(k, w[p + "k.norm"], eps)
    rot = mx.get("rot")
    if rot and rot.get("dims"):
        f = scaled_frequencies(float(rot["base"]), int(rot["dims"]), rot.get("scaling"), h.dtype)
        pos = torch.arange(T)
        q, k = rotate_interleaved(q, pos, f), rotate_interleaved(k, pos, f)
    mask = mx.get("mask") or {}
    vis = window_keep_mask(T, int(mask.get("size", T + 1)), int(mask.get("keep_first", 0)))
    out = torch.empty(T, H, dv, dtype=h.dtype)
    for hh in range(H):
        g = hh // (H // G)
        s = (q[:, hh] @ k[:, g].T) * float(mx["scale"])
        s = s.masked_fill(~vis, -math.inf)
        out[:, hh] = torch.softmax(s, dim=-1) @ v[:, g]
    gate = torch.sigmoid(h @ w[p + "g"].T)
    return (out.reshape(T, H * dv) * gate) @ w[p + "o"].T


# ---- the right mixer: gated delta rule ----------------------------------------------

def causal_conv(x, taps):
    """``y[t, c] = sum_j taps[c, j] x[t - (K - 1) + j, c]`` with zeros before the start (the last column is
    the current token's)."""
    T, C = x.shape
    K = taps.shape[1]
    xp = torch.cat([torch.zeros(K - 1, C, dtype=x.dtype), x], 0)
    y = torch.zeros_like(x)
    for j in range(K):
        y = y + xp[j:j + T] * taps[:, j]
    return y


def gated_delta(h, w, p, mx, eps):
    T = h.shape[0]
    H, G, d, dv = mx["heads"], mx["kv_heads"], mx["dim"], mx["vdim"]
    q = silu(causal_conv(h @ w[p + "q"].T, w[p + "q.conv"])).view(T, G, d)
    k = silu(causal_conv(h @ w[p + "k"].T, w[p + "k.conv"])).view(T, G, d)
    v = silu(causal_conv(h @ w[p + "v"].T, w[p + "v.conv"])).view(T, H, dv)
    q = unit(q) * d ** -0.5
    k = unit(k)
    beta = torch.sigmoid(h @ w[p + "b"].T)                                        # [T, H]
    decay = torch.exp(-torch.exp(w[p + "A_log"]) * softplus(h @ w[p + "a"].T + w[p + "dt_bias"]))   # [T, H]
    out = torch.empty(T, H, dv, dtype=h.dtype)
    for hh in range(H):
        g = hh // (H // G)
        S = torch.zeros(d, dv, dtype=h.dtype)
        for t in range(T):
            S = decay[t, hh] * S
            u = beta[t, hh] * (v[t, hh] - S.T @ k[t, g])
            S = S + torch.outer(k[t, g], u)
            out[t, hh] = S.T @ q[t, g]
    out = rms_norm(out, w[p + "norm"], eps) * silu(h @ w[p + "g"].T).view(T, H, dv)
    return out.reshape(T, H * dv) @ w[p + "o"].T


def parallel_mixer(h, w, p, mx, eps):
    return (float(mx["left_scale"]) * gated_window_attention(h, w, p + "left.", mx["left"], eps)
            + float(mx["right_scale"]) * gated_delta(h, w, p + "right.", mx["right"], eps))


# ---- the wkv mixer ---------------------------------------------------------------------

def wkv(h, w, p, mx, eps):
    T, D = h.shape
    H, d = mx["heads"], mx["dim"]
    prev = torch.cat([torch.zeros(1, D, dtype=h.dtype), h[:-1]], 0)
    mix = lambda s: h + (prev - h) * w[p + "mu." + s]
    r = (mix("r") @ w[p + "r"].T).view(T, H, d)
    k = (mix("k") @ w[p + "k"].T).view(T, H, d)
    v = (mix("v") @ w[p + "v"].T).view(T, H, d)
    gate = silu(mix("g") @ w[p + "g"].T)
    decay = torch.exp(-torch.exp(torch.tanh(mix("w") @ w[p + "w1"].T) @ w[p + "w2"].T + w[p + "w0"])).view(T, H, d)
    u = w[p + "u"]
    out = torch.empty(T, H, d, dtype=h.dtype)
    for hh in range(H):
        S = torch.zeros(d, d, dtype=h.dtype)
        for t in range(T):
            kv = torch.outer(k[t, hh], v[t, hh])
            out[t, hh] = (S + u[hh][:, None] * kv).T @ r[t, hh]
            S = decay[t, hh][:, None] * S + kv
    out = rms_norm(out, None, eps).reshape(T, H * d) * w[p + "norm"] * gate
    return out @ w[p + "o"].T


# ---- feed-forward, layers, model ----------------------------------------------------------

def gated_feed_forward(h, w, p):
    return (silu(h @ w[p + "gate"].T) * (h @ w[p + "up"].T)) @ w[p + "down"].T


def mixer(kind, h, w, p, mx, eps):
    if kind == "parallel":
        return parallel_mixer(h, w, p, mx, eps)
    if kind == "wkv":
        return wkv(h, w, p, mx, eps)
    raise ValueError(kind)


def forward(config, w, tokens, return_layers=False):
    """Logits ``[T, vocab]`` of one sequence (and the residual stream after every layer)."""
    eps = float(config["norm"]["eps"])
    alpha = float(config["postln_alpha"])
    x = rms_norm(w["embed"][torch.as_tensor(tokens, dtype=torch.long)], w["embed.norm"], eps)
    layers = []
    for i, layer in enumerate(config["layers"]):
        p = f"l{i}."
        x = rms_norm(alpha * x + mixer(layer["type"], x, w, p + "mix.", layer["mixer"], eps), w[p + "norm1"], eps)
        if layer.get("mlp") is not None:
            x = rms_norm(alpha * x + gated_feed_forward(x, w, p + "mlp."), w[p + "norm2"], eps)
        layers.append(x)
    logits = rms_norm(x, w["final.norm"], eps) @ w["head"].T
    return (logits, torch.stack(layers)) if return_layers else logits

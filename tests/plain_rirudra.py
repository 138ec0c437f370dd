"""Plain, slow implementation of the Rirudra decoder: whole sequences, no
cache, one function per mechanism, token-by-token loops for everything that
is a recurrence.  Nothing is imported from the product package.  All math is
done in the dtype asked for (float64 by default: the anchor the product's
float32 and bfloat16 paths are measured against).

Notation: T tokens, W model width, H heads, G key heads (or groups), d key
width per head, e value width per head, sigma(z) = 1 / (1 + exp(-z)).
"""
from __future__ import annotations

import math

import torch

from plain_zodosun import read_folder, write_folder  # noqa: F401  (the file format is the same)


# --------------------------------------------------------------------------
# mechanisms
# --------------------------------------------------------------------------
def rms(x: torch.Tensor, eps: float) -> torch.Tensor:
    """x / sqrt(mean(x^2) + eps) over the last dimension."""
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def offset_norm(x, weight, eps):
    """RMS norm whose stored weight is the distance from one."""
    return rms(x, eps) * (1.0 + weight)


def silu(z):
    return z * torch.sigmoid(z)


def softplus(z):
    return torch.where(z > 30.0, z, torch.log1p(torch.exp(torch.clamp(z, max=30.0))))


def causal_conv(x: torch.Tensor, taps: torch.Tensor, bias=None) -> torch.Tensor:
    """x [T, C], taps [C, K]: y[t, c] = sum_j taps[c, K-1-j] * x[t-j, c], with zeros before the start."""
    T, C = x.shape
    K = taps.shape[1]
    y = torch.zeros_like(x)
    for t in range(T):
        for j in range(K):
            if t - j >= 0:
                y[t] += taps[:, K - 1 - j] * x[t - j]
    if bias is not None:
        y = y + bias
    return y


def unit(x: torch.Tensor, eps: float = 1e-6) -> torch.Tensor:
    return x / torch.sqrt((x * x).sum(dim=-1, keepdim=True) + eps)


def rotate_pairs(x: torch.Tensor, positions: torch.Tensor, dims: int, base: float) -> torch.Tensor:
    """x [T, ..., n]: the first `dims` entries of the last axis are taken in neighbouring pairs (2i, 2i+1) and
    turned by the angle p * base^(-2i / dims); the rest pass."""
    half = dims // 2
    i = torch.arange(half, dtype=x.dtype)
    rate = torch.pow(torch.tensor(base, dtype=x.dtype), -2.0 * i / dims)
    ang = positions.to(x.dtype).reshape(-1, *([1] * (x.dim() - 1))) * rate
    c, s = torch.cos(ang), torch.sin(ang)
    out = x.clone()
    a, b = x[..., 0:dims:2], x[..., 1:dims:2]
    out[..., 0:dims:2] = a * c - b * s
    out[..., 1:dims:2] = b * c + a * s
    return out


def gated_delta(h, w, p, c, eps):
    """Per head a d x e state S with one decay g per head and token:
        S <- g S;  u = beta (v - S^T k);  S <- S + k u^T;  o = S^T q.
    q, k (G heads) and v (H heads) pass a short causal convolution and silu; q and k become unit vectors, q is
    also divided by sqrt(d)."""
    H, G, d, e = c["heads"], c["kv_heads"], c["dim"], c["vdim"]
    T = h.shape[0]
    q = silu(causal_conv(h @ w[p + "q"].T, w[p + "q.conv"])).reshape(T, G, d)
    k = silu(causal_conv(h @ w[p + "k"].T, w[p + "k.conv"])).reshape(T, G, d)
    v = silu(causal_conv(h @ w[p + "v"].T, w[p + "v.conv"])).reshape(T, H, e)
    q = unit(q) * d ** -0.5
    k = unit(k)
    beta = torch.sigmoid(h @ w[p + "b"].T)                                                   # [T, H]
    g = torch.exp(-torch.exp(w[p + "A_log"]) * softplus(h @ w[p + "a"].T + w[p + "dt_bias"]))  # [T, H]
    o = torch.zeros(T, H, e, dtype=h.dtype)
    for head in range(H):
        kh = head // (H // G)
        S = torch.zeros(d, e, dtype=h.dtype)
        for t in range(T):
            S = g[t, head] * S
            u = beta[t, head] * (v[t, head] - S.T @ k[t, kh])
            S = S + torch.outer(k[t, kh], u)
            o[t, head] = S.T @ q[t, kh]
    o = rms(o, eps) * w[p + "norm"]
    o = o.reshape(T, H * e) * silu(h @ w[p + "g"].T)
    return o @ w[p + "o"].T


def state_space(h, w, p, c, eps):
    """Per head an N x e state: S_t = exp(-exp(A) dt) S_{t-1} + dt B_t x_t^T, y_t = S_t^T C_t + D x_t; B and C
    are shared by the heads of a group.  x, B, C pass one causal convolution (with bias) and silu."""
    H, e, N, G, R = c["heads"], c["vdim"], c["state"], c["groups"], c["norm_groups"]
    T = h.shape[0]
    inner = H * e
    u = h @ w[p + "in"].T
    z, xbc, dt = u[:, :inner], u[:, inner:2 * inner + 2 * G * N], u[:, 2 * inner + 2 * G * N:]
    xbc = silu(causal_conv(xbc, w[p + "conv"], w[p + "conv.b"]))
    x = xbc[:, :inner].reshape(T, H, e)
    B = xbc[:, inner:inner + G * N].reshape(T, G, N)
    C = xbc[:, inner + G * N:].reshape(T, G, N)
    dt = softplus(dt + w[p + "dt_bias"])                        # [T, H]
    decay = torch.exp(-torch.exp(w[p + "A_log"]) * dt)
    y = torch.zeros(T, H, e, dtype=h.dtype)
    for head in range(H):
        grp = head // (H // G)
        S = torch.zeros(N, e, dtype=h.dtype)
        for t in range(T):
            S = decay[t, head] * S + dt[t, head] * torch.outer(B[t, grp], x[t, head])
            y[t, head] = S.T @ C[t, grp] + w[p + "D"][head] * x[t, head]
    y = y.reshape(T, inner) * silu(z)
    y = rms(y.reshape(T, R, inner // R), eps).reshape(T, inner) * w[p + "norm"]
    return y @ w[p + "o"].T


def latent_attention(h, w, p, c, eps, start=0):
    """Softmax attention whose keys and values are made per head from one small latent per token; a part of
    every key, shared by the heads, is rotated by position (and so is the matching part of the queries)."""
    H, d, r, e, n = c["heads"], c["dim"], c["rot_dim"], c["vdim"], c["kv_rank"]
    T = h.shape[0]
    pos = torch.arange(start, start + T)
    cq = rms(h @ w[p + "dq"].T, eps) * w[p + "dq.norm"]
    q = (cq @ w[p + "uq"].T).reshape(T, H, d + r)
    kv = h @ w[p + "dkv"].T
    lat = rms(kv[:, :n], eps) * w[p + "dkv.norm"]
    k_rot = rotate_pairs(kv[:, n:], pos, c["rot"]["dims"], c["rot"]["base"])           # [T, r]
    q_rot = rotate_pairs(q[:, :, d:], pos, c["rot"]["dims"], c["rot"]["base"])         # [T, H, r]
    k_flat = (lat @ w[p + "uk"].T).reshape(T, H, d)
    v = (lat @ w[p + "uv"].T).reshape(T, H, e)
    out = torch.zeros(T, H, e, dtype=h.dtype)
    for head in range(H):
        s = (q[:, head, :d] @ k_flat[:, head].T + q_rot[:, head] @ k_rot.T) * c["scale"]     # [T, T]
        s = s.masked_fill(torch.triu(torch.ones(T, T, dtype=torch.bool), 1), -math.inf)
        out[:, head] = torch.softmax(s, dim=-1) @ v[:, head]
    out = out.reshape(T, H * e) * torch.sigmoid(h @ w[p + "g"].T)
    return out @ w[p + "o"].T


def gated_feed_forward(x, w, p):
    return (silu(x @ w[p + "gate"].T) * (x @ w[p + "up"].T)) @ w[p + "down"].T


MIXERS = {"delta": gated_delta, "mamba2": state_space, "latent_attention": latent_attention}


# --------------------------------------------------------------------------
# the model
# --------------------------------------------------------------------------
def decoder(cfg: dict, weights: dict, tokens: list[int], dtype=torch.float64, layers_out: list | None = None):
    """Logits [T, vocab] at every position of `tokens` (a whole sequence from position 0).  `layers_out`, if
    given, collects the residual stream after every layer."""
    w = {n: t.to(dtype) for n, t in weights.items()}
    eps, m = cfg["norm"]["eps"], cfg["residual_mult"]
    x = w["embed"][torch.tensor(tokens)] * cfg["embedding"]["scale"]
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}."
        h = offset_norm(x, w[p + "norm1"], eps)
        y = MIXERS[layer["type"]](h, w, p + "mix.", layer["mixer"], eps)
        if layer.get("mlp") is not None:
            y = y + gated_feed_forward(h, w, p + "mlp.")
        x = x + m * y
        if layers_out is not None:
            layers_out.append(x.clone())
    x = offset_norm(x, w["final.norm"], eps)
    return x @ w["embed"].T


def greedy(cfg: dict, weights: dict, prompt: list[int], n: int, dtype=torch.float64) -> list[int]:
    """n greedy tokens after `prompt`, every step a whole forward pass (ties go to the lowest id)."""
    toks = list(prompt)
    for _ in range(n):
        toks.append(int(torch.argmax(decoder(cfg, weights, toks, dtype)[-1])))
    return toks[len(prompt):]

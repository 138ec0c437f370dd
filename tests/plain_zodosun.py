"""Plain, slow implementation of the Zodosun decoder: whole sequences, no
cache, one function per mechanism, token-by-token loops for everything that
is a recurrence.  Nothing is imported from the product package.  All math is
done in the dtype asked for (float64 by default: the anchor the product's
float32 and bfloat16 paths are measured against).

Notation: T tokens, W model width, H heads, G key/value heads, d key width
per head, e value width per head, sigma(z) = 1 / (1 + exp(-z)).
"""
from __future__ import annotations

import json
import math
import os
import struct

import torch


# --------------------------------------------------------------------------
# mechanisms
# --------------------------------------------------------------------------
def rms(x: torch.Tensor, eps: float) -> torch.Tensor:
    """x / sqrt(mean(x^2) + eps) over the last dimension."""
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def group_norm_rms(x: torch.Tensor, weight: torch.Tensor, groups: int, eps: float) -> torch.Tensor:
    """The last dimension is cut into `groups` equal consecutive parts; each
    part is scaled by its own root mean square; then the whole times weight."""
    shape = x.shape
    parts = x.reshape(*shape[:-1], groups, shape[-1] // groups)
    return rms(parts, eps).reshape(shape) * weight.to(x.dtype)


def sinusoid_positions(positions: torch.Tensor, width: int, dtype) -> torch.Tensor:
    """[T, W]: column 2i = sin(p * 10000^(-2i/W)), column 2i+1 = cos of it."""
    i = torch.arange(width // 2, dtype=dtype)
    rate = torch.pow(torch.tensor(10000.0, dtype=dtype), -2.0 * i / width)
    ang = positions.to(dtype).unsqueeze(1) * rate.unsqueeze(0)
    out = torch.zeros(positions.shape[0], width, dtype=dtype)
    out[:, 0::2] = torch.sin(ang)
    out[:, 1::2] = torch.cos(ang)
    return out


def distance_bucket(n: int, rows: int, far: int) -> int:
    """Row of the distance table for a key n places back: one row per
    distance below rows // 2, then rows that widen geometrically and reach the
    last row at distance `far`."""
    half = rows // 2
    if n < half:
        return n
    return min(rows - 1, half + int(math.floor(math.log(n / half) / math.log(far / half) * (rows - half))))


def query_temperature(p: int, coef: float, every: int) -> float:
    return 1.0 + coef * math.log((p + 1) // every + 1)


def sigmoid_attention(h, w, prefix, c, eps, start=0):
    """Attention without a softmax: every visible key j <= i weighs
    sigma(q_i . k_j * scale + table[bucket(i - j), head] + offset[head]); the
    weights are not normalised.  q and k are each scaled by the root mean
    square of their WHOLE row (all heads together) and a weight per entry; q
    also grows with its position.  Each head's result is gated by
    sigma(gate_row_head . h).  Returns [T, W]."""
    H, G, d, e = c["heads"], c["kv_heads"], c["dim"], c["vdim"]
    T = h.shape[0]
    q = h @ w[prefix + "q"].T + w[prefix + "q.b"]
    k = h @ w[prefix + "k"].T + w[prefix + "k.b"]
    v = h @ w[prefix + "v"].T + w[prefix + "v.b"]
    q = rms(q, eps) * w[prefix + "q.norm"]
    k = rms(k, eps) * w[prefix + "k.norm"]
    temp = torch.tensor([query_temperature(start + t, c["q_temp"]["coef"], c["q_temp"]["every"]) for t in range(T)],
                        dtype=h.dtype)
    q = (q * temp.unsqueeze(1)).reshape(T, H, d)
    k = k.reshape(T, G, d)
    v = v.reshape(T, G, e)
    table, offset = w[prefix + "rel"], w[prefix + "pb"]
    rows = table.shape[0]
    gate = torch.sigmoid(h @ w[prefix + "g"].T)                     # [T, H]
    row_of = torch.tensor([distance_bucket(n, rows, c["bias_max"]) for n in range(T)])
    out = torch.zeros(T, H, e, dtype=h.dtype)
    for head in range(H):
        g = head // (H // G)
        for i in range(T):
            s = (k[: i + 1, g] @ q[i, head]) * c["scale"]
            bias = table[row_of[torch.arange(i, -1, -1)], head]     # key j is i - j places back
            p = torch.sigmoid(s + bias + offset[head])
            out[i, head] = (p.unsqueeze(1) * v[: i + 1, g]).sum(0) * gate[i, head]
    return out.reshape(T, H * e) @ w[prefix + "o"].T


def silu(z):
    return z * torch.sigmoid(z)


def decayed_outer_sum(h, w, prefix, c, eps):
    """Per head a d x e state: S_t = decay_head * S_{t-1} + k_t v_t^T with
    S_{-1} = 0, read as o_t = S_t^T q_t; q, k, v pass through silu.  All heads
    of a token are normed together, gated entry by entry, projected."""
    H, d, e = c["heads"], c["dim"], c["vdim"]
    T = h.shape[0]
    q = silu(h @ w[prefix + "q"].T).reshape(T, H, d)
    k = silu(h @ w[prefix + "k"].T).reshape(T, H, d)
    v = silu(h @ w[prefix + "v"].T).reshape(T, H, e)
    o = torch.zeros(T, H, e, dtype=h.dtype)
    for head in range(H):
        S = torch.zeros(d, e, dtype=h.dtype)
        for t in range(T):
            S = c["decay"][head] * S + torch.outer(k[t, head], v[t, head])
            o[t, head] = S.T @ q[t, head]
    o = rms(o.reshape(T, H * e), eps) * w[prefix + "norm"]
    o = o * torch.sigmoid(h @ w[prefix + "g"].T)
    return o @ w[prefix + "o"].T


def side_by_side(h, w, prefix, c, eps, start=0):
    """Both mixers read h; each result is normed over the model width with a
    weight of its own; the answer is half their sum."""
    a = sigmoid_attention(h, w, prefix + "left.", c["left"], eps, start)
    b = decayed_outer_sum(h, w, prefix + "right.", c["right"], eps)
    return 0.5 * (rms(a, eps) * w[prefix + "left.out"] + rms(b, eps) * w[prefix + "right.out"])


def delta_rule(h, w, prefix, c, eps):
    """Per head a d x d state.  With the unit key u = k / sqrt(|k|^2 + 1e-6),
    a decay per key channel wt in (exp(-exp(-1/2)), 1) and a removal rate per
    key channel a in (0, 1):
        S_t = diag(wt) S_{t-1} - (a * u) (u^T S_{t-1}) + k v^T,   o_t = S_t^T r.
    Each head's o is scaled by its root mean square; then weight, gate,
    projection."""
    H, d = c["heads"], c["dim"]
    T = h.shape[0]
    r = (h @ w[prefix + "r"].T).reshape(T, H, d)
    k = (h @ w[prefix + "k"].T).reshape(T, H, d)
    v = (h @ w[prefix + "v"].T).reshape(T, H, d)
    low = torch.tanh(h @ w[prefix + "w1"].T) @ w[prefix + "w2"].T + w[prefix + "w0"]
    wt = torch.exp(-math.exp(-0.5) * torch.sigmoid(low)).reshape(T, H, d)
    a = torch.sigmoid(h @ w[prefix + "a"].T + w[prefix + "a.b"]).reshape(T, H, d)
    u = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
    o = torch.zeros(T, H, d, dtype=h.dtype)
    for head in range(H):
        S = torch.zeros(d, d, dtype=h.dtype)
        for t in range(T):
            uS = u[t, head] @ S
            S = wt[t, head].unsqueeze(1) * S - torch.outer(a[t, head] * u[t, head], uS) \
                + torch.outer(k[t, head], v[t, head])
            o[t, head] = S.T @ r[t, head]
    o = rms(o, eps).reshape(T, H * d) * w[prefix + "norm"]
    o = o * torch.sigmoid(h @ w[prefix + "g"].T)
    return o @ w[prefix + "o"].T


def gated_feed_forward(x, w, prefix):
    return (silu(x @ w[prefix + "gate"].T) * (x @ w[prefix + "up"].T)) @ w[prefix + "down"].T


# --------------------------------------------------------------------------
# the model
# --------------------------------------------------------------------------
def decoder(cfg: dict, weights: dict, tokens: list[int], dtype=torch.float64, layers_out: list | None = None):
    """Logits [T, vocab] at every position of `tokens` (a whole sequence from
    position 0).  `layers_out`, if given, collects the residual stream after
    every layer."""
    w = {n: t.to(dtype) for n, t in weights.items()}
    eps, groups, W = cfg["norm"]["eps"], cfg["norm"]["groups"], cfg["width"]
    T = len(tokens)
    x = w["embed"][torch.tensor(tokens)] + sinusoid_positions(torch.arange(T), W, dtype)
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}."
        h = group_norm_rms(x, w[p + "norm1"], groups, eps)
        if layer["type"] == "parallel":
            x = x + side_by_side(h, w, p + "mix.", layer["mixer"], eps)
        elif layer["type"] == "general_delta":
            x = x + delta_rule(h, w, p + "mix.", layer["mixer"], eps)
        else:
            raise ValueError(f"unknown layer type {layer['type']}")
        if layer.get("mlp") is not None:
            x = x + gated_feed_forward(group_norm_rms(x, w[p + "norm2"], groups, eps), w, p + "mlp.")
        if layers_out is not None:
            layers_out.append(x.clone())
    x = group_norm_rms(x, w["final.norm"], groups, eps)
    return (x @ w["head"].T) * cfg["logit_scale"]


# --------------------------------------------------------------------------
# files (a reader of this file's own: a length, a JSON header, raw data)
# --------------------------------------------------------------------------
_DT = {"BF16": (torch.bfloat16, 2), "F32": (torch.float32, 4), "I32": (torch.int32, 4), "F16": (torch.float16, 2)}


def read_folder(folder: str):
    with open(os.path.join(folder, "config.json")) as f:
        cfg = json.load(f)
    with open(os.path.join(folder, "model.safetensors"), "rb") as f:
        (n,) = struct.unpack("<Q", f.read(8))
        header = json.loads(f.read(n))
        data = f.read()
    out = {}
    for name, meta in header.items():
        if name == "__metadata__":
            continue
        dt, _ = _DT[meta["dtype"]]
        a, b = meta["data_offsets"]
        out[name] = torch.frombuffer(bytearray(data[a:b]), dtype=dt).reshape(meta["shape"]).clone()
    return cfg, out


def write_folder(folder: str, cfg: dict, weights: dict) -> str:
    """config.json and model.safetensors (bfloat16 / float32 / int32 tensors)."""
    os.makedirs(folder, exist_ok=True)
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(cfg, f, indent=1)
    names = {torch.bfloat16: "BF16", torch.float32: "F32", torch.int32: "I32", torch.float16: "F16"}
    header, blobs, at = {}, [], 0
    for name, t in weights.items():
        t = t.contiguous()
        raw = t.view(torch.uint8).numpy().tobytes() if t.dtype != torch.bfloat16 else \
            t.view(torch.int16).numpy().tobytes()
        header[name] = {"dtype": names[t.dtype], "shape": list(t.shape), "data_offsets": [at, at + len(raw)]}
        blobs.append(raw)
        at += len(raw)
    head = json.dumps(header).encode()
    head += b" " * (-len(head) % 8)
    with open(os.path.join(folder, "model.safetensors"), "wb") as f:
        f.write(struct.pack("<Q", len(head)))
        f.write(head)
        for b in blobs:
            f.write(b)
    return folder


def greedy(cfg: dict, weights: dict, prompt: list[int], n: int, dtype=torch.float64) -> list[int]:
    """n greedy tokens after `prompt`, every step a whole forward pass (ties go to the lowest id)."""
    toks = list(prompt)
    for _ in range(n):
        toks.append(int(torch.argmax(decoder(cfg, weights, toks, dtype)[-1])))
    return toks[len(prompt):]

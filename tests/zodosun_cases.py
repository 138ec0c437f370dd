"""Small Zodosun configurations, weights with a spread that lets every
mechanism matter, and the plain implementation as oracle (cached)."""
from __future__ import annotations

import os

import torch

import plain_zodosun as pz


def _left(heads, kv, dim, vdim, scale, far, coef, every, rows):
    return {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "scale": scale, "bias_max": far,
            "q_temp": {"coef": coef, "every": every}, "bias_rows": rows}


def _right(heads, dim, vdim, decay):
    return {"heads": heads, "dim": dim, "vdim": vdim, "decay": decay}


def _delta(heads, dim, rank):
    return {"type": "general_delta", "mixer": {"heads": heads, "dim": dim, "rank": rank}}


def _ff(n):
    return None if n is None else {"kind": "dense", "ff": n}


# A: three norm groups, six query heads on three key/value heads, keys and values of different widths, a
#    distance table that saturates after 40 places, layers in mixed order, with and without feed-forward.
Z_A = {
    "architecture": "Zodosun", "vocab": 300, "width": 96, "logit_scale": 0.75, "norm": {"eps": 1e-6, "groups": 3},
    "layers": [
        {"type": "parallel", "mlp": _ff(160),
         "mixer": {"left": _left(6, 3, 16, 24, 0.2, 40, 0.5, 7, 12), "right": _right(3, 24, 16, [0.5, 0.9, 0.99])}},
        {**_delta(3, 24, 8), "mlp": _ff(128)},
        {**_delta(2, 40, 12), "mlp": None},
        {"type": "parallel", "mlp": None,
         "mixer": {"left": _left(2, 2, 32, 8, 0.3, 100, 0.25, 16, 9), "right": _right(1, 8, 48, [0.97])}},
    ],
}
# B: one norm group, no logit scaling, one key/value head for three query heads, wider heads (other templates of
#    the scan kernel), a temperature that moves at every position.
Z_B = {
    "architecture": "Zodosun", "vocab": 1000, "width": 128, "logit_scale": 1.0, "norm": {"eps": 1e-5, "groups": 1},
    "layers": [
        {**_delta(2, 64, 16), "mlp": _ff(200)},
        {"type": "parallel", "mlp": _ff(96),
         "mixer": {"left": _left(3, 1, 48, 40, 0.1, 600, 0.1, 1, 20), "right": _right(2, 48, 80, [0.8, 0.999])}},
        {**_delta(1, 128, 64), "mlp": None},
        {**_delta(1, 160, 24), "mlp": None},
    ],
}
# C: delta rule first and last, two side-by-side layers in a row, a width that is no multiple of 8.
Z_C = {
    "architecture": "Zodosun", "vocab": 130, "width": 84, "logit_scale": 2.0, "norm": {"eps": 1e-5, "groups": 4},
    "layers": [
        {**_delta(5, 12, 4), "mlp": None},
        {"type": "parallel", "mlp": None,
         "mixer": {"left": _left(4, 4, 20, 20, 0.15, 30, 1.0, 3, 16), "right": _right(4, 20, 20, [0.3, 0.6, 0.9, 1.0])}},
        {"type": "parallel", "mlp": _ff(100),
         "mixer": {"left": _left(4, 2, 8, 12, 0.5, 17, 0.0, 5, 2), "right": _right(2, 16, 24, [0.95, 0.7])}},
        {**_delta(3, 28, 20), "mlp": _ff(64)},
    ],
}
# D: attention heads of 64 and 128 (the widths the tensor-core attention kernels take), five norm groups.
Z_D = {
    "architecture": "Zodosun", "vocab": 384, "width": 160, "logit_scale": 0.3, "norm": {"eps": 1e-6, "groups": 5},
    "layers": [
        {"type": "parallel", "mlp": None,
         "mixer": {"left": _left(2, 1, 64, 64, 0.11, 90, 0.4, 10, 24), "right": _right(5, 16, 32, [0.2, 0.5, 0.8, 0.95, 0.999])}},
        {**_delta(4, 40, 10), "mlp": _ff(96)},
        {"type": "parallel", "mlp": _ff(192),
         "mixer": {"left": _left(2, 2, 128, 128, 0.07, 300, 0.15, 50, 40), "right": _right(2, 64, 64, [0.9, 0.99])}},
    ],
}
# E: delta-rule layers only (no keys or values are cached at all), head widths that are no multiples of four.
Z_E = {
    "architecture": "Zodosun", "vocab": 200, "width": 72, "logit_scale": 1.5, "norm": {"eps": 1e-5, "groups": 2},
    "layers": [{**_delta(3, 10, 5), "mlp": _ff(80)}, {**_delta(2, 30, 7), "mlp": None}],
}
# F: side-by-side layers only, value widths that are no multiples of four, a distance table of two rows.
Z_F = {
    "architecture": "Zodosun", "vocab": 210, "width": 64, "logit_scale": 1.0, "norm": {"eps": 1e-5, "groups": 8},
    "layers": [
        {"type": "parallel", "mlp": _ff(72),
         "mixer": {"left": _left(2, 1, 10, 6, 0.4, 50, 0.3, 4, 2), "right": _right(3, 10, 6, [0.9, 0.8, 0.7])}},
        {"type": "parallel", "mlp": None,
         "mixer": {"left": _left(1, 1, 30, 7, 0.2, 20, 0.0, 1, 7), "right": _right(1, 30, 7, [0.99])}},
    ],
}
CASES = {"a": Z_A, "b": Z_B, "c": Z_C, "d": Z_D, "e": Z_E, "f": Z_F}


def make_weights(cfg: dict, seed: int) -> dict:
    """bfloat16 tensors by name: matrices N(0, 1/fan_in) times a gain, norm weights around 1, biases and tables with
    a spread of their own, so that scores, gates, decays and removal rates cover their ranges."""
    g = torch.Generator().manual_seed(seed)

    def normal(*shape, std=1.0, mean=0.0):
        return (torch.randn(*shape, generator=g) * std + mean).to(torch.bfloat16)

    def matrix(out, inp, gain=1.0):
        return normal(out, inp, std=gain / inp ** 0.5)

    W = cfg["width"]
    w = {"embed": normal(cfg["vocab"], W), "final.norm": normal(W, std=0.1, mean=1.0),
         "head": matrix(cfg["vocab"], W)}
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}."
        w[p + "norm1"] = normal(W, std=0.1, mean=1.0)
        m = layer["mixer"]
        if layer["type"] == "general_delta":
            n, r = m["heads"] * m["dim"], m["rank"]
            for x in ("r", "k", "v", "g", "a"):
                w[p + "mix." + x] = matrix(n, W, 1.5)
            w[p + "mix.a.b"] = normal(n, std=0.5)
            w[p + "mix.w1"] = matrix(r, W, 1.5)
            w[p + "mix.w2"] = matrix(n, r, 2.0)
            w[p + "mix.w0"] = normal(n, std=1.0)
            w[p + "mix.norm"] = normal(n, std=0.1, mean=1.0)
            w[p + "mix.o"] = matrix(W, n)
        else:
            l, r = m["left"], m["right"]
            q = p + "mix.left."
            nq, nk, nv = l["heads"] * l["dim"], l["kv_heads"] * l["dim"], l["kv_heads"] * l["vdim"]
            w[q + "q"], w[q + "k"], w[q + "v"] = matrix(nq, W, 2.0), matrix(nk, W, 2.0), matrix(nv, W)
            w[q + "q.b"], w[q + "k.b"], w[q + "v.b"] = normal(nq, std=0.3), normal(nk, std=0.3), normal(nv, std=0.3)
            w[q + "q.norm"], w[q + "k.norm"] = normal(nq, std=0.2, mean=2.0), normal(nk, std=0.2, mean=2.0)
            w[q + "rel"] = normal(l["bias_rows"], l["heads"], std=1.5)
            w[q + "pb"] = normal(l["heads"], std=0.5, mean=-2.0)
            w[q + "g"] = matrix(l["heads"], W, 2.0)
            w[q + "o"] = matrix(W, l["heads"] * l["vdim"])
            s = p + "mix.right."
            nq, nv = r["heads"] * r["dim"], r["heads"] * r["vdim"]
            w[s + "q"], w[s + "k"] = matrix(nq, W, 1.5), matrix(nq, W, 1.5)
            w[s + "v"], w[s + "g"] = matrix(nv, W, 1.5), matrix(nv, W, 1.5)
            w[s + "norm"] = normal(nv, std=0.1, mean=1.0)
            w[s + "o"] = matrix(W, nv)
            w[p + "mix.left.out"] = normal(W, std=0.1, mean=1.0)
            w[p + "mix.right.out"] = normal(W, std=0.1, mean=1.0)
        if layer["mlp"] is not None:
            f = layer["mlp"]["ff"]
            w[p + "norm2"] = normal(W, std=0.1, mean=1.0)
            w[p + "mlp.gate"], w[p + "mlp.up"], w[p + "mlp.down"] = matrix(f, W), matrix(f, W), matrix(W, f)
    return w


_folders: dict = {}
_oracle: dict = {}


def folder(tmp_root, name: str, seed: int = 5) -> str:
    key = (name, seed)
    if key not in _folders:
        _folders[key] = pz.write_folder(os.path.join(str(tmp_root), f"zodosun_{name}_{seed}"), CASES[name],
                                        make_weights(CASES[name], seed))
    return _folders[key]


def oracle_logits(path: str, tokens: list[int]) -> torch.Tensor:
    """float64 logits of the plain implementation at every position."""
    key = (path, tuple(tokens))
    if key not in _oracle:
        cfg, w = pz.read_folder(path)
        _oracle[key] = pz.decoder(cfg, w, tokens, torch.float64)
    return _oracle[key]


def tokens(n: int, vocab: int, seed: int) -> list[int]:
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (n,), generator=g).tolist()

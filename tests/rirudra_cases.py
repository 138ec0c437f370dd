"""Small Rirudra configurations, weights with a spread that lets every
mechanism matter, and the plain implementation as oracle (cached)."""
from __future__ import annotations

import os

import torch

import plain_rirudra as pr


def _latent(heads, dim, rot_dim, vdim, q_rank, kv_rank, scale, base=10000.0, dims=None):
    return {"type": "latent_attention",
            "mixer": {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "q_rank": q_rank, "kv_rank": kv_rank,
                      "scale": scale, "rot": {"base": base, "dims": rot_dim if dims is None else dims}}}


def _ssm(heads, vdim, state, groups, norm_groups, conv):
    return {"type": "mamba2", "mixer": {"heads": heads, "vdim": vdim, "state": state, "groups": groups,
                                         "norm_groups": norm_groups, "conv": conv}}


def _delta(heads, kv_heads, dim, vdim, conv):
    return {"type": "delta", "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": conv}}


def _ff(n):
    return None if n is None else {"kind": "dense", "ff": n}


def _model(vocab, width, emb, mult, eps, layers):
    return {"architecture": "Rirudra", "vocab": vocab, "width": width, "embedding": {"scale": emb},
            "residual_mult": mult, "norm": {"eps": eps}, "layers": layers}


# A: all three mixers in mixed order, with and without feed-forward; cached rows of 56 and 116 values (padded to 64
#    and 128); value widths that differ from the key widths; two heads per key head and per group.
R_A = _model(300, 96, 4.0, 0.5, 1e-6, [
    {**_latent(3, 16, 8, 24, 40, 48, 0.2), "mlp": _ff(160)},
    {**_ssm(4, 12, 16, 2, 2, 4), "mlp": None},
    {**_delta(4, 2, 24, 16, 3), "mlp": _ff(128)},
    {**_latent(2, 32, 16, 8, 24, 100, 0.15, base=500.0), "mlp": None},
])
# B: no scaling anywhere (embedding scale 1, residual factor 1: the layers' results go straight into the stream);
#    recurrences first; one group, one norm group, two taps; three heads on one key head; five taps.
R_B = _model(1000, 128, 1.0, 1.0, 1e-5, [
    {**_delta(2, 2, 64, 32, 2), "mlp": _ff(200)},
    {**_ssm(2, 64, 64, 1, 1, 2), "mlp": _ff(96)},
    {**_latent(5, 24, 24, 40, 64, 40, 0.12, base=1e6), "mlp": None},
    {**_delta(3, 1, 40, 72, 5), "mlp": None},
])
# C: a width that is no multiple of 8, head widths that are no multiples of four, one attention head, groups == heads.
R_C = _model(130, 84, 7.0, 0.25, 1e-5, [
    {**_ssm(6, 10, 12, 6, 3, 3), "mlp": None},
    {**_delta(2, 1, 10, 6, 4), "mlp": _ff(100)},
    {**_latent(1, 8, 4, 12, 10, 20, 0.3, base=100.0), "mlp": _ff(64)},
    {**_ssm(3, 7, 5, 1, 1, 1), "mlp": None},
])
# D: attention only (no state at all): cached rows of 128 and 64 values (what the tensor-core kernels take), of 192,
#    and of 304 (beyond 256); fewer rotated entries than the rotated part holds.
R_D = _model(384, 160, 10.0, 0.3, 1e-6, [
    {**_latent(4, 64, 32, 64, 96, 96, 0.1), "mlp": None},
    {**_latent(8, 32, 16, 32, 48, 48, 0.14, base=1e5), "mlp": _ff(96)},
    {**_latent(2, 48, 32, 16, 32, 160, 0.11, dims=16), "mlp": None},
    {**_latent(2, 16, 16, 24, 56, 288, 0.2), "mlp": _ff(192)},
])
# E: recurrences only (no keys are cached at all): wide states (other forms of the scan kernels), more value columns
#    than keys and fewer.
R_E = _model(200, 72, 3.0, 0.4, 1e-5, [
    {**_ssm(2, 64, 128, 1, 2, 4), "mlp": _ff(80)},
    {**_delta(1, 1, 128, 96, 4), "mlp": None},
    {**_delta(2, 2, 160, 8, 3), "mlp": None},
    {**_ssm(2, 40, 144, 2, 1, 8), "mlp": None},
])
# P: attention whose softmax is sharp (a large scale and large rotated keys): a single key, far back or at a page's
#    edge, decides a row's result, so that a kernel that loses or misplaces one key is off by the size of the logits.
R_P = _model(150, 64, 3.0, 1.0, 1e-5, [
    {**_latent(2, 16, 16, 16, 32, 48, 1.5, base=10000.0), "mlp": None},
])
CASES = {"a": R_A, "b": R_B, "c": R_C, "d": R_D, "e": R_E, "p": R_P}


def make_weights(cfg: dict, seed: int) -> dict:
    """bfloat16 tensors by name: matrices N(0, 1/fan_in) times a gain; norm weights around 0 where the design adds
    one and around 1 elsewhere; decays, step sizes and taps with a spread of their own."""
    g = torch.Generator().manual_seed(seed)

    def normal(*shape, std=1.0, mean=0.0):
        return (torch.randn(*shape, generator=g) * std + mean).to(torch.bfloat16)

    def matrix(out, inp, gain=1.0):
        return normal(out, inp, std=gain / inp ** 0.5)

    W = cfg["width"]
    w = {"embed": normal(cfg["vocab"], W, std=1.0 / cfg["embedding"]["scale"]), "final.norm": normal(W, std=0.2)}
    sharp = cfg is R_P
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}."
        w[p + "norm1"] = normal(W, std=0.2)
        m, q = layer["mixer"], p + "mix."
        if layer["type"] == "latent_attention":
            H, d, r, e = m["heads"], m["dim"], m["rot_dim"], m["vdim"]
            w[q + "dq"], w[q + "dq.norm"] = matrix(m["q_rank"], W), normal(m["q_rank"], std=0.15, mean=1.0)
            w[q + "uq"] = matrix(H * (d + r), m["q_rank"], 2.0)
            dkv = matrix(m["kv_rank"] + r, W, 1.5).float()
            if sharp:
                dkv[m["kv_rank"]:] *= 6.0
            w[q + "dkv"], w[q + "dkv.norm"] = dkv.to(torch.bfloat16), normal(m["kv_rank"], std=0.15, mean=1.0)
            w[q + "uk"], w[q + "uv"] = matrix(H * d, m["kv_rank"], 2.0), matrix(H * e, m["kv_rank"], 1.5)
            w[q + "g"], w[q + "o"] = matrix(H * e, W, 2.0), matrix(W, H * e)
        elif layer["type"] == "mamba2":
            H, e, N, G = m["heads"], m["vdim"], m["state"], m["groups"]
            inner, C = H * e, H * e + 2 * G * N
            w[q + "in"] = matrix(2 * inner + 2 * G * N + H, W, 1.5)
            w[q + "conv"], w[q + "conv.b"] = normal(C, m["conv"], std=0.5), normal(C, std=0.2)
            w[q + "dt_bias"], w[q + "A_log"] = normal(H, std=1.0, mean=-1.0), normal(H, std=1.0, mean=-0.5)
            w[q + "D"], w[q + "norm"] = normal(H, std=0.3, mean=1.0), normal(inner, std=0.15, mean=1.0)
            w[q + "o"] = matrix(W, inner)
        else:
            H, G, d, e = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
            w[q + "q"], w[q + "k"], w[q + "v"] = matrix(G * d, W, 1.5), matrix(G * d, W, 1.5), matrix(H * e, W, 1.5)
            for x, n in (("q", G * d), ("k", G * d), ("v", H * e)):
                w[q + x + ".conv"] = normal(n, m["conv"], std=0.5)
            w[q + "b"], w[q + "a"] = matrix(H, W, 2.0), matrix(H, W, 2.0)
            w[q + "A_log"], w[q + "dt_bias"] = normal(H, std=1.0, mean=-1.5), normal(H, std=1.0, mean=-2.0)
            w[q + "norm"] = normal(e, std=0.15, mean=1.0)
            w[q + "g"], w[q + "o"] = matrix(H * e, W, 1.5), matrix(W, H * e)
        if layer["mlp"] is not None:
            f = layer["mlp"]["ff"]
            w[p + "mlp.gate"], w[p + "mlp.up"], w[p + "mlp.down"] = matrix(f, W), matrix(f, W), matrix(W, f)
    return w


_folders: dict = {}
_oracle: dict = {}


def folder(tmp_root, name: str, seed: int = 5) -> str:
    key = (name, seed)
    if key not in _folders:
        _folders[key] = pr.write_folder(os.path.join(str(tmp_root), f"rirudra_{name}_{seed}"), CASES[name],
                                        make_weights(CASES[name], seed))
    return _folders[key]


def oracle_logits(path: str, tokens: list[int]) -> torch.Tensor:
    """float64 logits of the plain implementation at every position."""
    key = (path, tuple(tokens))
    if key not in _oracle:
        cfg, w = pr.read_folder(path)
        _oracle[key] = pr.decoder(cfg, w, tokens, torch.float64)
    return _oracle[key]


def tokens(n: int, vocab: int, seed: int) -> list[int]:
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (n,), generator=g).tolist()

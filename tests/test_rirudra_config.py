"""Rirudra: configuration, registry, tensor list, and the plain implementation's mechanisms against closed forms
(all on the CPU)."""
import copy
import math

import pytest
import torch

import plain_rirudra as pr
from rirudra_cases import CASES, make_weights, tokens


def _spec(cfg):
    from tq_kv_b200.config import spec_from_config_dict
    return spec_from_config_dict(cfg)


def test_the_architecture_is_registered_and_a_configuration_round_trips():
    from tq_kv_b200.config import registered_architectures
    assert "Rirudra" in registered_architectures()
    for name, cfg in CASES.items():
        arch, typed, spec = _spec(cfg)
        assert arch.name == "Rirudra" and typed.to_dict()["layers"] == cfg["layers"], name
        assert len(spec.layers) == len(cfg["layers"]) and all(l.block == "parallel_residual" for l in spec.layers)
        assert [l.mixer.kind for l in spec.layers] == [
            {"latent_attention": "latent_attention", "mamba2": "state_space_mixer", "delta": "gated_delta_mixer"}[x["type"]]
            for x in cfg["layers"]]
        assert [l.feed_forward is None for l in spec.layers] == [x["mlp"] is None for x in cfg["layers"]]
        # the stream is kept divided by the residual factor: embeddings and the norms' eps carry it
        m = cfg["residual_mult"]
        assert spec.head.params["tied_to"] == "embed" and spec.embedding.params["scale"] == cfg["embedding"]["scale"] / m
        assert spec.final_norm.params["eps"] == cfg["norm"]["eps"] / (m * m)
        assert all(l.block_params["residual_mult"] == 1.0 for l in spec.layers)
    zero = dict(CASES["a"], residual_mult=0.0)                       # nothing to fold: the block scales the sum
    spec = _spec(zero)[2]
    assert spec.layers[0].block_params["residual_mult"] == 0.0 and spec.embedding.params["scale"] == zero["embedding"]["scale"]


@pytest.mark.parametrize("path,key", [((), "vocab"), ((), "residual_mult"), (("embedding",), "scale"), (("norm",), "eps"),
                                      (("layers", 0, "mixer"), "kv_rank"), (("layers", 0, "mixer", "rot"), "base"),
                                      (("layers", 1, "mixer"), "norm_groups"), (("layers", 2, "mixer"), "kv_heads"),
                                      (("layers", 2), "type")])
def test_a_missing_key_is_named(path, key):
    from tq_kv_b200.config import ConfigError
    cfg = copy.deepcopy(CASES["a"])
    d = cfg
    for p in path:
        d = d[p]
    del d[key]
    with pytest.raises(ConfigError, match=key):
        _spec(cfg)


def test_sizes_that_contradict_each_other_are_refused():
    from tq_kv_b200.config import ConfigError
    for where, key, value in (((1,), "groups", 3), ((2,), "kv_heads", 3), ((0, "rot"), "dims", 7), ((1,), "norm_groups", 5)):
        cfg = copy.deepcopy(CASES["a"])
        d = cfg["layers"][where[0]]["mixer"]
        for p in where[1:]:
            d = d[p]
        d[key] = value
        with pytest.raises(ConfigError):
            _spec(cfg)
    cfg = copy.deepcopy(CASES["a"])
    cfg["layers"][0]["type"] = "something"
    with pytest.raises(ConfigError, match="something"):
        _spec(cfg)


def test_the_model_asks_for_exactly_the_tensors_of_the_design():
    from tq_kv_b200.engine.model import DecoderModel
    for name, cfg in CASES.items():
        model = DecoderModel(_spec(cfg)[2])
        want = make_weights(cfg, 1)
        specs = model.weight_specs()
        assert set(specs) == set(want), name
        assert all(tuple(specs[n].shape) == tuple(want[n].shape) for n in want), name
        kv, state = model.cache_requests()
        for i, layer in enumerate(cfg["layers"]):
            m = layer["mixer"]
            if layer["type"] == "latent_attention":        # one row per token: the latent and the rotated part, padded
                assert kv[i].n_kv_heads == 1 and kv[i].head_dim == -(-(m["kv_rank"] + m["rot_dim"]) // 16) * 16
            elif layer["type"] == "mamba2":
                chans = m["heads"] * m["vdim"] + 2 * m["groups"] * m["state"]
                assert state[i].shape == (m["heads"] * m["state"] * m["vdim"] + (m["conv"] - 1) * chans,)
            else:
                chans = 2 * m["kv_heads"] * m["dim"] + m["heads"] * m["vdim"]
                assert state[i].shape == (m["heads"] * m["dim"] * m["vdim"] + (m["conv"] - 1) * chans,)


# ---- the plain implementation's mechanisms ------------------------------------------------------------------
def test_causal_convolution_against_the_library_and_its_first_tokens():
    g = torch.Generator().manual_seed(0)
    x, taps = torch.randn(9, 5, generator=g, dtype=torch.float64), torch.randn(5, 4, generator=g, dtype=torch.float64)
    want = torch.nn.functional.conv1d(torch.nn.functional.pad(x.T.unsqueeze(0), (3, 0)), taps.unsqueeze(1), groups=5)[0].T
    assert torch.allclose(pr.causal_conv(x, taps), want, atol=1e-12)
    assert torch.allclose(pr.causal_conv(x, taps)[0], taps[:, -1] * x[0])          # nothing before the start


def test_rotation_keeps_lengths_and_depends_on_the_distance_only():
    g = torch.Generator().manual_seed(1)
    q, k = torch.randn(1, 12, generator=g, dtype=torch.float64), torch.randn(1, 12, generator=g, dtype=torch.float64)
    def dot(i, j):
        return float(pr.rotate_pairs(q, torch.tensor([i]), 8, 100.0)[0] @ pr.rotate_pairs(k, torch.tensor([j]), 8, 100.0)[0])
    assert abs(dot(7, 3) - dot(104, 100)) < 1e-9 and abs(dot(7, 3) - dot(7, 4)) > 1e-6
    r = pr.rotate_pairs(q, torch.tensor([5]), 8, 100.0)
    assert torch.allclose(r[0, 8:], q[0, 8:]) and abs(float(r.norm() - q.norm())) < 1e-12
    a = 5 * 100.0 ** (-2 / 8)                                   # the second pair's angle at position 5
    assert abs(float(r[0, 2]) - float(q[0, 2] * math.cos(a) - q[0, 3] * math.sin(a))) < 1e-12


def _one_layer(kind):
    cfg = copy.deepcopy(CASES["a"])
    cfg["layers"] = [l for l in cfg["layers"] if l["type"] == kind][:1]
    return cfg


def test_the_state_space_recurrence_as_a_weighted_sum_over_the_past():
    cfg = _one_layer("mamba2")
    w = {n: t.double() for n, t in make_weights(cfg, 3).items()}
    c, eps, p = cfg["layers"][0]["mixer"], cfg["norm"]["eps"], "l0.mix."
    h = torch.randn(7, cfg["width"], generator=torch.Generator().manual_seed(2), dtype=torch.float64)
    H, e, N, G = c["heads"], c["vdim"], c["state"], c["groups"]
    inner = H * e
    u = h @ w[p + "in"].T
    xbc = pr.silu(pr.causal_conv(u[:, inner:2 * inner + 2 * G * N], w[p + "conv"], w[p + "conv.b"]))
    x, B, C = xbc[:, :inner].reshape(7, H, e), xbc[:, inner:inner + G * N].reshape(7, G, N), xbc[:, inner + G * N:].reshape(7, G, N)
    dt = torch.log1p(torch.exp(u[:, 2 * inner + 2 * G * N:] + w[p + "dt_bias"]))
    g = torch.exp(-torch.exp(w[p + "A_log"]) * dt)
    y = torch.zeros(7, H, e, dtype=torch.float64)
    for head in range(H):
        grp = head // (H // G)
        for t in range(7):
            for s in range(t + 1):
                y[t, head] += torch.prod(g[s + 1:t + 1, head]) * dt[s, head] * (C[t, grp] @ B[s, grp]) * x[s, head]
            y[t, head] += w[p + "D"][head] * x[t, head]
    y = y.reshape(7, inner) * pr.silu(u[:, :inner])
    R = c["norm_groups"]
    y = (pr.rms(y.reshape(7, R, inner // R), eps).reshape(7, inner) * w[p + "norm"]) @ w[p + "o"].T
    assert torch.allclose(pr.state_space(h, w, p, c, eps), y, atol=1e-10)


def test_the_delta_rule_replaces_what_the_state_holds_along_a_key():
    """With full write strength and no decay, reading with a key returns the value last written with it."""
    d, e = 6, 4
    g = torch.Generator().manual_seed(4)
    keys = torch.linalg.qr(torch.randn(d, d, generator=g, dtype=torch.float64))[0]      # orthonormal rows
    S = torch.zeros(d, e, dtype=torch.float64)
    vals = torch.randn(5, e, generator=g, dtype=torch.float64)
    for t, ki in enumerate([0, 1, 2, 0, 1]):
        k = keys[ki]
        S = 1.0 * S
        S = S + torch.outer(k, 1.0 * (vals[t] - S.T @ k))
    assert torch.allclose(S.T @ keys[0], vals[3]) and torch.allclose(S.T @ keys[1], vals[4]) and torch.allclose(S.T @ keys[2], vals[2])


def test_latent_attention_equals_attention_in_the_latents_space():
    """score = q~ . [c, k_r] with q~ = [U_k^T q_flat, rot(q_rot)], and out = U_v (weighted mean of c)."""
    cfg = _one_layer("latent_attention")
    w = {n: t.double() for n, t in make_weights(cfg, 6).items()}
    c, eps, p = cfg["layers"][0]["mixer"], cfg["norm"]["eps"], "l0.mix."
    T = 9
    h = torch.randn(T, cfg["width"], generator=torch.Generator().manual_seed(5), dtype=torch.float64)
    H, d, r, e, n = c["heads"], c["dim"], c["rot_dim"], c["vdim"], c["kv_rank"]
    pos = torch.arange(T)
    q = ((pr.rms(h @ w[p + "dq"].T, eps) * w[p + "dq.norm"]) @ w[p + "uq"].T).reshape(T, H, d + r)
    kv = h @ w[p + "dkv"].T
    rows = torch.cat([pr.rms(kv[:, :n], eps) * w[p + "dkv.norm"], pr.rotate_pairs(kv[:, n:], pos, r, c["rot"]["base"])], 1)
    out = torch.zeros(T, H, e, dtype=torch.float64)
    for head in range(H):
        uk, uv = w[p + "uk"][head * d:(head + 1) * d], w[p + "uv"][head * e:(head + 1) * e]
        qt = torch.cat([q[:, head, :d] @ uk, pr.rotate_pairs(q[:, head, d:], pos, r, c["rot"]["base"])], 1)
        s = (qt @ rows.T * c["scale"]).masked_fill(torch.triu(torch.ones(T, T, dtype=torch.bool), 1), float("-inf"))
        out[:, head] = (torch.softmax(s, -1) @ rows[:, :n]) @ uv.T
    want = (out.reshape(T, H * e) * torch.sigmoid(h @ w[p + "g"].T)) @ w[p + "o"].T
    assert torch.allclose(pr.latent_attention(h, w, p, c, eps), want, atol=1e-10)
    # a later start only moves the positions: the first query sees itself alone, whatever its position
    assert torch.allclose(pr.latent_attention(h[:1], w, p, c, eps, start=40), pr.latent_attention(h[:1], w, p, c, eps))


def test_a_layers_sublayers_read_one_norm_and_enter_the_stream_scaled():
    cfg = copy.deepcopy(CASES["a"])
    cfg["layers"] = cfg["layers"][:1]
    w = make_weights(cfg, 8)
    toks = tokens(5, cfg["vocab"], 1)
    lay = []
    pr.decoder(cfg, w, toks, layers_out=lay)
    wd = {n: t.double() for n, t in w.items()}
    x = wd["embed"][torch.tensor(toks)] * cfg["embedding"]["scale"]
    h = pr.rms(x, cfg["norm"]["eps"]) * (1 + wd["l0.norm1"])
    y = pr.latent_attention(h, wd, "l0.mix.", cfg["layers"][0]["mixer"], cfg["norm"]["eps"]) + pr.gated_feed_forward(h, wd, "l0.mlp.")
    assert torch.allclose(lay[0], x + cfg["residual_mult"] * y, atol=1e-12)

"""Zodosun: configuration, registry, the model's tensor list, the oracle's own
mechanisms against closed forms (no GPU)."""
import copy
import json
import math
import os

import pytest
import torch

import plain_zodosun as pz
from zodosun_cases import CASES, Z_A, Z_B, make_weights


def test_the_registry_finds_the_architecture_by_its_own_key():
    from tq_kv_b200.config import ZodosunConfig, resolve, spec_from_config_dict
    assert resolve(Z_A).name == "Zodosun" and resolve({"architectures": ["Zodosun"]}).name == "Zodosun"
    arch, cfg, spec = spec_from_config_dict(Z_A)
    assert isinstance(cfg, ZodosunConfig) and len(spec.layers) == 4 and spec.vocab_size == 300
    kinds = [l.mixer.kind for l in spec.layers]
    assert kinds == ["side_by_side", "delta_rule_mixer", "delta_rule_mixer", "side_by_side"]
    from zodosun_cases import Z_E
    from tq_kv_b200.engine.model import DecoderModel
    kv, state = DecoderModel(spec_from_config_dict(Z_E)[2]).cache_requests()
    assert kv == {} and sorted(state) == [0, 1]                  # a model of state mixers only caches no keys
    assert [l.feed_forward is not None for l in spec.layers] == [True, True, False, False]
    assert spec.layers[0].mixer_norm.params["groups"] == 3 and spec.final_norm.params["groups"] == 3
    assert spec.head.params["logit_scale"] == 0.75


def test_round_trip_and_optional_sizes():
    from tq_kv_b200.config import ZodosunConfig
    for cfg in CASES.values():
        c = ZodosunConfig.from_dict(cfg)
        again = ZodosunConfig.from_dict(c.to_dict())
        assert again == c
    bare = copy.deepcopy(Z_A)
    del bare["layers"][1]["mixer"]["rank"], bare["layers"][0]["mixer"]["left"]["bias_rows"]
    c = ZodosunConfig.from_dict(bare)
    assert c.layers[1].mixer.rank is None and c.layers[0].mixer.left.bias_rows is None
    assert "rank" not in c.to_dict()["layers"][1]["mixer"]


@pytest.mark.parametrize("damage, text", [
    (lambda d: d.pop("width"), "width"),
    (lambda d: d["norm"].pop("groups"), "groups"),
    (lambda d: d["norm"].update(groups=5), "equal groups"),
    (lambda d: d["layers"][0].update(type="other"), "unknown layer type"),
    (lambda d: d["layers"][0]["mixer"]["left"].update(kv_heads=4), "cannot share"),
    (lambda d: d["layers"][0]["mixer"]["right"].update(decay=[0.5]), "decays for"),
    (lambda d: d["layers"][1]["mlp"].update(kind="routed"), "unknown kind"),
    (lambda d: d["layers"][0]["mixer"]["left"].pop("q_temp"), "q_temp"),
    (lambda d: d.update(layers=[]), "empty"),
])
def test_a_damaged_configuration_is_refused_with_the_key_named(damage, text):
    from tq_kv_b200.config import ConfigError, spec_from_config_dict
    d = copy.deepcopy(Z_A)
    damage(d)
    with pytest.raises(ConfigError, match=text):
        spec_from_config_dict(d)


def test_the_models_tensor_list_is_the_designs():
    from tq_kv_b200.config import spec_from_config_dict
    from tq_kv_b200.engine.model import DecoderModel
    for cfg in CASES.values():
        specs = DecoderModel(spec_from_config_dict(cfg)[2]).weight_specs()
        w = make_weights(cfg, 1)
        assert set(specs) == set(w)
        for n, s in specs.items():
            assert tuple(s.shape) == tuple(w[n].shape), n
    # without the optional sizes the two tensors that carry them accept any
    bare = copy.deepcopy(Z_A)
    del bare["layers"][1]["mixer"]["rank"], bare["layers"][0]["mixer"]["left"]["bias_rows"]
    specs = DecoderModel(spec_from_config_dict(bare)[2]).weight_specs()
    assert tuple(specs["l1.mix.w1"].shape) == (-1, 96) and tuple(specs["l1.mix.w2"].shape) == (72, -1)
    assert tuple(specs["l0.mix.left.rel"].shape) == (-1, 6)
    req_kv, req_state = DecoderModel(spec_from_config_dict(Z_A)[2]).cache_requests()
    assert sorted(req_kv) == [0, 3] and sorted(req_state) == [0, 1, 2, 3]
    assert (req_kv[0].n_kv_heads, req_kv[0].head_dim, req_kv[0].value_dim) == (3, 16, 24)
    assert tuple(req_state[0].shape) == (3, 24, 16) and tuple(req_state[2].shape) == (2, 40, 40)


def test_a_folder_of_random_weights_is_written_and_read_back(tmp_path):
    from tq_kv_b200.weights import write_model_folder
    f = write_model_folder(Z_B, str(tmp_path / "zb"), seed=3)
    cfg, w = pz.read_folder(f)
    assert cfg["architecture"] == "Zodosun" and "architectures" not in cfg
    assert tuple(w["l1.mix.left.rel"].shape) == (20, 3) and tuple(w["l0.mix.w2"].shape) == (128, 16)
    bare = copy.deepcopy(Z_B)
    del bare["layers"][0]["mixer"]["rank"]
    with pytest.raises(ValueError, match="only a checkpoint gives"):
        write_model_folder(bare, str(tmp_path / "zb2"), seed=3)


def test_the_products_distance_rows_equal_the_oracles_buckets():
    from tq_kv_b200.parts.sigmoid_attention import distance_rows
    for rows, far in ((12, 40), (9, 100), (20, 600), (16, 30), (2, 17), (32, 128), (3, 5), (64, 1 << 14)):
        got = distance_rows(rows, far, 3000).tolist()
        assert got == [pz.distance_bucket(n, rows, far) for n in range(3000)], (rows, far)
        assert got[0] == 0 and all(b >= a for a, b in zip(got, got[1:]))
        if far > rows // 2 and far < 3000:
            assert got[far] == rows - 1 == max(got)


# ---- the oracle's mechanisms against closed forms --------------------------------------------
def test_oracle_decayed_state_is_a_weighted_sum_over_the_past():
    torch.manual_seed(0)
    T, W, c = 9, 16, {"heads": 2, "dim": 4, "vdim": 6, "decay": [0.5, 0.9]}
    w = {"q": torch.randn(8, W), "k": torch.randn(8, W), "v": torch.randn(12, W), "g": torch.randn(12, W),
         "norm": torch.ones(12), "o": torch.eye(12)}
    w = {k: v.double() for k, v in w.items()}
    h = torch.randn(T, W).double()
    got = pz.decayed_outer_sum(h, w, "", c, 1e-6)
    q, k = pz.silu(h @ w["q"].T).reshape(T, 2, 4), pz.silu(h @ w["k"].T).reshape(T, 2, 4)
    v = pz.silu(h @ w["v"].T).reshape(T, 2, 6)
    o = torch.zeros(T, 2, 6, dtype=torch.float64)
    for t in range(T):
        for s in range(t + 1):
            for hd in range(2):
                o[t, hd] += c["decay"][hd] ** (t - s) * (q[t, hd] @ k[s, hd]) * v[s, hd]
    want = pz.rms(o.reshape(T, 12), 1e-6) * torch.sigmoid(h @ w["g"].T)
    assert torch.allclose(got, want, atol=1e-12)


def test_oracle_delta_rule_without_removal_and_decay_is_plain_linear_attention():
    torch.manual_seed(1)
    T, W, c = 7, 12, {"heads": 1, "dim": 5}
    w = {n: torch.randn(5, W).double() for n in ("r", "k", "v", "g")}
    w.update({"a": torch.zeros(5, W).double(), "a.b": torch.full((5,), -80.0).double(),     # a = sigmoid(-80) = 0
              "w1": torch.zeros(3, W).double(), "w2": torch.zeros(5, 3).double(),
              "w0": torch.full((5,), -80.0).double(),                                       # w = exp(-0) = 1
              "norm": torch.ones(5).double(), "o": torch.eye(5).double()})
    h = torch.randn(T, W).double()
    got = pz.delta_rule(h, w, "", c, 1e-6)
    r, k, v = h @ w["r"].T, h @ w["k"].T, h @ w["v"].T
    o = torch.stack([sum((r[t] @ k[s]) * v[s] for s in range(t + 1)) for t in range(T)])
    want = pz.rms(o, 1e-6) * torch.sigmoid(h @ w["g"].T)
    assert torch.allclose(got, want, atol=1e-10)


def test_oracle_delta_rule_full_removal_forgets_what_lay_along_the_key():
    """With a = 1 and w = 1 a second write with the same unit key replaces the first: u^T S becomes (u.k) v_2."""
    d = 4
    k = torch.tensor([1.0, 2.0, -1.0, 0.5], dtype=torch.float64)
    u = k / torch.sqrt((k * k).sum() + 1e-6)
    S = torch.zeros(d, d, dtype=torch.float64)
    for v in (torch.arange(4.0).double(), torch.tensor([3.0, -1.0, 2.0, 7.0]).double()):
        S = S - torch.outer(u, u @ S) + torch.outer(k, v)
    assert torch.allclose(u @ S, (u @ k) * torch.tensor([3.0, -1.0, 2.0, 7.0]).double(), atol=1e-5)


def test_oracle_sigmoid_attention_sees_exactly_the_past_and_uses_the_buckets():
    cfg, w = Z_A, {n: t.double() for n, t in make_weights(Z_A, 2).items()}
    c = cfg["layers"][0]["mixer"]["left"]
    torch.manual_seed(3)
    h = torch.randn(60, cfg["width"]).double()
    full = pz.sigmoid_attention(h, w, "l0.mix.left.", c, 1e-6)
    h2 = h.clone()
    h2[41:] = torch.randn(19, cfg["width"]).double()
    assert torch.equal(pz.sigmoid_attention(h2, w, "l0.mix.left.", c, 1e-6)[:41], full[:41])     # causal
    w2 = dict(w)
    rel = w["l0.mix.left.rel"].clone()
    rel[-1] += 5.0                                     # the last row serves distances >= bias_max (and a few before)
    w2["l0.mix.left.rel"] = rel
    moved = pz.sigmoid_attention(h, w2, "l0.mix.left.", c, 1e-6)
    first = min(n for n in range(100) if pz.distance_bucket(n, 12, 40) == 11)
    assert torch.equal(moved[:first], full[:first]) and not torch.allclose(moved[first], full[first])
    assert pz.distance_bucket(39, 12, 40) == 11 - 1 or first <= 39
    assert math.isclose(pz.query_temperature(13, 0.5, 7), 1 + 0.5 * math.log(3))

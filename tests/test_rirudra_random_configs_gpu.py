"""Seeded random Rirudra configurations (sizes, head counts, layer order, constants all drawn) through the engine in
both precisions against the plain implementation: a whole prompt over several pages, its last tokens one by one, and
an unequal batch that decodes together (GPU)."""
import os
import random

import pytest
import torch

import plain_rirudra as pr
from helpers import assert_close
from rirudra_cases import make_weights, tokens

pytestmark = pytest.mark.gpu
TOL = {"float32": 3e-5, "bfloat16": 4e-2}


def _divisor(rng, n):
    return rng.choice([d for d in range(1, n + 1) if n % d == 0])


def random_config(seed: int) -> dict:
    rng = random.Random(seed)
    layers = []
    for _ in range(rng.randint(2, 5)):
        kind = rng.choice(["latent_attention", "mamba2", "delta"])
        if kind == "latent_attention":
            d, r = rng.choice([8, 16, 24, 32, 48, 64]), rng.choice([4, 8, 16, 32, 64])
            m = {"heads": rng.randint(1, 8), "dim": d, "rot_dim": r, "vdim": rng.choice([8, 16, 24, 32, 64]),
                 "q_rank": rng.choice([16, 24, 40, 64, 96]), "kv_rank": rng.choice([16, 32, 56, 96, 128, 200]),
                 "scale": (d + r) ** -0.5 * rng.choice([0.7, 1.0, 1.6]),
                 "rot": {"base": rng.choice([1e4, 1e6, 300.0]), "dims": r}}
        elif kind == "mamba2":
            heads = rng.choice([2, 3, 4, 6, 8])
            m = {"heads": heads, "vdim": rng.choice([8, 16, 24, 48, 64]), "state": rng.choice([8, 16, 32, 64]),
                 "groups": _divisor(rng, heads), "norm_groups": _divisor(rng, heads), "conv": rng.choice([2, 3, 4])}
        else:
            heads = rng.choice([2, 3, 4, 6])
            m = {"heads": heads, "kv_heads": _divisor(rng, heads), "dim": rng.choice([16, 32, 48, 64]),
                 "vdim": rng.choice([16, 32, 64, 80]), "conv": rng.choice([2, 3, 4])}
        ff = rng.choice([None, 64, 160, 256])
        layers.append({"type": kind, "mixer": m, "mlp": None if ff is None else {"kind": "dense", "ff": ff}})
    return {"architecture": "Rirudra", "vocab": rng.randint(100, 700), "width": rng.choice([64, 96, 136, 192, 256]),
            "embedding": {"scale": rng.choice([1.0, 5.0, 12.0])}, "residual_mult": rng.choice([0.2, 0.3, 0.7, 1.0]),
            "norm": {"eps": rng.choice([1e-5, 1e-6])}, "layers": layers}


@pytest.fixture(scope="module")
def tmp_root(tmp_path_factory):
    return tmp_path_factory.mktemp("rirudra_random")


@pytest.mark.parametrize("seed", list(range(10)))
def test_a_random_configuration_whole_decoded_and_batched(tmp_root, seed):
    from tq_kv_b200.engine import Engine, StepRow
    cfg = random_config(seed)
    path = pr.write_folder(os.path.join(str(tmp_root), f"m{seed}"), cfg, make_weights(cfg, seed))
    w = pr.read_folder(path)[1]
    V = cfg["vocab"]
    long_, short, mid = tokens(330, V, seed), tokens(40, V, seed + 100), tokens(139, V, seed + 200)
    want = {id(t): pr.decoder(cfg, w, t) for t in (long_, short, mid)}
    for dtype in ("float32", "bfloat16"):
        eng = Engine.from_folder(path, dtype=dtype, max_tokens=1024)
        what = f"random {seed} {[l['type'] for l in cfg['layers']]} {dtype}"
        s = eng.new_sequence()
        got = [eng.step([StepRow(s, long_[:290], list(range(290)))])]
        got += [eng.step([StepRow(s, [t], [0])]) for t in long_[290:]]
        assert_close(torch.cat(got), want[id(long_)].float(), dtype, what + " whole and decoded", tol=TOL[dtype])
        eng.release(s)
        reqs, cut = [short, mid, long_[:200]], [30, 129, 190]
        slots = [eng.new_sequence() for _ in reqs]
        out = eng.step([StepRow(sl, r[:c], [c - 1]) for sl, r, c in zip(slots, reqs, cut)])
        got = [[out[i:i + 1]] for i in range(3)]
        for step in range(10):
            out = eng.step([StepRow(sl, [r[c + step]], [0]) for sl, r, c in zip(slots, reqs, cut)])
            for i in range(3):
                got[i].append(out[i:i + 1])
        for i, (r, c) in enumerate(zip(reqs, cut)):
            ref = want[id(long_)] if r is not short and r is not mid else want[id(r)]
            assert_close(torch.cat(got[i]), ref[c - 1:c + 10].float(), dtype, what + f" batch row {i}", tol=TOL[dtype])

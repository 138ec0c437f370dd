"""Rirudra through the engine against the plain implementation: whole prompts, token-by-token decoding, prompts in
portions, unequal batches, slots and pages used again, long decoding, a sharp softmax whose rows hang on single keys,
generation through the entry points (GPU)."""
import json
import os
import subprocess
import sys

import pytest
import torch

import plain_rirudra as pr
from helpers import assert_close
from rirudra_cases import CASES, folder, oracle_logits, tokens

pytestmark = pytest.mark.gpu
ROOT = os.path.join(os.path.dirname(os.path.abspath(__file__)), "..")
# max |difference| relative to the oracle's largest logit: the package's float32 bound, and in bfloat16 about twice
# the largest error seen
TOL = {"float32": 3e-5, "bfloat16": 4e-2}
# The sharp model's scores are large, and bfloat16 rounds what they are made of: its rows move by a tenth of the
# largest logit at most, while a lost key moves them by all of it; float32 keeps the tight bound.
SHARP_BF16 = 0.1


@pytest.fixture(scope="module")
def tmp_root(tmp_path_factory):
    return tmp_path_factory.mktemp("rirudra")


def _engine(path, dtype, **kw):
    from tq_kv_b200.engine import Engine
    kw.setdefault("max_tokens", 1024)
    return Engine.from_folder(path, dtype=dtype, **kw)


def _check(got, want, dtype, what):
    tol = SHARP_BF16 if dtype == "bfloat16" and (what.startswith("p ") or what.startswith("sharp")) else TOL[dtype]
    assert_close(got, want.float(), dtype, "rirudra " + what, tol=tol)


@pytest.mark.parametrize("name", sorted(CASES))
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_whole_prompts_and_decoding_token_by_token(tmp_root, name, dtype):
    from tq_kv_b200.engine import StepRow
    path = folder(tmp_root, name)
    eng = _engine(path, dtype)
    V = CASES[name]["vocab"]
    for n in (1, 2, 3, 70, 200):                             # the first tokens alone; over one and three pages
        toks = tokens(n, V, 10 + n)
        want = oracle_logits(path, toks)
        s = eng.new_sequence()
        _check(eng.step([StepRow(s, toks, list(range(n)))]), want, dtype, f"{name} whole {n}")
        eng.release(s)
    toks = tokens(200, V, 210)
    want = oracle_logits(path, toks)
    s = eng.new_sequence()
    got = [eng.step([StepRow(s, toks[:150], [149])])]
    for t in range(150, 200):                                # replayed graphs from the second step on
        got.append(eng.step([StepRow(s, [toks[t]], [0])]))
    _check(torch.cat(got), want[149:], dtype, f"{name} decode")
    eng.release(s)
    assert eng.cache.free_slots == eng.cache.max_slots
    eng.cache.book.check()


@pytest.mark.parametrize("name", sorted(CASES))
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_prompts_in_portions(tmp_root, name, dtype):
    """Portions down to one and two tokens: shorter than the convolutions' memory, across a page's edge."""
    from tq_kv_b200.engine import StepRow
    path = folder(tmp_root, name)
    eng = _engine(path, dtype)
    toks = tokens(180, CASES[name]["vocab"], 77)
    want = oracle_logits(path, toks)
    for cuts in ((2, 2, 60, 1, 63, 52), (64, 64, 52), (1, 1, 1, 2, 175), (127, 2, 51), (3, 61, 116)):
        assert sum(cuts) == 180
        s, at, got = eng.new_sequence(), 0, []
        for n in cuts:
            got.append(eng.step([StepRow(s, toks[at:at + n], list(range(n)))]))
            at += n
        _check(torch.cat(got), want, dtype, f"{name} portions {cuts}")
        eng.release(s)


@pytest.mark.parametrize("name", sorted(CASES))
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_unequal_batches_against_each_alone_and_slots_used_again(tmp_root, name, dtype):
    from tq_kv_b200.engine import StepRow
    path = folder(tmp_root, name)
    eng = _engine(path, dtype, max_tokens=640, max_slots=4)
    V = CASES[name]["vocab"]
    for round_ in range(3):                                  # the same slots and pages serve three batches
        lens = [(1, 130, 66), (64, 2, 100), (129, 65, 1)][round_]
        extra = [12, 30, 20]                                 # tokens decoded after the prompt; rows end at different steps
        reqs = [tokens(n + m, V, 100 * round_ + n) for n, m in zip(lens, extra)]
        wants = [oracle_logits(path, r) for r in reqs]
        slots = [eng.new_sequence() for _ in reqs]
        got = [[] for _ in reqs]
        out = eng.step([StepRow(s, r[:n], [n - 1]) for s, r, n in zip(slots, reqs, lens)])
        for i in range(3):
            got[i].append(out[i:i + 1])
        live = [0, 1, 2]
        for step in range(max(extra)):
            live = [i for i in live if step < extra[i]]
            out = eng.step([StepRow(slots[i], [reqs[i][lens[i] + step]], [0]) for i in live])
            for j, i in enumerate(live):
                got[i].append(out[j:j + 1])
            for i in list(live):
                if step + 1 == extra[i]:
                    eng.release(slots[i])                    # its slot, pages and state go back while the others go on
        for i in range(3):
            _check(torch.cat(got[i]), wants[i][lens[i] - 1:], dtype, f"{name} batch round {round_} row {i}")
        assert eng.cache.free_slots == 4
        eng.cache.book.check()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_new_prompt_beside_decoding_rows_and_a_long_decode(tmp_root, dtype):
    """A prompt joins rows that decode (through the paged path), and 300 tokens are decoded one by one."""
    from tq_kv_b200.engine import StepRow
    path = folder(tmp_root, "a")
    eng = _engine(path, dtype)
    a, b = tokens(330, 300, 1), tokens(90, 300, 2)
    wa, wb = oracle_logits(path, a), oracle_logits(path, b)
    sa, sb = eng.new_sequence(), eng.new_sequence()
    got_a = [eng.step([StepRow(sa, a[:30], [29])])]
    out = eng.step([StepRow(sa, [a[30]], [0]), StepRow(sb, b[:70], [0, 69])])
    got_a.append(out[:1])
    got_b = [out[1:]]
    for t in range(31, 330):
        rows = [StepRow(sa, [a[t]], [0])]
        if 70 + (t - 31) < 90:
            rows.append(StepRow(sb, [b[70 + t - 31]], [0]))
        out = eng.step(rows)
        got_a.append(out[:1])
        if len(rows) == 2:
            got_b.append(out[1:])
    _check(torch.cat(got_a), wa[29:], dtype, "long decode")
    _check(torch.cat(got_b), torch.cat([wb[:1], wb[69:]]), dtype, "prompt beside decoding rows")


def test_a_residual_factor_of_zero_and_of_one(tmp_root):
    """Factors that cannot, or need not, be folded into the stream: 0 (the layers add nothing; the block scales the
    sum itself) and 1."""
    from tq_kv_b200.engine import StepRow
    from rirudra_cases import make_weights
    for m in (0.0, 1.0):
        cfg = dict(CASES["a"], residual_mult=m)
        path = pr.write_folder(os.path.join(str(tmp_root), f"factor_{m}"), cfg, make_weights(cfg, 2))
        toks = tokens(70, cfg["vocab"], 3)
        want = pr.decoder(cfg, pr.read_folder(path)[1], toks)
        eng = _engine(path, "float32")
        s = eng.new_sequence()
        got = [eng.step([StepRow(s, toks[:60], list(range(60)))])]
        got += [eng.step([StepRow(s, [t], [0])]) for t in toks[60:]]
        _check(torch.cat(got), want, "float32", f"residual factor {m}")


def _deciding_keys(path, toks):
    """For the one-layer sharp model: per position and head the key with the largest softmax weight, and that weight
    (from the plain implementation's own formulas)."""
    cfg, w = pr.read_folder(path)
    w = {n: t.double() for n, t in w.items()}
    c, eps = cfg["layers"][0]["mixer"], cfg["norm"]["eps"]
    x = w["embed"][torch.tensor(toks)] * cfg["embedding"]["scale"]
    h = pr.offset_norm(x, w["l0.norm1"], eps)
    H, d, r, n = c["heads"], c["dim"], c["rot_dim"], c["kv_rank"]
    T = len(toks)
    pos = torch.arange(T)
    q = ((pr.rms(h @ w["l0.mix.dq"].T, eps) * w["l0.mix.dq.norm"]) @ w["l0.mix.uq"].T).reshape(T, H, d + r)
    kv = h @ w["l0.mix.dkv"].T
    lat = pr.rms(kv[:, :n], eps) * w["l0.mix.dkv.norm"]
    k_rot = pr.rotate_pairs(kv[:, n:], pos, c["rot"]["dims"], c["rot"]["base"])
    q_rot = pr.rotate_pairs(q[:, :, d:], pos, c["rot"]["dims"], c["rot"]["base"])
    k_flat = (lat @ w["l0.mix.uk"].T).reshape(T, H, d)
    best, weight = [], []
    for head in range(H):
        s = (q[:, head, :d] @ k_flat[:, head].T + q_rot[:, head] @ k_rot.T) * c["scale"]
        s = s.masked_fill(torch.triu(torch.ones(T, T, dtype=torch.bool), 1), float("-inf"))
        p = torch.softmax(s, -1)
        weight.append(p.max(-1).values)
        best.append(p.argmax(-1))
    return torch.stack(best, 1), torch.stack(weight, 1)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_rows_that_hang_on_single_keys_far_back_and_at_page_edges(tmp_root, dtype):
    """The sharp model: most rows give nearly all their weight to one key.  The test first makes sure that such
    keys lie far back (hundreds of tokens), at position 0, and on both sides of page edges, then runs the prompt
    whole, in portions and decoded token by token: a kernel that loses one key is off by the size of the logits."""
    from tq_kv_b200.engine import StepRow
    path = folder(tmp_root, "p")
    toks = tokens(700, 150, 9)
    best, weight = _deciding_keys(path, toks)
    sharp = weight > 0.9
    dist = (torch.arange(700).unsqueeze(1) - best)[sharp]
    keys = best[sharp]
    assert sharp.float().mean() > 0.3 and (dist > 300).sum() >= 5 and (keys == 0).any()
    assert any(((keys % 64) == e).any() for e in (63,)) and ((keys % 64) == 0).sum() > 1
    want = oracle_logits(path, toks)
    eng = _engine(path, dtype)
    s = eng.new_sequence()
    _check(eng.step([StepRow(s, toks, list(range(700)))]), want, dtype, "sharp whole")
    eng.release(s)
    s, at, got = eng.new_sequence(), 0, []
    for n in (64, 1, 63, 2, 190, 320, 60):
        got.append(eng.step([StepRow(s, toks[at:at + n], list(range(n)))]))
        at += n
    _check(torch.cat(got), want, dtype, "sharp portions")
    eng.release(s)
    s = eng.new_sequence()
    got = [eng.step([StepRow(s, toks[:500], [499])])]
    for t in range(500, 700):
        got.append(eng.step([StepRow(s, [toks[t]], [0])]))
    _check(torch.cat(got), want[499:], dtype, "sharp decode")
    far_decoded = ((torch.arange(700).unsqueeze(1) - best) > 300) & sharp
    assert far_decoded[500:].any()                          # decoded rows, too, hang on keys far back


def test_greedy_generation_through_the_entry_point_and_the_command_line(tmp_root):
    import tq_kv_b200 as tq
    path = folder(tmp_root, "c")
    cfg, w = pr.read_folder(path)
    prompts = [tokens(n, 130, 300 + n) for n in (3, 20, 9)]
    want = [pr.greedy(cfg, w, p, 10) for p in prompts]
    eng = tq.load(path, dtype="float32", max_batch=2, max_context=128)      # three requests, two slots
    res = eng.generate(prompts, tq.GenerationParams.greedy(10, stop_token_ids=()))
    assert [r.tokens for r in res] == want and all(r.finish_reason == "length" for r in res)
    assert eng.cache.free_slots == 2
    env = dict(os.environ, PYTHONPATH=ROOT)
    p = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "tq"), "run", path, "--dtype", "float32",
                        "--prompt-ids", ",".join(map(str, prompts[1])), "-n", "10", "--temperature", "0",
                        "--repeat-penalty", "1.0", "--max-context", "128"], capture_output=True, text=True, env=env, timeout=600)
    assert p.returncode == 0, p.stderr[-2000:]
    assert [int(t) for t in p.stdout.strip().splitlines()[-1].split(",")] == want[1]


def test_trace_replay_as_a_program(tmp_root, tmp_path):
    import numpy as np
    path = folder(tmp_root, "b")
    a, b = tokens(100, 1000, 5), tokens(40, 1000, 6)
    wa, wb = oracle_logits(path, a), oracle_logits(path, b)
    steps = [{"step": 0, "entries": [{"id": "x", "tokens": a[:90], "want": [0, 89]}, {"id": "y", "tokens": b[:38], "want": [37]}],
              "end": []}]
    for i in range(10):
        e = [{"id": "x", "tokens": [a[90 + i]], "want": [0]}]
        if i < 2:
            e.append({"id": "y", "tokens": [b[38 + i]], "want": [0] if i else []})
        steps.append({"step": i + 1, "entries": e, "end": ["y"] if i == 1 else (["x"] if i == 9 else [])})
    out = tmp_path / "out"
    p = subprocess.run([os.path.join(ROOT, "bin", "trace_run"), "--model", path, "--dtype", "float32", "--out", str(out),
                        "--max-tokens", "256"], input="\n".join(json.dumps(s) for s in steps) + "\n",
                       capture_output=True, text=True, timeout=900)
    assert p.returncode == 0, p.stderr[-2000:]
    assert [l for l in p.stdout.splitlines() if l.startswith("done")] == [f"done {i}" for i in range(11)]
    first = torch.from_numpy(np.fromfile(out / "0.f32", dtype="<f4").reshape(3, 1000).copy())
    _check(first, torch.stack([wa[0], wa[89], wb[37]]), "float32", "trace step 0")
    last = torch.from_numpy(np.fromfile(out / "10.f32", dtype="<f4").reshape(1, 1000).copy())
    _check(last, wa[99:100], "float32", "trace last step")
    two = torch.from_numpy(np.fromfile(out / "2.f32", dtype="<f4").reshape(2, 1000).copy())
    _check(two, torch.stack([wa[91], wb[39]]), "float32", "trace step 2")


def test_random_weights_from_a_named_shape(tmp_path):
    """`rirudra-tiny` with random weights: the engine made on the device and the folder written on the host hold the
    same weights, and the oracle agrees with both."""
    import tq_kv_b200 as tq
    from tq_kv_b200.config import named_shape
    from tq_kv_b200.weights import write_model_folder
    cfg = named_shape("rirudra-tiny")
    path = write_model_folder(cfg, str(tmp_path / "m"), 3)
    toks = tokens(40, cfg["vocab"], 4)
    want = oracle_logits(path, toks)
    from tq_kv_b200.engine import Engine, StepRow
    for eng in (Engine.from_random(cfg, 3, dtype="float32", max_tokens=256),
                Engine.from_folder(path, dtype="float32", max_tokens=256)):
        s = eng.new_sequence()
        _check(eng.step([StepRow(s, toks, list(range(40)))]), want, "float32", "named shape, random weights")

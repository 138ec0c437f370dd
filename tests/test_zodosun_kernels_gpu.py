"""The kernels of the state mixers, the sigmoid attention and the grouped norm, each alone against a float64
computation of the same formula at several sizes (GPU)."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _close(got, want, tol, what=""):
    got, want = got.double().cpu(), want.double().cpu()
    err = (got - want).abs().max().item()
    ref = want.abs().max().item()
    assert math.isfinite(err) and err <= tol * max(ref, 1e-30), f"{what}: {err:.3e} of {ref:.3e} > {tol:.1e}"


def _i32(x):
    return torch.tensor(x, dtype=torch.int32, device=DEV)


@pytest.mark.parametrize("width", [6, 7, 96, 1030])
def test_embedding_with_sinusoidal_positions(width):
    from tq_kv_b200 import kernels
    torch.manual_seed(width)
    V, T = 50, 40
    table = torch.randn(V, width, device=DEV).to(torch.bfloat16)
    toks = torch.randint(0, V, (T,), device=DEV, dtype=torch.int32)
    pos = torch.randint(0, 5000, (T,), device=DEV, dtype=torch.int32)
    pos[0], pos[1] = 0, 1
    i = torch.arange((width + 1) // 2, dtype=torch.float64, device=DEV)
    rate = torch.pow(torch.tensor(10000.0, dtype=torch.float64, device=DEV), -2.0 * i / width)
    out = torch.empty(T, width, dtype=torch.float32, device=DEV)
    kernels.embed_sinusoid(toks, pos, table, rate.float(), out)
    ang = pos.double().unsqueeze(1) * rate.unsqueeze(0)
    pe = torch.stack([torch.sin(ang), torch.cos(ang)], dim=2).reshape(T, -1)[:, :width]
    want = table[toks.long()].double() + pe
    assert (out.double() - want).abs().max().item() < 2e-3          # float32 angles up to 5,000 rad
    assert (out[:2].double() - want[:2]).abs().max().item() < 1e-6  # small angles: exact to rounding


@pytest.mark.parametrize("width, groups", [(96, 3), (84, 4), (128, 1), (120, 120), (4096, 2)])
@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16])
def test_grouped_norm_with_gate_rows_and_strides(width, groups, out_dtype):
    from tq_kv_b200 import kernels
    torch.manual_seed(groups)
    T, eps = 9, 1e-5
    wide = torch.randn(T, 3 * width + 5, device=DEV) * 3
    x, gate = wide[:, 2:2 + width], wide[:, width + 3:2 * width + 3]        # slices of a wider buffer
    w = torch.randn(width, device=DEV)
    tol = 1e-5 if out_dtype == torch.float32 else 1e-2

    def ref(x, gate=None):
        p = x.double().reshape(x.shape[0], groups, -1)
        y = (p / torch.sqrt((p * p).mean(-1, keepdim=True) + eps)).reshape(x.shape[0], width) * w.double()
        return y if gate is None else y * torch.sigmoid(gate.double())

    out = torch.empty(T, width, dtype=out_dtype, device=DEV)
    _close(kernels.group_rmsnorm(x, w, eps, out, groups=groups), ref(x), tol, "plain")
    _close(kernels.group_rmsnorm(x, w, eps, out, groups=groups, gate=gate), ref(x, gate), tol, "gated")
    rows = _i32([7, 0, 7, 3])
    out4 = torch.empty(4, width, dtype=out_dtype, device=DEV)
    _close(kernels.group_rmsnorm(x, w, eps, out4, groups=groups, rows=rows), ref(x)[rows.long()], tol, "rows")


def test_normed_sum_tanh_and_scale():
    from tq_kv_b200 import kernels
    torch.manual_seed(0)
    T, W, eps = 11, 84, 1e-6
    acc = torch.randn(T, W, device=DEV)
    srcs = [(torch.randn(T, W, device=DEV) * (k + 1), torch.randn(W, device=DEV)) for k in range(3)]
    for n in (1, 2, 3):
        a = acc.clone()
        kernels.add_normed(a, srcs[:n], eps, 0.5)
        want = acc.double() + 0.5 * sum(
            x.double() / torch.sqrt((x.double() ** 2).mean(-1, keepdim=True) + eps) * w.double() for x, w in srcs[:n])
        _close(a, want, 1e-5, f"{n} sources")
    wide = torch.randn(T, 40, device=DEV) * 2
    for dt, tol in ((torch.float32, 1e-6), (torch.bfloat16, 1e-2)):
        out = torch.empty(T, 13, dtype=dt, device=DEV)
        _close(kernels.tanh_rows(wide[:, 20:33], out), torch.tanh(wide[:, 20:33].double()), tol, "tanh")
    x = torch.randn(7, 33, device=DEV)
    _close(kernels.scale_inplace(x.clone(), 0.3), x.double() * 0.3, 1e-6, "scale")


# ---- the scan ----------------------------------------------------------------------------------
def _scan_reference(mode, proj, offs, H, d, e, state0, bounds, decay=None, decay_logit=None, silu=False):
    """float64: per sequence [a, b) and head, token by token."""
    p = proj.double().cpu()
    out = torch.zeros(p.shape[0], H * e, dtype=torch.float64)
    states = []
    act = (lambda z: z * torch.sigmoid(z)) if silu else (lambda z: z)
    for (a, b), S0 in zip(bounds, state0):
        S = S0.double().cpu().clone()
        for t in range(a, b):
            for h in range(H):
                q = act(p[t, offs["q"] + h * d: offs["q"] + (h + 1) * d])
                k = act(p[t, offs["k"] + h * d: offs["k"] + (h + 1) * d])
                v = act(p[t, offs["v"] + h * e: offs["v"] + (h + 1) * e])
                if mode == "decay":
                    S[h] = decay[h] * S[h] + torch.outer(k, v)
                else:
                    lw = decay_logit.double().cpu()[t, h * d:(h + 1) * d]
                    w = torch.exp(-math.exp(-0.5) * torch.sigmoid(lw))
                    r = torch.sigmoid(p[t, offs["a"] + h * d: offs["a"] + (h + 1) * d])
                    u = k / torch.sqrt((k * k).sum() + 1e-6)
                    S[h] = w.unsqueeze(1) * S[h] - torch.outer(r * u, u @ S[h]) + torch.outer(k, v)
                out[t, h * e:(h + 1) * e] = S[h].T @ q
        states.append(S)
    return out, states


@pytest.mark.parametrize("H, d, e", [(3, 8, 48), (2, 24, 16), (1, 32, 32), (2, 40, 40), (1, 64, 130), (1, 100, 20),
                                     (1, 128, 64), (1, 160, 33), (1, 256, 16), (3, 10, 6), (1, 30, 7), (2, 1, 1)])
def test_scan_with_constant_decay(H, d, e):
    from tq_kv_b200 import kernels
    torch.manual_seed(d + e)
    lens = [17, 1, 33, 16]
    T, ld = sum(lens), 2 * H * d + H * e + 7
    offs = {"q": 3, "k": 3 + H * d, "v": 5 + 2 * H * d}
    proj = torch.randn(T, ld, device=DEV)
    decay = [0.5, 0.95, 1.0][:H]
    slots = [5, 2, 7, 0]
    state = torch.randn(8, H, d, e, device=DEV)
    before = state.clone()
    cu = [0]
    for n in lens:
        cu.append(cu[-1] + n)
    out = torch.full((T, H * e), float("nan"), device=DEV)
    given = proj.clone()
    for silu in (True, False):
        state.copy_(before)
        proj = given.clone()                                    # the kernels work in place
        kernels.linear_scan(proj, state, _i32(cu), _i32(slots), out, n_seqs=4, heads=H, key_dim=d, value_dim=e,
                            off_q=offs["q"], off_k=offs["k"], off_v=offs["v"],
                            head_decay=torch.tensor(decay, device=DEV), silu=silu)
        want, st = _scan_reference("decay", given, offs, H, d, e, [before[s] for s in slots],
                                   list(zip(cu, cu[1:])), decay=decay, silu=silu)
        _close(out, want, 2e-5, f"outputs silu={silu}")
        for s, S in zip(slots, st):
            _close(state[s], S, 2e-5, f"state of slot {s}")
        for s in (1, 3, 4, 6):
            assert torch.equal(state[s], before[s])                  # slots of no sequence are not touched


@pytest.mark.parametrize("H, d", [(5, 12), (3, 24), (2, 32), (2, 40), (1, 64), (1, 128), (1, 160), (1, 256), (3, 10),
                                  (2, 30), (2, 1)])
def test_scan_with_the_delta_rule(H, d):
    from tq_kv_b200 import kernels
    torch.manual_seed(d)
    lens = [15, 2, 1, 40]
    T, n = sum(lens), H * d
    ld = 5 * n + 9
    offs = {"q": 0, "k": n, "v": 2 * n, "a": 4 * n}
    proj = torch.randn(T, ld, device=DEV)
    decay_logit = torch.randn(T, n, device=DEV) * 2
    slots = [1, 4, 0, 2]
    state = torch.randn(5, H, d, d, device=DEV) * 0.5
    before = state.clone()
    cu = [0]
    for m in lens:
        cu.append(cu[-1] + m)
    out = torch.full((T, n), float("nan"), device=DEV)
    kernels.linear_scan(proj.clone(), state, _i32(cu), _i32(slots), out, n_seqs=4, heads=H, key_dim=d, value_dim=d,
                        off_q=0, off_k=n, off_v=2 * n, off_a=4 * n, decay_logit=decay_logit.clone())      # (in place)
    want, st = _scan_reference("delta", proj, offs, H, d, d, [before[s] for s in slots], list(zip(cu, cu[1:])),
                               decay_logit=decay_logit)
    _close(out, want, 5e-5, "outputs")
    for s, S in zip(slots, st):
        _close(state[s], S, 5e-5, f"state of slot {s}")
    assert torch.equal(state[3], before[3])


def test_scan_in_portions_equals_scan_at_once():
    """One sequence of 70 tokens at once, and in portions of 1, 2, 16, 17, 31 and 3 tokens through the state."""
    from tq_kv_b200 import kernels
    torch.manual_seed(7)
    H, d, T = 2, 24, 70
    n = H * d
    proj = torch.randn(T, 5 * n, device=DEV)
    logit = torch.randn(T, n, device=DEV)
    for mode in ("delta", "decay"):
        kw = dict(n_seqs=1, heads=H, key_dim=d, value_dim=d, off_q=0, off_k=n, off_v=2 * n)
        kw.update(dict(off_a=4 * n) if mode == "delta" else dict(head_decay=torch.tensor([0.9, 0.99], device=DEV), silu=True))
        whole, s1 = torch.empty(T, n, device=DEV), torch.zeros(3, H, d, d, device=DEV)
        kernels.linear_scan(proj.clone(), s1, _i32([0, T]), _i32([1]), whole,
                            **kw, **(dict(decay_logit=logit.clone()) if mode == "delta" else {}))
        parts, s2, at = torch.empty(T, n, device=DEV), torch.zeros(3, H, d, d, device=DEV), 0
        for m in (1, 2, 16, 17, 31, 3):
            kernels.linear_scan(proj[at:at + m].clone(), s2, _i32([0, m]), _i32([2]), parts[at:at + m],
                                single_tokens=m == 1,
                                **kw, **(dict(decay_logit=logit[at:at + m].clone()) if mode == "delta" else {}))
            at += m
        assert at == T
        _close(parts, whole, 1e-6, mode)
        _close(s2[2], s1[1], 1e-6, mode + " state")


# ---- sigmoid attention ---------------------------------------------------------------------------
def _attention_reference(q, k, v, H, G, dk, dv, scale, bias, gate, pos0=0):
    """float64, one sequence whose keys are k[0:], queries at positions pos0 .. pos0 + len(q) - 1."""
    q, k, v = q.double().cpu(), k.double().cpu(), v.double().cpu()
    T = q.shape[0]
    out = torch.zeros(T, H * dv, dtype=torch.float64)
    for t in range(T):
        i = pos0 + t
        for h in range(H):
            g = h // (H // G)
            s = (k[: i + 1, g * dk:(g + 1) * dk] @ q[t, h * dk:(h + 1) * dk]) * scale
            if bias is not None:
                n = torch.arange(i, -1, -1).clamp(max=bias.shape[1] - 1)
                s = s + bias.double().cpu()[h, n]
            o = torch.sigmoid(s) @ v[: i + 1, g * dv:(g + 1) * dv]
            if gate is not None:
                o = o * torch.sigmoid(gate.double().cpu()[t, h])
            out[t, h * dv:(h + 1) * dv] = o
    return out


def _pages(k, v, G, dk, dv, page_tokens, order):
    """Keys and values of one sequence laid into pages in the physical order `order`."""
    T = k.shape[0]
    n_pages = max(order) + 1
    kp = torch.zeros(n_pages, G, page_tokens, dk, dtype=k.dtype, device=DEV)
    vp = torch.zeros(n_pages, G, page_tokens, dv, dtype=k.dtype, device=DEV)
    for t in range(T):
        kp[order[t // page_tokens], :, t % page_tokens] = k[t].reshape(G, dk)
        vp[order[t // page_tokens], :, t % page_tokens] = v[t].reshape(G, dv)
    return kp, vp


@pytest.mark.parametrize("H, G, dk, dv", [(6, 3, 16, 24), (3, 1, 48, 40), (4, 4, 20, 12), (2, 2, 64, 64), (8, 2, 128, 128),
                                         (1, 1, 6, 256)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_sigmoid_attention_packed_and_paged_with_splits(H, G, dk, dv, dtype):
    from tq_kv_b200 import kernels
    torch.manual_seed(dk * dv)
    T, scale, n_dist = 150, 0.3 / math.sqrt(dk), 41
    q = torch.randn(T, H * dk, device=DEV).to(dtype)
    k = torch.randn(T, G * dk, device=DEV).to(dtype)
    v = torch.randn(T, G * dv, device=DEV).to(dtype)
    v[3] *= 30                                                   # a far key that matters
    bias = torch.randn(H, n_dist, device=DEV) * 2 - 1
    gate = torch.randn(T, H + 3, device=DEV)[:, 2:2 + H]
    want = _attention_reference(q, k, v, H, G, dk, dv, scale, bias, gate)
    tol = 2e-5 if dtype == torch.float32 else 2e-2
    pos = torch.arange(T, dtype=torch.int32, device=DEV)
    seq = torch.zeros(T, dtype=torch.int32, device=DEV)
    common = dict(n_heads=H, n_kv_heads=G, key_dim=dk, value_dim=dv, scale=scale, tok_pos=pos, tok_seq=seq,
                  cu_seqlens=_i32([0, T]), start_pos=_i32([0]), bias=bias, gate=gate)
    out = torch.empty(T, H * dv, dtype=dtype, device=DEV)
    _close(kernels.sigmoid_attention(q, out, k_packed=k, v_packed=v, **common), want, tol, "packed")
    order = [2, 0, 3]
    kp, vp = _pages(k, v, G, dk, dv, 64, order)
    table = _i32(order)
    for n_splits in (1, 3):
        scratch = torch.empty(T * H * n_splits * dv, device=DEV) if n_splits > 1 else None
        out.fill_(float("nan"))
        kernels.sigmoid_attention(q, out, k_pages=kp, v_pages=vp, block_table=table, table_width=3, page_tokens=64,
                                  n_splits=n_splits, scratch=scratch, **common)
        _close(out, want, tol, f"paged, {n_splits} splits")
    # the last tokens alone, as decoding does: queries at positions 140.. over the cached keys
    tail = slice(140, T)
    common.update(tok_pos=pos[tail].contiguous(), tok_seq=seq[tail].contiguous(), cu_seqlens=_i32([0, 10]),
                  start_pos=_i32([140]), gate=gate[tail])
    out10 = torch.empty(10, H * dv, dtype=dtype, device=DEV)
    kernels.sigmoid_attention(q[tail].contiguous(), out10, k_pages=kp, v_pages=vp, block_table=table, table_width=3,
                              page_tokens=64, **common)
    _close(out10, want[tail], tol, "continuation")


@pytest.mark.parametrize("key_at", [0, 1, 63, 64, 65, 127, 128, 600])
def test_one_decisive_key_wherever_it_stands(key_at):
    """Every score is about -14 except the planted key's, which is +14: the output is that key's value, if and only
    if the kernel sees the key — the first token, both sides of a page's edge, far back among 700."""
    from tq_kv_b200 import kernels
    torch.manual_seed(key_at)
    T, H, G, dk, dv = 700, 2, 1, 32, 16
    k = torch.randn(T, dk, device=DEV) * 0.01
    direction = torch.zeros(dk, device=DEV)
    direction[5] = 1.0
    k[key_at] = direction * 28.0
    v = torch.randn(T, dv, device=DEV)
    q = direction.repeat(1, H).repeat(2, 1).contiguous()            # two queries: at the key itself, and the last token
    bias = torch.full((H, 1), -14.0, device=DEV)
    pos = _i32([key_at, T - 1])
    kp, vp = _pages(k, v, G, dk, dv, 64, list(range(11)))
    out = torch.empty(2, H * dv, device=DEV)
    kernels.sigmoid_attention(q, out, n_heads=H, n_kv_heads=G, key_dim=dk, value_dim=dv, scale=1.0, tok_pos=pos,
                              tok_seq=_i32([0, 0]), cu_seqlens=_i32([0, 2]), start_pos=_i32([0]), bias=bias, k_pages=kp,
                              v_pages=vp, block_table=_i32(list(range(11))), table_width=11, page_tokens=64, n_splits=4,
                              scratch=torch.empty(2 * H * 4 * dv, device=DEV))
    for row in (0, 1):
        for h in range(H):
            assert (out[row, h * dv:(h + 1) * dv] - v[key_at]).abs().max().item() < 5e-3
    # the query one place before the key must not see it
    if key_at > 0:
        kernels.sigmoid_attention(q[:1].contiguous(), out[:1], n_heads=H, n_kv_heads=G, key_dim=dk, value_dim=dv,
                                  scale=1.0, tok_pos=_i32([key_at - 1]), tok_seq=_i32([0]), cu_seqlens=_i32([0, 1]),
                                  start_pos=_i32([0]), bias=bias, k_pages=kp, v_pages=vp,
                                  block_table=_i32(list(range(11))), table_width=11, page_tokens=64)
        assert out[0].abs().max().item() < 5e-3


def test_distance_table_edges_decide():
    """A bias table that is -20 everywhere except at one distance: only the key at that distance counts, also at
    the table's last entry, which serves every larger distance."""
    from tq_kv_b200 import kernels
    T, dk, dv, n_dist = 90, 8, 8, 33
    q = torch.zeros(T, dk, device=DEV)
    k = torch.zeros(T, dk, device=DEV)
    v = torch.arange(T, device=DEV, dtype=torch.float32).reshape(T, 1).repeat(1, dv) + 1
    pos = torch.arange(T, dtype=torch.int32, device=DEV)
    seq = torch.zeros(T, dtype=torch.int32, device=DEV)
    for open_at in (0, 1, 31, 32):
        bias = torch.full((1, n_dist), -40.0, device=DEV)
        bias[0, open_at] = 40.0
        out = torch.empty(T, dv, device=DEV)
        kernels.sigmoid_attention(q, out, k_packed=k, v_packed=v, n_heads=1, n_kv_heads=1, key_dim=dk, value_dim=dv,
                                  scale=1.0, tok_pos=pos, tok_seq=seq, cu_seqlens=_i32([0, T]), start_pos=_i32([0]),
                                  bias=bias)
        for i in (0, 1, 31, 32, 33, 50, 89):
            if open_at < n_dist - 1:
                want = float(i - open_at + 1) if i >= open_at else 0.0
            else:                                   # the last entry: every key at distance >= 32
                want = float(sum(j + 1 for j in range(0, i - open_at + 1)))
            assert abs(out[i, 0].item() - want) < 1e-3 * max(1.0, want), (open_at, i, out[i, 0].item(), want)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_row_norm_temperature_and_cache_append(dtype):
    from tq_kv_b200 import kernels
    torch.manual_seed(2)
    H, G, dk, dv, eps, coef, every = 3, 1, 12, 20, 1e-5, 0.7, 5
    lens, starts = [70, 3], [0, 62]                      # the second row crosses a page's edge at 64
    T = sum(lens)
    nq, nk, nv = H * dk, G * dk, G * dv
    x = torch.randn(T, nq + nk + nv + H, device=DEV) * 2
    wq, wk = torch.randn(nq, device=DEV), torch.randn(nk, device=DEV)
    pos = _i32(list(range(70)) + [62, 63, 64])
    seq = _i32([0] * 70 + [1] * 3)
    new_lens = _i32([70, 65])
    table = _i32([4, 1, 0, 3])                           # row 0: pages 4, 1; row 1: pages 0, 3
    kp = torch.zeros(5, G, 64, dk, dtype=dtype, device=DEV)
    vp = torch.zeros(5, G, 64, dv, dtype=dtype, device=DEV)
    q_out = torch.empty(T, nq, dtype=dtype, device=DEV)
    k_out = torch.empty(T, nk, dtype=dtype, device=DEV)
    v_out = torch.empty(T, nv, dtype=dtype, device=DEV)
    kernels.rownorm_qkv_store(x, q_out, n_heads=H, n_kv_heads=G, key_dim=dk, value_dim=dv, tok_pos=pos, tok_seq=seq,
                              new_lens=new_lens, q_weight=wq, k_weight=wk, eps=eps, temp_coef=coef, temp_every=every,
                              k_out=k_out, v_out=v_out, k_pages=kp, v_pages=vp, block_table=table, table_width=2)
    xd = x.double()
    rq = xd[:, :nq] / torch.sqrt((xd[:, :nq] ** 2).mean(-1, keepdim=True) + eps) * wq.double()
    rk = xd[:, nq:nq + nk] / torch.sqrt((xd[:, nq:nq + nk] ** 2).mean(-1, keepdim=True) + eps) * wk.double()
    temp = torch.tensor([1 + coef * math.log((p + 1) // every + 1) for p in pos.tolist()], device=DEV).double()
    tol = 1e-5 if dtype == torch.float32 else 1e-2
    _close(q_out, rq * temp.unsqueeze(1), tol, "q")
    _close(k_out, rk, tol, "k")
    _close(v_out, xd[:, nq + nk:nq + nk + nv], tol, "v")
    for t, (b, p) in enumerate(zip(seq.tolist(), pos.tolist())):
        page = table[b * 2 + p // 64].item()
        assert torch.equal(kp[page, 0, p % 64], k_out[t]) and torch.equal(vp[page, 0, p % 64], v_out[t])
    assert kp[2].abs().max().item() == 0                 # a page of no sequence


@pytest.mark.parametrize("H, d, e", [(2, 24, 24), (1, 64, 64), (1, 128, 128), (1, 200, 200), (3, 8, 48), (1, 100, 20)])
def test_the_one_token_kernel_equals_the_scan(H, d, e):
    """Six sequences of one token each through the kernel for decoding and through the general one."""
    from tq_kv_b200 import kernels
    torch.manual_seed(e)
    B, n = 6, H * d
    slots = _i32([4, 0, 5, 2, 7, 1])
    cu = _i32(list(range(B + 1)))
    for mode in (["delta", "decay"] if d == e else ["decay"]):
        proj = torch.randn(B, 4 * n + H * e + 4, device=DEV)
        logit = torch.randn(B, n, device=DEV)
        outs, states = [], []
        for single in (True, False):
            state = torch.randn(8, H, d, e, generator=torch.Generator(device=DEV).manual_seed(1), device=DEV)
            out = torch.empty(B, H * e, device=DEV)
            kw = dict(n_seqs=B, heads=H, key_dim=d, value_dim=e, off_q=0, off_k=n, off_v=2 * n, single_tokens=single)
            if mode == "delta":
                kw.update(off_a=3 * n + H * e, decay_logit=logit.clone())
            else:
                kw.update(head_decay=torch.tensor([0.9, 0.5, 0.99][:H], device=DEV), silu=True)
            kernels.linear_scan(proj.clone(), state, cu, slots, out, **kw)
            outs.append(out)
            states.append(state)
        _close(outs[0], outs[1], 1e-5, mode + " outputs")
        _close(states[0], states[1], 1e-5, mode + " states")


@pytest.mark.parametrize("H, G, d", [(4, 2, 32), (2, 2, 64), (3, 1, 96), (8, 2, 128), (34, 2, 64), (2, 1, 48)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_sigmoid_attention_of_single_decoded_tokens(H, G, d, dtype):
    """Rows of one token each (what a decode step brings) at several positions of the same cached keys, with one
    split and with several: the kernel that streams the cache once for a group's heads (bfloat16, widths 32 to 128,
    up to 16 heads a group) and the general one (everything else) against float64."""
    from tq_kv_b200 import kernels
    torch.manual_seed(H * d)
    T, scale, n_dist = 200, 0.25 / math.sqrt(d), 57
    q = torch.randn(T, H * d, device=DEV).to(dtype)
    k = torch.randn(T, G * d, device=DEV).to(dtype)
    v = torch.randn(T, G * d, device=DEV).to(dtype)
    bias = torch.randn(H, n_dist, device=DEV) * 2 - 1
    gate = torch.randn(T, H, device=DEV)
    want = _attention_reference(q, k, v, H, G, d, d, scale, bias, gate)
    order = [3, 1, 0, 2]
    kp, vp = _pages(k, v, G, d, d, 64, order)
    rows = [199, 0, 63, 64, 128, 31]
    table = _i32(order * len(rows))
    pos = _i32(rows)
    sel = torch.tensor(rows, device=DEV)
    tol = 2e-5 if dtype == torch.float32 else 2e-2
    for n_splits in (1, 4):
        out = torch.full((len(rows), H * d), float("nan"), dtype=dtype, device=DEV)
        scratch = torch.empty(len(rows) * H * n_splits * d, device=DEV) if n_splits > 1 else None
        kernels.sigmoid_attention(q[sel].contiguous(), out, n_heads=H, n_kv_heads=G, key_dim=d, value_dim=d, scale=scale,
                                  tok_pos=pos, tok_seq=_i32(list(range(len(rows)))),
                                  cu_seqlens=_i32(list(range(len(rows) + 1))), start_pos=pos, bias=bias,
                                  gate=gate[sel].contiguous(), k_pages=kp, v_pages=vp, block_table=table, table_width=4,
                                  page_tokens=64, n_splits=n_splits, scratch=scratch)
        _close(out, want[sel.cpu()], tol, f"{n_splits} splits")

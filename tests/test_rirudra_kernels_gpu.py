"""The kernels that the Rirudra mixers add — short convolution with its state, the scans with one decay per head and
token, the gated norms, the kernels around attention through a latent — each alone against a float64 computation of
the same formula at several sizes (GPU)."""
import math

import pytest
import torch

import plain_rirudra as pr

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _close(got, want, tol, what=""):
    got, want = got.double().cpu(), want.double().cpu()
    err = (got - want).abs().max().item()
    ref = want.abs().max().item()
    assert math.isfinite(err) and err <= tol * max(ref, 1e-30), f"{what}: {err:.3e} of {ref:.3e} > {tol:.1e}"


def _i32(x):
    return torch.tensor(x, dtype=torch.int32, device=DEV)


def _batch(lens):
    cu = [0]
    for n in lens:
        cu.append(cu[-1] + n)
    seq = [b for b, n in enumerate(lens) for _ in range(n)]
    return _i32(cu), _i32(seq), cu


# ---- short convolution ------------------------------------------------------------------------------------
@pytest.mark.parametrize("C, K, lens", [(40, 4, (9, 1, 2, 30)), (7, 2, (5, 3)), (300, 3, (1, 1, 1)), (33, 1, (4, 6)),
                                        (64, 8, (3, 20))])
def test_short_convolution_with_state_in_portions_and_single_tokens(C, K, lens):
    """Sequences in a ragged batch on shuffled slots; the same sequences again in portions of 1, 2 and the rest, and
    with the one-token form: the state carries the last taps - 1 inputs from call to call."""
    from tq_kv_b200 import kernels
    torch.manual_seed(C + K)
    B, T = len(lens), sum(lens)
    wide = torch.randn(T, C + 11, device=DEV)
    x = wide[:, 5:5 + C]                                                 # a column slice
    w, bias = torch.randn(C, K, device=DEV), torch.randn(C, device=DEV)
    cu, seq, cu_h = _batch(lens)
    slots = _i32([3, 0, 5, 1][:B])
    pad = 6                                                              # the state sits behind other floats of the slot
    want = torch.cat([pr.silu(pr.causal_conv(x[cu_h[b]:cu_h[b + 1]].double().cpu(), w.double().cpu(), bias.double().cpu()))
                      for b in range(B)])

    def run(x_part, lens_part, state, single=False):
        cu_p, seq_p, _ = _batch(lens_part)
        out = torch.full((x_part.shape[0], C + 2), 7.0, device=DEV)
        kernels.short_conv(x_part, w, bias, out, state[:, pad:], tok_seq=seq_p, cu_seqlens=cu_p, slots=slots,
                           n_seqs=B, regions=[(0, C, min(C, 128), False, 1.0)], silu=True, single_tokens=single)
        assert (out[:, C:] == 7.0).all()
        return out[:, :C]

    state = torch.zeros(6, pad + (K - 1) * C, device=DEV)
    _close(run(x, lens, state), want, 1e-5, "whole")
    for b in range(B):                                                   # the state now holds each sequence's last inputs
        tail = x[cu_h[b]:cu_h[b + 1]][-(K - 1):] if K > 1 else x[:0]
        got = state[int(slots[b]), pad:].reshape(K - 1, C)[(K - 1) - tail.shape[0]:]
        assert torch.equal(got, tail) and (state[int(slots[b]), :pad] == 0).all()
    # portions: every sequence one token, then up to two, then the rest; rows of a sequence that has ended are dropped
    state = torch.zeros(6, pad + (K - 1) * C, device=DEV)
    at = [0] * B
    pieces = [[] for _ in range(B)]
    for step, take in enumerate((1, 2, 10 ** 6)):
        part = [min(take, lens[b] - at[b]) for b in range(B)]
        rows = torch.cat([x[cu_h[b] + at[b]:cu_h[b] + at[b] + part[b]] for b in range(B)])
        if rows.shape[0] == 0:
            break
        wide_p = torch.zeros(rows.shape[0], C + 3, device=DEV)
        wide_p[:, 1:1 + C] = rows
        live = [b for b in range(B) if part[b] > 0]
        cu_p, seq_p, cu_ph = _batch([part[b] for b in live])
        out = torch.empty(rows.shape[0], C, device=DEV)
        kernels.short_conv(wide_p[:, 1:1 + C], w, bias, out, state[:, pad:], tok_seq=seq_p, cu_seqlens=cu_p,
                           slots=_i32([int(slots[b]) for b in live]), n_seqs=len(live),
                           regions=[(0, C, min(C, 128), False, 1.0)], silu=True,
                           single_tokens=all(part[b] == 1 for b in live))
        for j, b in enumerate(live):
            pieces[b].append(out[cu_ph[j]:cu_ph[j + 1]])
            at[b] += part[b]
    _close(torch.cat([torch.cat(p) for p in pieces]), want, 1e-5, "portions")


def test_short_convolution_unit_vectors_and_the_recurrences_scalars():
    from tq_kv_b200 import kernels
    torch.manual_seed(3)
    T, H, d, e, K = 13, 3, 20, 12, 3
    C = 2 * 2 * d + H * e                                                # two key heads
    x, w = torch.randn(T, C, device=DEV), torch.randn(C, K, device=DEV)
    gate, beta = torch.randn(T, H + 4, device=DEV) * 3, torch.randn(T, H, device=DEV) * 3
    a_log, dt_bias = torch.randn(H, device=DEV), torch.randn(H, device=DEV)
    cu, seq, _ = _batch([T])
    out, scal = torch.empty(T, C, device=DEV), torch.empty(T, H, 4, device=DEV)
    state = torch.zeros(2, (K - 1) * C, device=DEV)
    kernels.short_conv(x, w, None, out, state, tok_seq=seq, cu_seqlens=cu, slots=_i32([1]), n_seqs=1,
                       regions=[(0, 2 * d, d, True, 0.25), (2 * d, 2 * d, d, True, 1.0), (4 * d, H * e, 36, False, 1.0)],
                       unit_eps=1e-6, gate_raw=gate[:, 2:2 + H], beta_raw=beta, a_log=a_log, dt_bias=dt_bias, scalars=scal)
    y = pr.silu(pr.causal_conv(x.double().cpu(), w.double().cpu()))
    q = pr.unit(y[:, :2 * d].reshape(T, 2, d)).reshape(T, -1) * 0.25
    k = pr.unit(y[:, 2 * d:4 * d].reshape(T, 2, d)).reshape(T, -1)
    _close(out, torch.cat([q, k, y[:, 4 * d:]], 1), 1e-5, "unit vectors")
    sp = pr.softplus(gate[:, 2:2 + H].double().cpu() + dt_bias.double().cpu())
    _close(scal[:, :, 0], torch.exp(-torch.exp(a_log.double().cpu()) * sp), 1e-5, "decay")
    _close(scal[:, :, 1], torch.sigmoid(beta.double().cpu()), 1e-5, "write strength")
    kernels.short_conv(x, w, None, out, state, tok_seq=seq, cu_seqlens=cu, slots=_i32([0]), n_seqs=1,
                       regions=[(0, C, 64, False, 1.0)], gate_raw=gate[:, 2:2 + H], a_log=a_log, dt_bias=dt_bias, scalars=scal)
    _close(scal[:, :, 1], sp, 1e-5, "step size")


# ---- the scans with one decay per head and token ----------------------------------------------------------
def _scan_reference(delta, q, k, v, scal, skip, H, G, d, e, state0, bounds):
    q, k, v, scal = q.double().cpu(), k.double().cpu(), v.double().cpu(), scal.double().cpu()
    out = torch.zeros(q.shape[0], H * e, dtype=torch.float64)
    states = []
    for (a, b), S0 in zip(bounds, state0):
        S = S0.double().cpu().clone()
        for t in range(a, b):
            for h in range(H):
                kh = h // (H // G)
                qq, kk, vv = q[t, kh * d:(kh + 1) * d], k[t, kh * d:(kh + 1) * d], v[t, h * e:(h + 1) * e]
                g, s2 = scal[t, h, 0], scal[t, h, 1]
                S[h] = g * S[h]
                if delta:
                    S[h] = S[h] + torch.outer(kk, s2 * (vv - S[h].T @ kk))
                else:
                    S[h] = S[h] + s2 * torch.outer(kk, vv)
                out[t, h * e:(h + 1) * e] = S[h].T @ qq + (0 if skip is None else skip.double().cpu()[h] * vv)
        states.append(S)
    return out, states


@pytest.mark.parametrize("delta", [False, True])
@pytest.mark.parametrize("H, G, d, e, lens", [(4, 2, 16, 12, (9, 1, 30)), (2, 2, 64, 64, (70,)), (3, 1, 24, 7, (2, 2, 2, 5)),
                                              (1, 1, 128, 40, (20, 3)), (2, 1, 160, 6, (12,)), (6, 3, 5, 33, (4, 8)),
                                              (2, 2, 256, 8, (6,)), (2, 2, 160, 8, (3, 11)), (1, 1, 200, 4, (10,))])
def test_gated_scans_ragged_slots_states_and_the_one_token_form(delta, H, G, d, e, lens):
    from tq_kv_b200 import kernels
    torch.manual_seed(H * d + e)
    B, T = len(lens), sum(lens)
    C = 2 * G * d + H * e
    buf = torch.randn(T, C + 3, device=DEV)
    buf[:, :2 * G * d] *= d ** -0.5
    q, k, v = buf[:, :G * d], buf[:, G * d:2 * G * d], buf[:, 2 * G * d:2 * G * d + H * e]
    scal = torch.zeros(T, H, 4, device=DEV)
    scal[:, :, 0] = torch.rand(T, H, device=DEV) * 0.6 + 0.4
    scal[:, :, 1] = torch.rand(T, H, device=DEV)
    skip = None if delta else torch.randn(H, device=DEV)
    cu, _, cu_h = _batch(lens)
    slots_h = [4, 1, 6, 0][:B]
    n_state, pad = H * d * e, 5
    state = torch.randn(8, n_state + pad, device=DEV) * 0.3                # states that are not zero: a continuation
    before = state.clone()
    s0 = [state[s, :n_state].reshape(H, d, e).clone() for s in slots_h]
    bounds = [(cu_h[b], cu_h[b + 1]) for b in range(B)]
    want, want_states = _scan_reference(delta, q, k, v, scal, skip, H, G, d, e, s0, bounds)
    out = torch.empty(T, H * e, device=DEV)
    kernels.gated_scan(q, k, v, scal, state[:, :n_state], cu, _i32(slots_h), out, n_seqs=B, heads=H, qk_heads=G,
                       key_dim=d, value_dim=e, delta=delta, skip=skip)
    _close(out, want, 2e-5, "outputs")
    for b, s in enumerate(slots_h):
        _close(state[s, :n_state].reshape(H, d, e), want_states[b], 2e-5, f"state of slot {s}")
    untouched = [s for s in range(8) if s not in slots_h]
    assert torch.equal(state[untouched], before[untouched]) and torch.equal(state[:, n_state:], before[:, n_state:])
    # token by token with the one-token form, from the same start
    state2 = before.clone()
    got = torch.zeros_like(out)
    for step in range(max(lens)):
        live = [b for b in range(B) if step < lens[b]]
        rows = [cu_h[b] + step for b in live]
        part = buf[rows].contiguous()
        o = torch.empty(len(live), H * e, device=DEV)
        kernels.gated_scan(part[:, :G * d], part[:, G * d:2 * G * d], part[:, 2 * G * d:2 * G * d + H * e],
                           scal[rows].contiguous(), state2[:, :n_state], _i32(list(range(len(live) + 1))),
                           _i32([slots_h[b] for b in live]), o, n_seqs=len(live), heads=H, qk_heads=G, key_dim=d,
                           value_dim=e, delta=delta, skip=skip, single_tokens=True)
        got[rows] = o
    _close(got, want, 2e-5, "one token at a time")
    _close(state2, state, 2e-5, "states after one token at a time")


def test_a_state_written_long_ago_is_still_read():
    """One key direction is written once, with a large value, then 600 tokens with decay 1 and keys orthogonal to it
    follow: the last token, whose query is that key, reads the old value (delta rule and plain decay)."""
    from tq_kv_b200 import kernels
    torch.manual_seed(1)
    T, d, e = 601, 16, 8
    basis = torch.linalg.qr(torch.randn(d, d, dtype=torch.float64))[0].float().to(DEV)
    for delta in (False, True):
        buf = torch.zeros(T, 2 * d + e, device=DEV)
        buf[0, d:2 * d], buf[0, 2 * d:] = basis[0], torch.arange(1, e + 1, device=DEV) * 10.0
        idx = torch.randint(1, d, (T - 1,))
        buf[1:, d:2 * d], buf[1:, 2 * d:] = basis[idx], torch.randn(T - 1, e, device=DEV)
        buf[1:, :d] = basis[idx]
        buf[T - 1, :d] = basis[0]
        scal = torch.zeros(T, 1, 4, device=DEV)
        scal[:, :, 0], scal[:, :, 1] = 1.0, 1.0
        state, out = torch.zeros(1, d * e, device=DEV), torch.empty(T, e, device=DEV)
        kernels.gated_scan(buf[:, :d], buf[:, d:2 * d], buf[:, 2 * d:], scal, state, _i32([0, T]), _i32([0]), out,
                           n_seqs=1, heads=1, qk_heads=1, key_dim=d, value_dim=e, delta=delta)
        _close(out[T - 1], torch.arange(1, e + 1) * 10.0, 1e-4, f"delta={delta}")


# ---- gated norms, scaled sums ----------------------------------------------------------------------------
@pytest.mark.parametrize("width, groups", [(96, 3), (84, 4), (120, 1)])
@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16])
def test_grouped_norm_gate_modes(width, groups, out_dtype):
    from tq_kv_b200 import kernels
    torch.manual_seed(groups)
    T, eps = 9, 1e-5
    wide = torch.randn(T, 3 * width + 5, device=DEV) * 3
    x, gate = wide[:, 2:2 + width], wide[:, width + 3:2 * width + 3]
    w = torch.randn(width, device=DEV)
    tol = 1e-5 if out_dtype == torch.float32 else 1e-2

    def norm(z):
        p = z.reshape(T, groups, -1)
        return (p / torch.sqrt((p * p).mean(-1, keepdim=True) + eps)).reshape(T, width) * w.double().cpu()

    xd, gd = x.double().cpu(), gate.double().cpu()
    out = torch.empty(T, width, dtype=out_dtype, device=DEV)
    _close(kernels.group_rmsnorm(x, w, eps, out, groups=groups, gate=gate, gate_mode=kernels.GATE_SILU),
           norm(xd) * pr.silu(gd), tol, "silu after")
    _close(kernels.group_rmsnorm(x, w, eps, out, groups=groups, gate=gate, gate_mode=kernels.GATE_SILU_FIRST),
           norm(xd * pr.silu(gd)), tol, "silu before")
    _close(kernels.group_rmsnorm(x, w, eps, out, groups=groups, gate=gate), norm(xd) * torch.sigmoid(gd), tol, "sigmoid")


def test_scaled_sum_and_scaled_embedding():
    from tq_kv_b200 import kernels
    torch.manual_seed(0)
    for n in (7 * 33, 8 * 64):
        a, x = torch.randn(n, device=DEV), torch.randn(n, device=DEV)
        _close(kernels.add_scaled(a.clone(), x, 0.3), a.double() + 0.3 * x.double(), 1e-6, "axpy")
    table = torch.randn(20, 24, device=DEV).to(torch.bfloat16)
    toks = _i32([3, 19, 0])
    out = torch.empty(3, 24, device=DEV)
    _close(kernels.embed(toks, table, out, None, 12.5), table[toks.long()].double() * 12.5, 1e-6, "scaled rows")


# ---- around attention through a latent ---------------------------------------------------------------------
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H, d, r, e, qr, n, dims, paired", [(3, 16, 8, 24, 40, 48, 8, True), (2, 8, 12, 5, 10, 30, 8, True),
                                                             (1, 32, 16, 16, 24, 100, 16, False), (4, 64, 32, 64, 96, 96, 32, True)])
def test_latent_rows_query_and_expansion(dtype, H, d, r, e, qr, n, dims, paired):
    from tq_kv_b200 import kernels
    torch.manual_seed(n + r)
    tol = 1e-5 if dtype == torch.float32 else 1.2e-2
    T, eps, rp = 11, 1e-5, -(-(n + r) // 16) * 16
    pos_h = [0, 1, 62, 63, 64, 65, 127, 128, 199, 5, 6]                   # two sequences; the first crosses page edges
    seq_h = [0] * 9 + [1] * 2
    pos, seq, new_lens = _i32(pos_h), _i32(seq_h), _i32([200, 7])
    proj = torch.randn(T, 3 + qr + n + r, device=DEV) * 2
    wq, wkv = torch.rand(qr, device=DEV) + 0.5, torch.rand(n, device=DEV) + 0.5
    half = dims // 2
    rate = torch.pow(torch.tensor(1e4, dtype=torch.float64), -2.0 * torch.arange(half, dtype=torch.float64) / dims)
    ang = torch.arange(256, dtype=torch.float64).unsqueeze(1) * rate
    cos, sin = torch.cos(ang).float().to(DEV), torch.sin(ang).float().to(DEV)

    def rot(x, p):                                                          # x [..., r] float64 on the CPU
        x = x.clone()
        c, s = torch.cos(ang[p]), torch.sin(ang[p])
        if paired:
            a, b = x[..., 0:dims:2].clone(), x[..., 1:dims:2].clone()
            x[..., 0:dims:2], x[..., 1:dims:2] = a * c - b * s, b * c + a * s
        else:
            a, b = x[..., :half].clone(), x[..., half:dims].clone()
            x[..., :half], x[..., half:dims] = a * c - b * s, b * c + a * s
        return x

    cq = torch.empty(T, qr, dtype=dtype, device=DEV)
    rows = torch.empty(T, rp, dtype=dtype, device=DEV)
    pages = torch.zeros(9, 1, 64, rp, dtype=dtype, device=DEV)
    table = _i32([[7, 2, 5, 0], [3, 8, 8, 8]])
    kernels.latent_rows(proj, cq, off_q=3, off_kv=3 + qr, q_rank=qr, kv_rank=n, rot_dim=r, row_width=rp, q_weight=wq,
                        kv_weight=wkv, eps=eps, cos=cos, sin=sin, rot_dims=dims, paired=paired, tok_pos=pos, tok_seq=seq,
                        new_lens=new_lens, row_out=rows, pages=pages, block_table=table, table_width=4)
    p64 = proj.double().cpu()
    _close(cq, pr.rms(p64[:, 3:3 + qr], eps) * wq.double().cpu(), tol, "query latent")
    want_rows = torch.zeros(T, rp, dtype=torch.float64)
    want_rows[:, :n] = pr.rms(p64[:, 3 + qr:3 + qr + n], eps) * wkv.double().cpu()
    for t in range(T):
        want_rows[t, n:n + r] = rot(p64[t, 3 + qr + n:], pos_h[t])
    _close(rows, want_rows, tol, "rows")
    for t in range(T):                                                      # each row lies in its sequence's page
        page = int(table[seq_h[t], pos_h[t] // 64])
        assert torch.equal(pages[page, 0, pos_h[t] % 64], rows[t])
    assert int((pages.float().abs().sum(-1) > 0).sum()) == T
    # the query in the latent's space
    q = torch.randn(T, H * (d + r), device=DEV)
    uk = (torch.randn(H * d, n, device=DEV) / d ** 0.5).to(dtype)
    qa = torch.empty(T, H * rp, dtype=dtype, device=DEV)
    kernels.latent_query(q, uk, qa, heads=H, dim=d, rot_dim=r, kv_rank=n, row_width=rp, cos=cos, sin=sin, rot_dims=dims,
                         paired=paired, tok_pos=pos)
    q64 = q.double().cpu().reshape(T, H, d + r)
    want_q = torch.zeros(T, H, rp, dtype=torch.float64)
    for h in range(H):
        want_q[:, h, :n] = q64[:, h, :d] @ uk.double().cpu()[h * d:(h + 1) * d]
        for t in range(T):
            want_q[t, h, n:n + r] = rot(q64[t, h, d:], pos_h[t])
    _close(qa, want_q.reshape(T, -1), tol, "query")
    # the expansion of a head's mean latent, gated
    lat = torch.randn(T, H * rp, device=DEV).to(dtype)
    uv = (torch.randn(H * e, n, device=DEV) / n ** 0.5).to(dtype)
    gate = torch.randn(T, H * e + 2, device=DEV)
    y = torch.empty(T, H * e, dtype=dtype, device=DEV)
    kernels.latent_expand(lat, uv, y, heads=H, kv_rank=n, row_width=rp, value_dim=e, gate=gate[:, 1:1 + H * e])
    l64 = lat.double().cpu().reshape(T, H, rp)[:, :, :n]
    want_y = torch.stack([l64[:, h] @ uv.double().cpu()[h * e:(h + 1) * e].T for h in range(H)], 1).reshape(T, -1)
    _close(y, want_y * torch.sigmoid(gate[:, 1:1 + H * e].double().cpu()), tol, "expansion")
    kernels.latent_expand(lat, uv, y, heads=H, kv_rank=n, row_width=rp, value_dim=e)
    _close(y, want_y, tol, "expansion without a gate")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H, d, r, e, n", [(3, 16, 8, 24, 48), (2, 8, 12, 40, 30), (4, 64, 64, 128, 96)])
def test_expanded_heads_for_prompts(dtype, H, d, r, e, n):
    from tq_kv_b200 import kernels
    torch.manual_seed(e)
    tol = 1e-6 if dtype == torch.float32 else 1e-2
    T, rp, hw = 7, -(-(n + r) // 16) * 16, -(-max(d + r, e) // 16) * 16
    pos_h = [0, 1, 2, 63, 64, 5, 130]
    rate = torch.pow(torch.tensor(1e4, dtype=torch.float64), -2.0 * torch.arange(r // 2, dtype=torch.float64) / r)
    ang = torch.arange(200, dtype=torch.float64).unsqueeze(1) * rate
    cos, sin = torch.cos(ang).float().to(DEV), torch.sin(ang).float().to(DEV)
    q, kfv = torch.randn(T, H * (d + r), device=DEV), torch.randn(T, H * (d + e), device=DEV)
    rows = torch.randn(T, rp, device=DEV).to(dtype)
    qo, ko, vo = (torch.full((T, H * hw), 9.0, dtype=dtype, device=DEV) for _ in range(3))
    kernels.latent_heads(q, kfv, rows, qo, ko, vo, heads=H, dim=d, rot_dim=r, value_dim=e, kv_rank=n, cos=cos, sin=sin,
                         rot_dims=r, paired=True, tok_pos=_i32(pos_h))
    q64 = q.double().cpu().reshape(T, H, d + r)
    wq, wk, wv = (torch.zeros(T, H, hw, dtype=torch.float64) for _ in range(3))
    wq[:, :, :d] = q64[:, :, :d]
    wq[:, :, d:d + r] = pr.rotate_pairs(q64[:, :, d:], torch.tensor(pos_h), r, 1e4)
    wk[:, :, :d] = kfv.double().cpu()[:, :H * d].reshape(T, H, d)
    wk[:, :, d:d + r] = rows.double().cpu()[:, n:n + r].unsqueeze(1)
    wv[:, :, :e] = kfv.double().cpu()[:, H * d:].reshape(T, H, e)
    _close(qo, wq.reshape(T, -1), tol, "queries")
    _close(ko, wk.reshape(T, -1), tol, "keys")
    _close(vo, wv.reshape(T, -1), tol, "values")
    gate = torch.randn(T, H * e, device=DEV)
    y = torch.empty(T, H * e, dtype=dtype, device=DEV)
    kernels.latent_expand(vo, None, y, heads=H, kv_rank=hw, row_width=hw, value_dim=e, gate=gate)
    _close(y, wv[:, :, :e].reshape(T, -1) * torch.sigmoid(gate.double().cpu()), tol, "gated heads")


@pytest.mark.parametrize("heads, width", [(32, 128), (24, 64), (17, 128), (6, 96)])
def test_many_heads_on_one_shared_cache_row(heads, width):
    """Decoded tokens whose heads all read ONE key/value head whose values are the keys themselves (the cache of a
    latent), with more heads than one tensor-core tile holds: positions around page edges, one and several splits."""
    from tq_kv_b200 import kernels
    torch.manual_seed(heads)
    pos_h = [0, 1, 63, 64, 65, 200, 399]
    T = len(pos_h)
    pages = torch.randn(T * 7, 1, 64, width, device=DEV).to(torch.bfloat16)
    table = torch.randperm(T * 7, device=DEV).to(torch.int32).reshape(T, 7).contiguous()
    q = (torch.randn(T, heads * width, device=DEV) * 0.5).to(torch.bfloat16)
    want = torch.zeros(T, heads, width, dtype=torch.float64)
    for t, p in enumerate(pos_h):
        rows = torch.cat([pages[int(table[t, j]), 0] for j in range(p // 64 + 1)])[:p + 1].double().cpu()
        s = q[t].double().cpu().reshape(heads, width) @ rows.T * 0.2
        want[t] = torch.softmax(s, -1) @ rows
    for n_splits in (1, 3):
        out = torch.empty_like(q)
        scratch = torch.empty(kernels.split_scratch_floats(T, heads, width, n_splits), device=DEV) if n_splits > 1 else None
        kernels.attention(q, out, n_heads=heads, n_kv_heads=1, head_dim=width, tok_pos=_i32(pos_h),
                          tok_seq=_i32(list(range(T))), cu_seqlens=_i32(list(range(T + 1))), start_pos=_i32(pos_h),
                          window=None, scale=0.2, k_pages=pages, v_pages=pages, block_table=table, table_width=7,
                          n_splits=n_splits, scratch=scratch)
        _close(out, want.reshape(T, -1), 1.5e-2, f"{n_splits} splits")

"""The kernels of the Redudra parts one by one, each against the oracle's function of the same mechanism on the same
(bfloat16-rounded) inputs: a request's tokens cut into steps of several sizes (down to one and two tokens) against the
whole sequence, states carried in slots that are not the requests' indices, keys far away, at page borders, among the
kept first tokens and on both sides of a window's edge, with planted scores that stand out."""

from __future__ import annotations

import math
import random

import numpy as np
import pytest
import torch

import plain_redudra as pr

pytestmark = pytest.mark.gpu

DEV = "cuda:0"
DT = {"float32": torch.float32, "bfloat16": torch.bfloat16}
CUTS = ([1] * 9, [2, 2, 2, 2, 1], [9], [3, 1, 5], [1, 8], [7, 2], [4, 5])


def dev(a, dtype=torch.float32):
    return torch.as_tensor(np.asarray(a)).to(device=DEV, dtype=dtype).contiguous()


def i32(a):
    return torch.tensor(list(a), dtype=torch.int32, device=DEV)


def bf(a):
    """float64 numpy values that bfloat16 holds exactly."""
    return torch.as_tensor(np.asarray(a, dtype=np.float64)).to(torch.bfloat16).to(torch.float64).numpy()


def close(got, want, tol, what=""):
    got, want = np.asarray(got.detach().float().cpu() if torch.is_tensor(got) else got, dtype=np.float64), np.asarray(want)
    scale = max(float(np.abs(want).max()), 1e-30)
    err = float(np.abs(got - want).max()) / scale
    assert err < tol, f"{what}: largest difference {err:.3e} of the largest value"


def batches(lengths, cuts_of):
    """Steps over several requests: each step is [(request, first token, count)], requests advancing side by side."""
    at = [0] * len(lengths)
    turn = [0] * len(lengths)
    steps = []
    while any(a < n for a, n in zip(at, lengths)):
        step = []
        for r, n in enumerate(lengths):
            if at[r] < n:
                c = min(cuts_of[r][turn[r] % len(cuts_of[r])], n - at[r])
                step.append((r, at[r], c))
                at[r] += c
                turn[r] += 1
        steps.append(step)
    return steps


def segments(q_lens, seg_len):
    """The step's (request, segment) items on the device, for segments of ``seg_len`` tokens (0: none, whole portions)."""
    from acvram_b200.kernels import ops
    if not seg_len:
        return None
    arrays, values = ops.segment_work(q_lens, seg_len)
    return {**{k: i32(v) for k, v in arrays.items()}, **values}


def step_arrays(step):
    cu = [0]
    seq_of = []
    for i, (_, _, c) in enumerate(step):
        cu.append(cu[-1] + c)
        seq_of += [i] * c
    return i32(cu), i32(seq_of)


# --------------------------------------------------------------------------- layer norm and token shift
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H", [32, 100, 1024])
def test_layernorm_and_token_shift_over_steps(H, dtype):
    from acvram_b200.kernels import ops
    rng = np.random.default_rng(H)
    lengths = [9, 5, 1]
    w, b, mu = bf(1 + 0.2 * rng.standard_normal(H)), bf(0.1 * rng.standard_normal(H)), bf(rng.random(H))
    xs = [rng.standard_normal((n, H)) * 3 + 1 for n in lengths]
    ds = [bf(rng.standard_normal((n, H))) for n in lengths]
    m, eps = 0.3, 1e-5
    want = [pr.token_shift(pr.layer_norm(np.float32(x).astype(np.float64) + m * d, w, b, eps), mu) for x, d in zip(xs, ds)]
    tol = 2e-6 if dtype == "float32" else 6e-3
    for fused in (False, True):
        cuts = [[1]] * 3 if fused else [CUTS[3], CUTS[1], CUTS[0]]
        state = torch.full((6, H), 7.0, device=DEV)
        slots = [4, 0, 2]
        state[slots] = 0.0
        got = [np.zeros((n, H)) for n in lengths]
        for step in batches(lengths, cuts):
            cu, seq_of = step_arrays(step)
            x = dev(np.concatenate([xs[r][a:a + c] for r, a, c in step]))
            d = dev(np.concatenate([ds[r][a:a + c] for r, a, c in step]), DT[dtype])
            sl = i32([slots[r] for r, _, _ in step])
            out = torch.empty(x.shape, device=DEV, dtype=DT[dtype])
            if fused:
                ops.add_layernorm_shift(x, d, dev(w), dev(b), eps, dev(mu), state, sl, out, m)
            else:
                n = ops.add_layernorm(x, d, dev(w), dev(b), eps, torch.empty_like(x), None, m)
                ops.token_shift(n, dev(mu), state, sl, cu, seq_of, out)
            o = 0
            for r, a, c in step:
                got[r][a:a + c] = out[o:o + c].float().cpu().numpy()
                # the stream itself took the sum
                close(x[o:o + c], np.float32(xs[r][a:a + c]).astype(np.float64) + m * ds[r][a:a + c], 1e-6, "stream")
                o += c
        for r in range(3):
            close(got[r], want[r], tol, f"request {r}, fused {fused}")
        assert float(state[1, 0]) == 7.0, "a slot of no request was written"


def test_layernorm_of_chosen_rows_leaves_the_stream():
    from acvram_b200.kernels import ops
    rng = np.random.default_rng(1)
    x, d = rng.standard_normal((7, 48)), bf(rng.standard_normal((7, 48)))
    w, b = bf(1 + 0.1 * rng.standard_normal(48)), bf(0.1 * rng.standard_normal(48))
    xd = dev(x)
    out = ops.add_layernorm(xd, dev(d), dev(w), dev(b), 1e-6, torch.empty((2, 48), device=DEV), i32([5, 0]), 0.5)
    close(out, pr.layer_norm(np.float32(x).astype(np.float64)[[5, 0]] + 0.5 * d[[5, 0]], w, b, 1e-6), 2e-6)
    assert torch.equal(xd, dev(x))


# --------------------------------------------------------------------------- gated linear recurrence
@pytest.mark.parametrize("taps", [1, 2, 4, 5])
def test_causal_conv_over_steps(taps):
    from acvram_b200.kernels import ops
    rng = np.random.default_rng(taps)
    C = 72
    lengths = [9, 9, 4]
    xs = [bf(rng.standard_normal((n, C))) for n in lengths]
    xb, w, cb = bf(0.1 * rng.standard_normal(C)), bf(rng.standard_normal((C, taps))), bf(0.1 * rng.standard_normal(C))
    want = [pr.causal_conv(x + xb, w, cb) for x in xs]
    for cuts in ([CUTS[0], CUTS[1], CUTS[5]], [CUTS[2], CUTS[3], CUTS[0]], [CUTS[4], CUTS[6], CUTS[1]]):
        state = torch.zeros((5, max(taps - 1, 1), C), device=DEV)
        slots = [3, 1, 4]
        got = [np.zeros((n, C)) for n in lengths]
        for step in batches(lengths, cuts):
            cu, seq_of = step_arrays(step)
            x = dev(np.concatenate([xs[r][a:a + c] for r, a, c in step]), torch.bfloat16)
            wide = torch.zeros((x.shape[0], C + 10), device=DEV, dtype=torch.bfloat16)      # a view with a row stride of its own
            wide[:, 3:3 + C] = x
            out = torch.empty((x.shape[0], C), device=DEV)
            sl = i32([slots[r] for r, _, _ in step])
            # float inputs in a view whose rows and start are aligned take the form with four channels to a thread;
            # it works on a copy of the state and must leave the same outputs and the same state
            wide32 = torch.zeros((x.shape[0], 2 * C), device=DEV)
            wide32[:, :C] = x.float()
            state32, out32 = state.clone(), torch.empty_like(out)
            ops.causal_conv(wide32[:, :C], dev(xb), dev(w), dev(cb), state32, sl, cu, seq_of, out32, taps_t=dev(w.T.copy()))
            ops.causal_conv(wide[:, 3:3 + C], dev(xb), dev(w), dev(cb), state, sl, cu, seq_of, out)
            assert torch.equal(out32, out) and torch.equal(state32, state)
            o = 0
            for r, a, c in step:
                got[r][a:a + c] = out[o:o + c].cpu().numpy()
                o += c
        for r in range(3):
            close(got[r], want[r], 2e-6, f"taps {taps}, request {r}")


@pytest.mark.parametrize("C,blocks", [(64, 1), (96, 3), (100, 5), (512, 2)])
def test_gates_and_scan_over_steps(C, blocks):
    from acvram_b200.kernels import ops
    rng = np.random.default_rng(C)
    bw = C // blocks
    lengths = [40, 9, 1]
    us = [rng.standard_normal((n, C)).astype(np.float32).astype(np.float64) for n in lengths]
    ys = [rng.standard_normal((n, C)).astype(np.float32).astype(np.float64) for n in lengths]
    wa, wb = rng.standard_normal((blocks, bw, bw)) / math.sqrt(bw), rng.standard_normal((blocks, bw, bw)) / math.sqrt(bw)
    wa, wb = np.float32(wa).astype(np.float64), np.float32(wb).astype(np.float64)
    ba, bb, yb = (np.float32(0.5 * rng.standard_normal(C)).astype(np.float64) for _ in range(3))
    lam = np.linspace(-7.0, 2.0, C)      # from channels that keep for thousands of tokens to channels that forget at once
    sp = np.float32(pr.softplus(lam)).astype(np.float64)

    def whole(u, y):
        ub = u.reshape(-1, blocks, bw)
        r = pr.sigmoid(np.einsum("tbi,boi->tbo", ub, wa).reshape(-1, C) + ba)
        g = pr.sigmoid(np.einsum("tbi,boi->tbo", ub, wb).reshape(-1, C) + bb)
        a = np.exp(-8.0 * r * sp)
        S, out = np.zeros(C), np.zeros_like(u)
        for t in range(u.shape[0]):
            S = a[t] * S + np.sqrt(1 - a[t] ** 2) * g[t] * u[t]
            out[t] = S * pr.gelu_tanh(y[t] + yb)
        return out

    want = [whole(u, y) for u, y in zip(us, ys)]
    wa_t, wb_t = dev(wa.transpose(0, 2, 1)), dev(wb.transpose(0, 2, 1))
    for cuts, seg_len in (([[40], CUTS[1], [1]], 0), ([[17, 1, 2, 20], CUTS[0], [1]], 0), ([[1], CUTS[3], [1]], 0),
                          ([[40], CUTS[2], [1]], 7), ([[25, 15], CUTS[1], [1]], 5), ([[40], CUTS[3], [1]], 40)):
        state = torch.zeros((4, C), device=DEV)
        slots = [2, 3, 0]
        got = [np.zeros((n, C)) for n in lengths]
        for step in batches(lengths, cuts):
            cu, _ = step_arrays(step)
            u = dev(np.concatenate([us[r][a:a + c] for r, a, c in step]))
            y = dev(np.concatenate([ys[r][a:a + c] for r, a, c in step]))
            a_, b_ = torch.empty_like(u), torch.empty_like(u)
            ops.block_gates(u, wa_t, dev(ba), wb_t, dev(bb), dev(sp), -8.0, a_, b_)
            out = torch.empty_like(u)
            ops.gated_scan(a_, b_, y, dev(yb), state, i32([slots[r] for r, _, _ in step]), cu, len(step), out,
                           work=segments([c for _, _, c in step], seg_len))
            o = 0
            for r, a, c in step:
                got[r][a:a + c] = out[o:o + c].cpu().numpy()
                o += c
        for r in range(3):
            close(got[r], want[r], 1e-5, f"request {r}")


# --------------------------------------------------------------------------- retention
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H,D,DV,rot", [(3, 8, 16, 8), (1, 32, 32, 0), (5, 12, 20, 12), (2, 64, 80, 32), (2, 128, 128, 64), (1, 256, 64, 0),
                                          (2, 96, 192, 32), (1, 128, 256, 0), (1, 48, 300, 16)])     # heads too wide for one block's threads
def test_retention_over_steps(H, D, DV, rot, dtype):
    from acvram_b200.kernels import ops
    rng = np.random.default_rng(D + DV)
    lengths = [70, 9, 2]
    decay = [0.5, 0.9, 0.99, 0.999, 0.97][:H]
    rs = {"base": 500.0, "dims": rot} if rot else None
    width = H * (2 * D + 2 * DV)
    rows = [bf(rng.standard_normal((n, width))) for n in lengths]
    eps, out_scale = 1e-5, 0.7

    def whole(x):
        T = x.shape[0]
        q, k = x[:, :H * D].reshape(T, H, D), x[:, H * D:2 * H * D].reshape(T, H, D)
        v, g = x[:, 2 * H * D:2 * H * D + H * DV].reshape(T, H, DV), x[:, 2 * H * D + H * DV:]
        if rs:
            q, k = pr.rotate(q, rs, np.arange(T)), pr.rotate(k, rs, np.arange(T))
        k = k * D ** -0.5
        o = np.zeros((T, H, DV))
        for a in range(H):
            S = np.zeros((D, DV))
            for t in range(T):
                S = decay[a] * S + np.outer(k[t, a], v[t, a])
                o[t, a] = S.T @ q[t, a]
        return pr.unit_rms(o, eps).reshape(T, H * DV) * pr.silu(g) * out_scale

    want = [whole(x) for x in rows]
    table = None
    if rs:
        f, mag = pr.rotary_frequencies(rs)
        ang = np.arange(128)[:, None] * f[None, :]
        table = dev(np.concatenate([np.cos(ang), np.sin(ang)], axis=1) * mag)
    tol = 3e-5 if dtype == "float32" else 1.2e-2
    for cuts, seg_len in (([[70], CUTS[1], [2]], 0), ([[33, 1, 16, 2, 18], CUTS[0], [1]], 0), ([[1], CUTS[3], [2]], 0),
                          ([[70], CUTS[2], [2]], 16), ([[33, 37], CUTS[1], [2]], 9), ([[70], CUTS[3], [1]], 70)):
        state = torch.zeros((4, H, D, DV), device=DEV)
        slots = [1, 3, 0]
        got = [np.zeros((n, H * DV)) for n in lengths]
        for step in batches(lengths, cuts):
            cu, _ = step_arrays(step)
            x = dev(np.concatenate([rows[r][a:a + c] for r, a, c in step]), DT[dtype])
            pos = i32([p for r, a, c in step for p in range(a, a + c)])
            o = torch.empty((x.shape[0], H * DV), device=DEV)
            ops.retention(x[:, :H * D], x[:, H * D:2 * H * D], x[:, 2 * H * D:2 * H * D + H * DV], table, pos,
                          dev(decay), D ** -0.5, state, i32([slots[r] for r, _, _ in step]), cu, len(step), o, H, D, DV,
                          work=segments([c for _, _, c in step], seg_len))
            out = torch.empty((x.shape[0], H * DV + 6), device=DEV, dtype=DT[dtype])
            ops.retention_gate(o, x[:, 2 * H * D + H * DV:], out[:, 6:], H, DV, eps, out_scale)
            at = 0
            for r, a, c in step:
                got[r][a:a + c] = out[at:at + c, 6:].float().cpu().numpy()
                at += c
        for r in range(3):
            close(got[r], want[r], tol, f"request {r}")


# --------------------------------------------------------------------------- attention: value rows, window, kept first tokens
class Paged:
    """One request's keys and values in pages handed out in a shuffled order, on a row of the block table that is not
    the request's index."""

    def __init__(self, n, NKV, D, DV, page, dtype, seed):
        pages = -(-n // page) + 2
        order = list(range(pages))
        random.Random(seed).shuffle(order)
        self.table = torch.full((3, pages), -1, dtype=torch.int32)
        self.table[2, :-(-n // page)] = torch.tensor(order[:-(-n // page)], dtype=torch.int32)
        self.table = self.table.to(DEV)
        self.k = torch.zeros((pages, NKV, page, D), device=DEV, dtype=dtype)
        self.v = torch.zeros((pages, NKV, page, DV), device=DEV, dtype=dtype)
        self.rows = i32([2])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("NH,NKV,D,DV,rot,window,keep,page,n", [
    (4, 2, 16, 24, 8, 20, 3, 16, 200), (2, 2, 32, 32, 32, 24, 0, 16, 200), (3, 3, 24, 40, 10, 7, 9, 8, 200),
    (6, 2, 64, 80, 48, 120, 5, 16, 200), (2, 1, 64, 64, 64, 48, 4, 16, 200), (2, 2, 16, 16, 16, 0, 0, 16, 200),
    (4, 2, 128, 128, 64, 100, 140, 64, 700), (2, 2, 64, 64, 32, 130, 1, 32, 450),
    (2, 1, 128, 128, 64, 900, 8, 64, 1300)])      # a window that the decode kernel cuts into several splits
def test_rope_append_and_attention_with_planted_keys(NH, NKV, D, DV, rot, window, keep, page, n, dtype):
    """Keys are planted so that, for the last query, one key far back would win the softmax by a wide margin if it were
    seen: at the last kept position and the first one not kept, just inside and just outside the window, at a page's
    first and last row.  Whether it is seen follows the oracle's ``visible``; a kernel that is one off shows."""
    from types import SimpleNamespace
    from acvram_b200.kernels import ops
    rng = np.random.default_rng(NH * 100 + D)
    rs = {"base": 3000.0, "dims": rot, "scaling": {"factor": 2.0, "original": 64, "fast": 8.0, "slow": 1.0}}
    f, mag = pr.rotary_frequencies(rs)
    ang = np.arange(n + 8)[:, None] * f[None, :]
    table = dev(np.concatenate([np.cos(ang), np.sin(ang)], axis=1) * mag)
    scale, v_scale = 0.4, 0.6
    places = sorted({0, max(keep - 1, 0), keep, n - window - 1 if window else 5, n - window if window else 6, n - window + 1 if window else 7,
                     page - 1, page, n - page, n - 2})
    if n > 200:     # the long cases: the edges alone
        places = sorted({max(keep - 1, 0), keep, n - window - 1, n - window})
    if n > 1000:
        places = [keep - 1, keep]
    for place in places:
        x = bf(rng.standard_normal((n, NH * D + NKV * D + NKV * DV)))
        q = x[:, :NH * D].reshape(n, NH, D)
        k = x[:, NH * D:NH * D + NKV * D].reshape(n, NKV, D)
        # the planted key: along the last query of head 0 on the elements that do not turn, or, where the whole head turns,
        # simply long (its score then still stands out in size)
        if rot < D:
            k[place, 0, rot:] = bf(6.0 * q[n - 1, 0, rot:] / np.linalg.norm(q[n - 1, 0, rot:]) * math.sqrt(D))
        else:
            k[place, 0] = bf(5.0 * k[place, 0])
        v = x[:, NH * D + NKV * D:].reshape(n, NKV, DV)
        qr, kr = pr.rotate(q, rs, np.arange(n)), pr.rotate(k, rs, np.arange(n))
        want = np.zeros((n, NH, DV))
        for a in range(NH):
            g = a // (NH // NKV)
            s = (qr[:, a] @ kr[:, g].T) * scale
            for i in range(n):
                js = [j for j in range(i + 1) if pr.visible(i, j, window, keep)]
                w = np.exp(s[i, js] - s[i, js].max())
                want[i, a] = (w / w.sum()) @ (v[js, g] * v_scale)
        want = want.reshape(n, NH * DV)
        for cuts in ([n], [n - 1, 1], [37, 2, n - 50, 1, 1, 9], [n - 140, 130, 1] + [1] * 9) if n <= 1000 else ([n - 3, 1, 1, 1],):
            pc = Paged(n, NKV, D, DV, page, DT[dtype], place)
            got = np.zeros((n, NH * DV))
            at = 0
            for c in cuts:
                rows = dev(x[at:at + c], DT[dtype])
                pos, seq_of = i32(range(at, at + c)), i32([0] * c)
                ops.qk_norm_rope_append(rows, NH, NKV, D, None, None, 0.0, table, pos, seq_of, pc.table, pc.k, pc.v,
                                        table_rows=pc.rows, value_dim=DV, v_scale=v_scale)
                out = torch.empty((c, NH * DV), device=DEV, dtype=DT[dtype])
                ctx = SimpleNamespace(positions=pos, seq_of_token=seq_of, table_rows=pc.rows, cu_q=i32([0, c]), kv_len=i32([at + c]),
                                      work={})
                work = ops.attention_work([c], [at + c], [0, c])
                work = {**{k_: dev(v_, torch.int32) for k_, v_ in work[0].items()}, **work[1]}
                ops.attention(rows, out, pc.k, pc.v, ctx, pc.table, NH, NKV, D, scale, window, work=work, value_dim=DV, keep_first=keep)
                got[at:at + c] = out.float().cpu().numpy()
                at += c
            close(got, want, 3e-5 if dtype == "float32" else 4e-2, f"planted at {place}, cuts {cuts}")


# --------------------------------------------------------------------------- the tensor-core product with a bias
@pytest.mark.parametrize("M", [1, 8, 33, 200, 2048])
@pytest.mark.parametrize("N,K", [(96, 64), (512, 256), (2048, 2048), (1000, 4096)])
def test_tensor_core_product_adds_its_bias(M, N, K):
    """Few tokens (weights on the tensor core's rows, split K, tiles staged in shared memory) and many (tokens on the
    rows, pairs of CTAs): the bias joins the float accumulator in every epilogue, also in front of the paired SiLU."""
    from acvram_b200.kernels import ops
    g = torch.Generator(device="cpu").manual_seed(M * 7 + N)
    x = (torch.randn(M, K, generator=g) * 0.5).to(torch.bfloat16).to(DEV)
    w = (torch.randn(N, K, generator=g) / math.sqrt(K)).to(torch.bfloat16).to(DEV)
    bias = (torch.randn(N, generator=g) * 2.0).to(DEV)
    want = x.float() @ w.float().t() + bias
    for dtype in (torch.bfloat16, torch.float32):
        out = torch.empty(M, N, device=DEV, dtype=dtype)
        ops.gemm_tc(x, w, out, bias=bias)
        close(out, want.double().cpu().numpy(), 1e-2 if dtype == torch.bfloat16 else 2e-5, f"plain, {dtype}")
    gate, up = want[:, 0::2], want[:, 1::2]
    r = lambda t: t.to(torch.bfloat16).float()
    paired = r(r(torch.nn.functional.silu(r(gate))) * r(up))
    out = torch.empty(M, N // 2, device=DEV, dtype=torch.bfloat16)
    ops.gemm_tc(x, w, out, swiglu_pairs=True, bias=bias)
    close(out, paired.double().cpu().numpy(), 2e-2, "paired")


@pytest.mark.parametrize("T", [1, 64, 200])
@pytest.mark.parametrize("C,blocks", [(512, 2), (96, 3), (128, 8), (2048, 16)])
def test_gates_on_the_tensor_cores_equal_the_float_ones(C, blocks, T):
    """With inputs and weights that bfloat16 holds exactly the two forms compute the same sums (every product of two
    bfloat16 numbers is exact in float): they may differ by the order of the additions alone."""
    from acvram_b200.kernels import ops
    g = torch.Generator().manual_seed(C + T)
    bw = C // blocks
    u = torch.randn(T, C, generator=g).to(torch.bfloat16)
    wa = (torch.randn(blocks, bw, bw, generator=g) / math.sqrt(bw)).to(torch.bfloat16)
    wb = (torch.randn(blocks, bw, bw, generator=g) / math.sqrt(bw)).to(torch.bfloat16)
    ba, bb = torch.randn(C, generator=g).to(DEV), torch.randn(C, generator=g).to(DEV)
    sp = torch.rand(C, generator=g).to(DEV) * 0.7
    ud = u.float().to(DEV)
    wa_t, wb_t = wa.float().transpose(1, 2).contiguous().to(DEV), wb.float().transpose(1, 2).contiguous().to(DEV)
    a0, b0, a1, b1 = (torch.empty(T, C, device=DEV) for _ in range(4))
    ops.block_gates(ud, wa_t, ba, wb_t, bb, sp, -8.0, a0, b0)
    ops.block_gates(ud, wa_t, ba, wb_t, bb, sp, -8.0, a1, b1, bf16_weights=(wa.to(DEV), wb.to(DEV)))
    close(a1, a0.double().cpu().numpy(), 2e-5, "a")
    close(b1, b0.double().cpu().numpy(), 2e-5, "b")

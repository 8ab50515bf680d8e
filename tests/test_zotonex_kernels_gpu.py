"""The kernels of the Zotonex parts one by one, each against the oracle's function of the same mechanism on the same
(bfloat16-rounded) inputs, so that single positions can be judged sharply in both precisions: keys far away, at page
borders, just inside and just outside a chunk or a window, the first tokens, planted scores that stand out."""

from __future__ import annotations

import math
import random
from types import SimpleNamespace

import pytest
import torch

import plain_zotonex as pz
import zotonex_util as zu

pytestmark = pytest.mark.gpu

DEV = "cuda:0"


# --------------------------------------------------------------------------- differential attention
class PagedCase:
    """Requests with contexts of given lengths, the last ``q_lens`` tokens of each being this step's; pages handed out
    in a shuffled order so that neighbours in a request are no neighbours in memory."""

    def __init__(self, kv_lens, q_lens, NH, NKV, D, DV, page, dtype, seed, plant=None):
        from acvram_b200.kernels import ops
        g = torch.Generator().manual_seed(seed)
        self.kv_lens, self.q_lens, self.NH, self.NKV, self.D, self.DV = kv_lens, q_lens, NH, NKV, D, DV
        B = len(kv_lens)
        width = 2 * NH * D + 2 * NKV * D + NKV * DV
        self.rows = [torch.randn(n, width, generator=g).to(torch.bfloat16).double() for n in kv_lens]
        if plant:
            plant(self)
        self.q_w = (1 + 0.2 * torch.randn(D, generator=g)).to(torch.bfloat16).double()
        self.k_w = (1 + 0.2 * torch.randn(D, generator=g)).to(torch.bfloat16).double()
        n_pages = sum(-(-n // page) for n in kv_lens) + 3
        order = list(range(n_pages))
        random.Random(seed).shuffle(order)
        width_t = max(-(-n // page) for n in kv_lens) + 1
        table = torch.full((B + 2, width_t), -1, dtype=torch.int32)
        self.table_rows = torch.tensor([(i * 2 + 1) % (B + 1) if B > 1 else 0 for i in range(B)], dtype=torch.int32)
        assert len(set(self.table_rows.tolist())) == B
        for i, n in enumerate(kv_lens):
            for c in range(-(-n // page)):
                table[self.table_rows[i], c] = order.pop()
        self.table = table.to(DEV)
        self.k_pages = torch.zeros((n_pages, NKV, page, 2 * D), device=DEV, dtype=dtype)
        self.v_pages = torch.zeros((n_pages, NKV, page, DV), device=DEV, dtype=dtype)
        self.dtype, self.eps = dtype, 1e-5
        # every request's whole context goes through the append kernel (as one step), then this step's queries
        all_rows = torch.cat(self.rows).to(DEV, dtype)
        positions = torch.cat([torch.arange(n) for n in kv_lens]).to(DEV, torch.int32)
        seq_of = torch.cat([torch.full((n,), i) for i, n in enumerate(kv_lens)]).to(DEV, torch.int32)
        tr = self.table_rows.to(DEV)
        ops.heads_norm_append(all_rows, 2 * NH, 2 * NKV, NKV, D, DV, self.q_w.float().to(DEV), self.k_w.float().to(DEV), self.eps,
                              positions, seq_of, self.table, self.k_pages, self.v_pages, table_rows=tr)
        # this step's batch
        q_rows = torch.cat([r[n - q:] for r, n, q in zip(self.rows, kv_lens, q_lens)]).to(DEV, dtype)
        cu = [0]
        for q in q_lens:
            cu.append(cu[-1] + q)
        arrays, values = ops.attention_work(q_lens, kv_lens, cu)
        self.ctx = SimpleNamespace(
            positions=torch.cat([torch.arange(n - q, n) for n, q in zip(kv_lens, q_lens)]).to(DEV, torch.int32),
            seq_of_token=torch.cat([torch.full((q,), i) for i, q in enumerate(q_lens)]).to(DEV, torch.int32),
            cu_q=torch.tensor(cu, dtype=torch.int32, device=DEV), kv_len=torch.tensor(kv_lens, dtype=torch.int32, device=DEV),
            table_rows=tr, work={})
        self.work = {**{k: torch.as_tensor(v, dtype=torch.int32).to(DEV) for k, v in arrays.items()}, **values}
        self.q_rows = q_rows

    def oracle(self, scale, lam, diff, window, chunk):
        NH, NKV, D, DV = self.NH, self.NKV, self.D, self.DV
        outs = []
        for rows, n, q in zip(self.rows, self.kv_lens, self.q_lens):
            qv = pz.unit_rms(rows[n - q:, :2 * NH * D].view(q, NH, 2, D), self.eps) * self.q_w
            kv = pz.unit_rms(rows[:, 2 * NH * D:2 * NH * D + 2 * NKV * D].view(n, NKV, 2, D), self.eps) * self.k_w
            vv = rows[:, 2 * NH * D + 2 * NKV * D:].view(n, NKV, DV)
            if self.dtype == torch.bfloat16:       # what the pages and the query buffer hold
                qv, kv = qv.to(torch.bfloat16).double(), kv.to(torch.bfloat16).double()
            i = torch.arange(n - q, n)[:, None]
            j = torch.arange(n)[None, :]
            seen = j <= i
            if window:
                seen &= j > i - window
            if chunk:
                seen &= (i // chunk) == (j // chunk)
            outs.append(pz.diff_core(qv, kv, vv, seen, scale, lam, diff, self.eps))
        return torch.cat(outs)

    def run(self, path, scale, lam, diff, window, chunk):
        from acvram_b200.kernels import ops
        NH, NKV, D, DV = self.NH, self.NKV, self.D, self.DV
        T = self.q_rows.shape[0]
        qkv = self.q_rows.clone()
        out = torch.empty((T, NH * DV), device=DEV, dtype=self.dtype)
        qw, kw = self.q_w.float().to(DEV), self.k_w.float().to(DEV)
        if path == "generic":
            ops.heads_norm_append(qkv, 2 * NH, 2 * NKV, NKV, D, DV, qw, kw, self.eps, self.ctx.positions, self.ctx.seq_of_token,
                                  None, None, None)
            ops.diff_attention_generic(qkv, out, self.k_pages, self.v_pages, self.ctx.positions, self.ctx.seq_of_token, self.table,
                                       NH, NKV, D, DV, scale, lam, self.eps, 1.0 - diff, window, chunk, table_rows=self.ctx.table_rows)
        else:
            assert ops.diff_attention_as_heads_takes(self.dtype, NH, NKV, D, DV)
            wide = torch.empty((T, 4 * NH * D), device=DEV, dtype=self.dtype)
            ops.heads_norm_append(qkv, 2 * NH, 2 * NKV, NKV, D, DV, qw, kw, self.eps, self.ctx.positions, self.ctx.seq_of_token,
                                  None, None, None, q_out=wide)
            maps = torch.empty((T, 2 * NH * DV), device=DEV, dtype=torch.float32)
            ops.attention(wide, maps, self.k_pages, self.v_pages, self.ctx, self.table, 2 * NH, NKV, 2 * D, scale, window,
                          work=self.work, chunk=chunk)
            ops.diff_combine(maps, out, NH, DV, lam, self.eps, 1.0 - diff)
        torch.cuda.synchronize()
        return out.double().cpu()


def plant_scores(case):
    """Request 0's last query looks hard at key 2 (far back, first page) in map 1 and at key n - 9 in map 2; request 1's
    at the key just outside and the key just inside its chunk / window in the tests that have one."""
    NH, D = case.NH, case.D
    for r, targets in ((0, (2, case.kv_lens[0] - 9)), (1 % len(case.rows), (case.kv_lens[1 % len(case.rows)] - 24, case.kv_lens[1 % len(case.rows)] - 25))):
        rows = case.rows[r]
        n = rows.shape[0]
        if min(targets) < 0:
            continue
        for a, j in enumerate(targets):
            direction = rows[n - 1, a * D:(a + 1) * D].clone()          # head 0, map a of the last query
            k0 = 2 * NH * D + a * D
            rows[j, k0:k0 + D] = (direction * 6).to(torch.bfloat16).double()


CASES = [
    # kv_lens, q_lens: prompts whole and in part, beside requests that decode
    ("prompts", (150, 77, 1, 2), (150, 40, 1, 2)),
    ("decode", (333, 49, 200, 17), (1, 1, 1, 1)),
    ("mixed", (260, 130, 64, 5), (130, 1, 64, 1)),
]


@pytest.mark.parametrize("mask", [(0, 0), (0, 24), (0, 136), (40, 0), (0, 7)], ids=lambda m: f"window{m[0]}-chunk{m[1]}")
@pytest.mark.parametrize("name,kv_lens,q_lens", CASES, ids=[c[0] for c in CASES])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["float32", "bfloat16"])
def test_generic_kernel(dtype, name, kv_lens, q_lens, mask):
    case = PagedCase(kv_lens, q_lens, 3, 1, 24, 40, 8, dtype, 5, plant=plant_scores)      # sizes that are multiples of little
    window, chunk = mask
    got = case.run("generic", 0.31, 0.8, 0.3, window, chunk)
    err = zu.row_errors(got, case.oracle(0.31, 0.8, 0.3, window, chunk))
    assert float(err.max()) < (1e-4 if dtype == torch.float32 else 0.02), (float(err.max()), int(err.argmax()))


@pytest.mark.parametrize("mask", [(0, 0), (0, 24), (0, 136), (40, 0), (0, 129), (100, 64)], ids=lambda m: f"window{m[0]}-chunk{m[1]}")
@pytest.mark.parametrize("name,kv_lens,q_lens", CASES, ids=[c[0] for c in CASES])
@pytest.mark.parametrize("sizes", [(4, 2, 32, 16), (8, 1, 64, 16), (2, 2, 32, 64), (4, 1, 64, 32)], ids=lambda s: "h%d-g%d-d%d-page%d" % s)
def test_maps_as_heads_on_the_tensor_core_kernels(sizes, name, kv_lens, q_lens, mask):
    NH, NKV, D, page = sizes
    case = PagedCase(kv_lens, q_lens, NH, NKV, D, 2 * D, page, torch.bfloat16, 9, plant=plant_scores)
    window, chunk = mask
    scale = 1.0 / math.sqrt(D)
    got = case.run("heads", scale, 0.7, 0.25, window, chunk)
    want = case.oracle(scale, 0.7, 0.25, window, chunk)
    err = zu.row_errors(got, want)
    assert float(err.max()) < 0.03, (float(err.max()), int(err.argmax()))
    # and the planted keys decide: without them the answer would be another one
    generic = case.run("generic", scale, 0.7, 0.25, window, chunk)
    assert float(zu.row_errors(generic, want).max()) < 0.02


def test_planted_keys_matter():
    """The oracle's own answer moves by far more than the tests' bounds when a planted key is hidden."""
    case = PagedCase((333, 49), (1, 1), 2, 1, 32, 64, 16, torch.bfloat16, 9, plant=plant_scores)
    full = case.oracle(0.18, 0.7, 0.25, 0, 0)
    case.rows[0][2] = 0.0           # the far key of request 0
    case.rows[1][49 - 24] = 0.0
    assert float(zu.row_errors(case.oracle(0.18, 0.7, 0.25, 0, 0), full).min()) > 0.1


# --------------------------------------------------------------------------- mixture of experts
def moe_case(T, H, E, top, F, S, seed, dtype):
    g = torch.Generator().manual_seed(seed)
    r = lambda *shape, gain=1.0: (torch.randn(*shape, generator=g) * gain).to(torch.bfloat16)
    w = {"router": r(E, H, gain=2.0 / math.sqrt(H))}
    for e in range(E):
        w[f"e{e}.gate"], w[f"e{e}.up"], w[f"e{e}.down"] = r(F, H, gain=1.5 / math.sqrt(H)), r(F, H, gain=1.5 / math.sqrt(H)), r(H, F, gain=1 / math.sqrt(F))
    if S:
        w.update({"shared.gate": r(S, H, gain=1.5 / math.sqrt(H)), "shared.up": r(S, H, gain=1.5 / math.sqrt(H)),
                  "shared.down": r(H, S, gain=1 / math.sqrt(S)), "shared.sg": r(1, H, gain=2.0 / math.sqrt(H))})
    return r(T, H), w


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["float32", "bfloat16"])
@pytest.mark.parametrize("shape", [(1, 64, 3, 1, 48, 0), (5, 100, 5, 3, 36, 20), (300, 128, 8, 2, 72, 136), (77, 96, 6, 6, 40, 56),
                                   (130, 256, 16, 4, 192, 0), (700, 128, 8, 2, 80, 120), (520, 256, 16, 4, 192, 0),
                                   (1100, 64, 3, 1, 40, 24), (600, 2048, 8, 2, 64, 72)], ids=lambda s: "t%d-h%d-e%d-top%d-f%d-s%d" % s)
def test_routed_experts_part(shape, dtype):
    from acvram_b200.parts import PartSpec, Runtime, build
    T, H, E, top, F, S = shape
    h, w = moe_case(T, H, E, top, F, S, 3, dtype)
    part = build("feed_forward", PartSpec("moe", {"experts": E, "top": top, "expert_ff": F, "expert_limit": 1.25, "shared_ff": S,
                                                  "shared_limit": 0.75, "prefix": ""}), H)
    part.load(w, Runtime(torch.device(DEV), dtype))
    got = part.forward(h.to(DEV, dtype), None).double().cpu()
    f = {"router": {"experts": E, "top": top}, "expert": {"ff": F, "limit": 1.25}}
    if S:
        f["shared"] = {"ff": S, "limit": 0.75}
    want = pz.mixture(h.double(), {k: v.double() for k, v in w.items()}, f)
    err = zu.row_errors(got, want)
    # (from 1024 (token, choice) rows on, the bfloat16 run goes through the grouped tcgen05 product)
    # bfloat16: products are rounded to bfloat16 on their way (activations, the shared expert's output)
    assert float(err.max()) < (1e-4 if dtype == torch.float32 else 0.02), (float(err.max()), int(err.argmax()))


def test_routing_and_grouping():
    from acvram_b200.kernels import ops
    T, H, E, top = 200, 80, 7, 3
    g = torch.Generator().manual_seed(1)
    h = torch.randn(T, H, generator=g)
    router = torch.randn(E, H, generator=g) / math.sqrt(H)
    ids = torch.empty(T * top, device=DEV, dtype=torch.int32)
    weights = torch.empty(T * top, device=DEV, dtype=torch.float32)
    ops.moe_route(h.to(DEV), router.to(DEV), None, top, False, False, ids, weights, None)
    want_idx, want_w = pz.route(h.double(), router.double(), top)
    assert ids.view(T, top).cpu().tolist() == want_idx.tolist()
    assert torch.allclose(weights.view(T, top).cpu().double(), want_w, atol=1e-6)
    tiles = ops.moe_max_tiles(T * top, E)
    grouped = torch.empty(tiles * ops.MOE_TILE, device=DEV, dtype=torch.int32)
    place = torch.empty(T * top, device=DEV, dtype=torch.int32)
    tile_expert = torch.empty(tiles, device=DEV, dtype=torch.int32)
    ops.moe_group(ids, E, grouped, place, tile_expert)
    grouped, place, tile_expert, ids = grouped.cpu(), place.cpu(), tile_expert.cpu(), ids.cpu()
    n_used = int((tile_expert >= 0).sum())
    assert (tile_expert[:n_used] >= 0).all(), "the tiles in use come first"
    grouped = grouped[:n_used * ops.MOE_TILE]           # what lies behind the tiles in use is never read
    rows = grouped[grouped >= 0]
    assert sorted(rows.tolist()) == list(range(T * top)), "every (token, choice) row has one place"
    for at, r in enumerate(grouped.tolist()):
        if r >= 0:
            assert place[r] == at and tile_expert[at // ops.MOE_TILE] == ids[r]
    used = tile_expert[tile_expert >= 0]
    assert used.tolist() == sorted(used.tolist()), "experts follow one another in the grouped list"

"""Each kernel that the Tomalix family brought to include/b200_serve.h, alone, against the plain functions of
tomalix_oracle.py (or a line of torch): the residual update fused with the offset-weight RMS norm, rotary tables with an
amplitude, projected value stores of the q / k preparation, paged attention with a block mask, several score maps per
head and unequal key / value sizes, the map combination and the sigmoid gate, the causal convolution with silu and its
carried inputs, the selective scan with its carried state, the logits router, and the squared-relu GEMM epilogues."""
import ctypes as C
import math

import numpy as np
import pytest
import torch

import tomalix_oracle as O

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def S(pkg):
    if not torch.cuda.is_available():
        pytest.fail("no CUDA device: the library has no CPU path")
    return pkg.serve


_alive = []


def dev(t, dtype=None):
    t = torch.as_tensor(t).cuda()
    t = t.to(dtype).contiguous() if dtype is not None else t.contiguous()
    _alive.append(t)
    return t


def ints(a):
    return dev(torch.as_tensor(a, dtype=torch.int32))


@pytest.fixture(autouse=True)
def _drop_device_tensors():
    yield
    torch.cuda.synchronize()
    _alive.clear()


def tdt(S, code):
    return torch.bfloat16 if code == S.BF16 else torch.float32


def code_of(S, kind):
    return S.BF16 if kind == "bf16" else S.F32


def rel(got, want):
    return float((got.double().cpu() - want.double()).abs().max() / want.double().abs().max().clamp_min(1e-30))


def sync_ok(rc):
    assert rc == 0, f"rc={rc}"
    torch.cuda.synchronize()


def gen(seed):
    return torch.Generator().manual_seed(seed)


def ptr(t):
    return t.data_ptr() if t is not None else None


# ---------------------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("kind", ["f32", "bf16"])
@pytest.mark.parametrize("width", [1, 5, 48, 300, 2048, 5000, 9000])
def test_residual_update_with_the_next_norm(S, width, kind):
    code, g, T, top = code_of(S, kind), gen(width), 7, 3
    x, y1, y2 = (torch.randn(T, width, generator=g) for _ in range(3))
    eo = torch.randn(T * top, width, generator=g)
    dest = torch.randperm(T * top, generator=g).reshape(T, top).int()
    wt = torch.rand(T, top, generator=g)
    bc, w = torch.randn(width, generator=g), torch.randn(width, generator=g) * 0.2
    want_x = x.double() + 1.25 * y1.double() - 0.5 * y2.double() + bc.double() + \
        (wt.double()[:, :, None] * eo.double()[dest.long()]).sum(1)
    want_h = O.rms_norm(want_x, w.double(), 1e-5)
    dx, out = dev(x), torch.zeros(T, width, dtype=tdt(S, code), device="cuda")
    a = S.RmsnormResidualArgs(dx.data_ptr(), dev(y1).data_ptr(), 1.25, dev(y2).data_ptr(), -0.5, dev(eo).data_ptr(), dev(dest).data_ptr(),
                              dev(wt).data_ptr(), top, dev(bc).data_ptr(), None, dev(w).data_ptr(), 1.0, 1e-5, out.data_ptr(), code, T, width)
    sync_ok(S.lib().b200_rmsnorm_residual(C.byref(a), None))
    assert rel(dx, want_x) < 1e-6
    assert rel(out.float(), want_h) < (1e-2 if kind == "bf16" else 1e-5)
    # listed rows only, nothing added, a weight stored around one; then an update without a norm
    rows = [5, 0, 5]
    out2 = torch.zeros(3, width, dtype=tdt(S, code), device="cuda")
    a = S.RmsnormResidualArgs(dx.data_ptr(), None, 0.0, None, 0.0, None, None, None, 0, None, ints(rows).data_ptr(), dev(w).data_ptr(), 0.0, 1e-5,
                              out2.data_ptr(), code, 3, width)
    sync_ok(S.lib().b200_rmsnorm_residual(C.byref(a), None))
    assert rel(dx, want_x) < 1e-6
    assert rel(out2.float(), O.unit_rms(want_x[rows], 1e-5) * w.double()) < (1e-2 if kind == "bf16" else 1e-5)
    a = S.RmsnormResidualArgs(dx.data_ptr(), dev(y1).data_ptr(), 1.0, None, 0.0, None, None, None, 0, None, None, None, 0.0, 1e-5, None, code, T, width)
    sync_ok(S.lib().b200_rmsnorm_residual(C.byref(a), None))
    assert rel(dx, want_x + y1.double()) < 1e-6


def test_rope_tables_with_an_amplitude(S):
    pos = [0, 1, 77, 100000]
    f, amp = O.rot_frequencies(dict(dims=12, base=50.0, scaling=dict(factor=4.0, original=32, fast=8.0, slow=1.0)), "ramp")
    assert amp == pytest.approx(0.1 * math.log(4.0) + 1) and float(f[0]) == 1.0 and float(f[-1]) == pytest.approx(50.0 ** (-10 / 12) / 4)
    c, s = torch.zeros(4, 6, device="cuda"), torch.zeros(4, 6, device="cuda")
    sync_ok(S.lib().b200_rope_angles_amp(ints(pos).data_ptr(), 4, dev(f).data_ptr(), 6, amp, c.data_ptr(), s.data_ptr(), None))
    ang = torch.tensor(pos, dtype=torch.float64)[:, None] * f[None]
    assert rel(c, amp * torch.cos(ang)) < 1e-6 and rel(s, amp * torch.sin(ang)) < 1e-6


def paged(S, code, k, v, PR, perm_seed):
    """k, v: dict slot -> [n, units, d]; scatters them into shuffled pages. Returns pools, page table, max_pages"""
    n_slots, max_pages = len(k), max((len(x) + PR - 1) // PR for x in k.values())
    total = n_slots * max_pages + 3
    order = torch.randperm(total, generator=gen(perm_seed)).tolist()
    table = torch.zeros(n_slots, max_pages, dtype=torch.int32)
    k0, v0 = next(iter(k.values())), next(iter(v.values()))
    kp = torch.full((total * PR, k0.shape[1], k0.shape[2]), 300.0)    # rows nobody owns would dominate every softmax if they were read
    vp = torch.full((total * PR, v0.shape[1], v0.shape[2]), -500.0)
    for b in k:
        for i in range((len(k[b]) + PR - 1) // PR):
            pg = order.pop()
            table[b, i] = pg
            n = min(PR, len(k[b]) - i * PR)
            kp[pg * PR: pg * PR + n] = k[b][i * PR: i * PR + n]
            vp[pg * PR: pg * PR + n] = v[b][i * PR: i * PR + n]
    return dev(kp, tdt(S, code)), dev(vp, tdt(S, code)), dev(table), max_pages


def run_attention(S, code, q, slot, pos, kp, vp, table, max_pages, PR, heads, kv, dim, vdim, scale, longest, chunk=0, maps=1, f32_out=False):
    T = len(slot)
    out = torch.empty(T, heads * maps * vdim, dtype=torch.float32 if f32_out else tdt(S, code), device="cuda")
    need = S.lib().b200_paged_attention_workspace_bytes(T, heads * maps, vdim)
    ws = torch.empty(max(need, 16), dtype=torch.uint8, device="cuda")
    _alive.append(ws)
    a = S.PagedAttentionArgs(dev(q, tdt(S, code)).data_ptr(), out.data_ptr(), kp.data_ptr(), vp.data_ptr(), table.data_ptr(), max_pages, PR,
                             ints(slot).data_ptr(), ints(pos).data_ptr(), T, heads, kv, dim, vdim, scale, 0.0, 0.0, code, longest,
                             max(pos) + 1, ws.data_ptr(), need, chunk, maps, int(f32_out))
    sync_ok(S.lib().b200_paged_attention(C.byref(a), None))
    return out.float().cpu()


def plain_maps(q, k, v, pos, heads, kv, maps, scale, chunk):
    """q [T, heads, maps, d] at positions pos of ONE sequence; k [n, kv, maps, d], v [n, kv, dv] -> [T, heads * maps * dv]"""
    out = []
    for t, p in enumerate(pos):
        lo = (p // chunk) * chunk if chunk else 0
        row = []
        for h in range(heads):
            g = h // (heads // kv)
            for m in range(maps):
                s = (k[lo: p + 1, g, m] @ q[t, h, m]) * scale
                row.append(torch.softmax(s, 0) @ v[lo: p + 1, g])
        out.append(torch.cat(row))
    return torch.stack(out)


@pytest.mark.parametrize("kind", ["f32", "bf16"])
@pytest.mark.parametrize("heads,kv,dim,vdim,chunk,maps", [(4, 2, 16, 8, 7, 1), (6, 1, 64, 64, 40, 1), (3, 3, 10, 6, 0, 2), (2, 1, 32, 64, 0, 2),
                                                          (8, 2, 64, 128, 16, 1), (4, 1, 128, 128, 100, 2), (2, 2, 48, 48, 0, 1),
                                                          (2, 1, 128, 256, 0, 2), (4, 4, 128, 256, 50, 1), (2, 2, 32, 32, 5, 1), (4, 2, 32, 64, 33, 2)])
def test_paged_attention_with_blocks_and_maps(S, kind, heads, kv, dim, vdim, chunk, maps):
    code, g = code_of(S, kind), gen(heads * dim + chunk)
    PR, scale = 16, 1.7 / math.sqrt(dim)
    lens = {0: 150, 1: 33, 2: 1}
    bf = (lambda t: t.bfloat16().float()) if kind == "bf16" else (lambda t: t)
    k = {b: bf(torch.randn(n, kv, maps, dim, generator=g)) for b, n in lens.items()}
    v = {b: bf(torch.randn(n, kv, vdim, generator=g)) for b, n in lens.items()}
    q = {b: bf(torch.randn(n, heads, maps, dim, generator=g)) for b, n in lens.items()}
    kp, vp, table, max_pages = paged(S, code, {b: x.reshape(len(x), kv * maps, dim) for b, x in k.items()}, v, PR, 5)
    tol = 2e-2 if kind == "bf16" else 2e-5
    # whole prompts of unequal length in one batch; the last tokens alone (a decode batch); portions beside single tokens
    batches = [[(0, 0, 150), (1, 0, 33), (2, 0, 1)], [(0, 149, 150), (1, 32, 33)], [(1, 15, 33), (0, 149, 150)], [(0, 61, 131), (2, 0, 1), (1, 16, 17)]]
    for batch in batches:
        rows = [(b, p) for b, lo, hi in batch for p in range(lo, hi)]
        slot, pos = [b for b, _ in rows], [p for _, p in rows]
        qq = torch.stack([q[b][p] for b, p in rows]).reshape(len(rows), heads * maps * dim)
        longest = max(hi - lo for _, lo, hi in batch)
        want = torch.cat([plain_maps(q[b][lo:hi].double(), k[b].double(), v[b].double(), list(range(lo, hi)), heads, kv, maps, scale, chunk)
                          for b, lo, hi in batch])
        for f32_out in (False, True):
            got = run_attention(S, code, qq, slot, pos, kp, vp, table, max_pages, PR, heads, kv, dim, vdim, scale, longest, chunk, maps, f32_out)
            assert rel(got, want) < tol, (batch, f32_out)


@pytest.mark.parametrize("kind", ["f32", "bf16"])
@pytest.mark.parametrize("chunk,edge", [(48, 0), (48, 1), (64, 0), (64, 1), (100, 0), (100, 1), (0, 0)])
def test_a_key_at_the_edge_of_a_block(S, kind, chunk, edge):
    """one key among hundreds matches the query. Without a mask (chunk 0) it is the very first key, far away. With blocks
    it is the first key of the query's block (edge 0: its value must come through, in a prompt portion and decoded) or the
    last key of the block before (edge 1: it must not be seen at all), also where the block border is a page border."""
    code, g = code_of(S, kind), gen(chunk + edge)
    heads, kv, dim, vdim, PR, n = 2, 1, 32, 16, 16, 700
    k = torch.randn(n, kv, dim, generator=g) * 0.05
    v = torch.randn(n, kv, vdim, generator=g)
    p_query = n - 1
    lo = (p_query // chunk) * chunk if chunk else 0
    hot = lo - edge
    k[hot, 0, :] = 1.0
    q = torch.randn(2, heads, dim, generator=g) * 0.05       # the last token of a prompt portion, and the same decoded
    q[:, 1, :] = 1.0                                          # head 1 looks for the hot key: raw score = dim * scale
    if kind == "bf16":
        k, v, q = k.bfloat16().float(), v.bfloat16().float(), q.bfloat16().float()
    kp, vp, table, max_pages = paged(S, code, {0: k}, {0: v}, PR, 9)
    want = plain_maps(q.double()[:, :, None], k.double()[:, :, None], v.double(), [p_query - 1, p_query], heads, kv, 1, 0.5, chunk)
    close = (want[1, vdim:] - v[hot, 0].double()).abs().max()
    assert close < 0.05 if edge == 0 else close > 0.3         # the case is what it says: seen and dominant, or absent
    for longest in (2, 1):
        got = run_attention(S, code, q.reshape(2, heads * dim), [0, 0], [p_query - 1, p_query], kp, vp, table, max_pages, PR, heads, kv, dim, vdim,
                            0.5, longest, chunk)
        assert rel(got, want) < (2e-2 if kind == "bf16" else 2e-5), longest


@pytest.mark.parametrize("kind", ["f32", "bf16"])
@pytest.mark.parametrize("H,G,maps,d,dv,rot,pad", [(3, 1, 2, 10, 6, 4, 3), (3, 1, 2, 16, 8, 8, 4), (2, 2, 1, 64, 128, 64, 0), (4, 2, 1, 32, 32, 0, 8),
                                                     (2, 1, 1, 24, 20, 16, 4), (2, 1, 1, 16, 8, 12, 0)])
def test_qk_prepare_stores_projected_values(S, kind, H, G, maps, d, dv, rot, pad):
    """two score maps per head as twice the heads, partial rotate-half rotation with an amplitude, values copied as they are;
    sizes in whole groups of four take the vector kernel, the others (and a rotated part of 12) the warp-per-head one"""
    code, g = code_of(S, kind), gen(3)
    PR = 4
    lens = {0: 9, 1: 5}
    n_in = H * maps * d + G * maps * d + G * dv + pad        # unrelated columns behind the values
    rows = [(b, p) for b, n in lens.items() for p in range(n)]
    T = len(rows)
    proj = torch.randn(T, n_in, generator=g)
    sc = dict(dims=rot, base=100.0, scaling=dict(factor=2.0, original=16, fast=4.0, slow=1.0))
    slot, pos = [b for b, _ in rows], [p for _, p in rows]
    cs, sn = torch.zeros(T, max(rot // 2, 1), device="cuda"), torch.zeros(T, max(rot // 2, 1), device="cuda")
    if rot:
        f, amp = O.rot_frequencies(sc, "ramp")
        sync_ok(S.lib().b200_rope_angles_amp(ints(pos).data_ptr(), T, dev(f).data_ptr(), rot // 2, amp, cs.data_ptr(), sn.data_ptr(), None))
    table = dev(torch.tensor([[2, 0, 5], [4, 1, 3]], dtype=torch.int32))
    kp = torch.full((6 * PR, G * maps, d), 7.0, dtype=tdt(S, code), device="cuda")
    vp = torch.full((6 * PR, G, dv), 7.0, dtype=tdt(S, code), device="cuda")
    qo = torch.zeros(T, H * maps * d, dtype=tdt(S, code), device="cuda")
    v_off = (H + G) * maps * d
    a = S.QkPrepareArgs(dev(proj).data_ptr(), n_in, None, 1, None, None, None, 1e-5, cs.data_ptr(), sn.data_ptr(), rot, S.ROPE_HALF,
                        qo.data_ptr(), kp.data_ptr(), vp.data_ptr(), 0, table.data_ptr(), 3, PR, ints(slot).data_ptr(), ints(pos).data_ptr(),
                        ints([0] * T).data_ptr(), T, H * maps, G * maps, d, code, 0, G, dv, v_off)
    sync_ok(S.lib().b200_qk_prepare(C.byref(a), None))
    tol = 1e-2 if kind == "bf16" else 1e-6
    for b, n in lens.items():
        idx = [i for i, (bb, _) in enumerate(rows) if bb == b]
        wq = O.rotate_half(proj[idx, : H * maps * d].double().reshape(n, H * maps, d), sc, "ramp")
        wk = O.rotate_half(proj[idx, H * maps * d: v_off].double().reshape(n, G * maps, d), sc, "ramp")
        assert rel(qo[idx].float().reshape(n, H * maps, d), wq) < tol
        for p in range(n):
            row = int(table[b, p // PR]) * PR + p % PR
            assert rel(kp[row].float(), wk[p]) < tol
            assert rel(vp[row].float().reshape(-1), proj[idx[p], v_off: v_off + G * dv].double()) < tol


@pytest.mark.parametrize("kind", ["f32", "bf16"])
def test_map_combination_and_gate(S, kind):
    code, g = code_of(S, kind), gen(8)
    T, H, dv, lam = 5, 3, 20, 0.37
    a = torch.randn(T, H, 2, dv, generator=g)
    out = torch.zeros(T, H * dv, dtype=tdt(S, code), device="cuda")
    sync_ok(S.lib().b200_diff_combine(dev(a).data_ptr(), lam, 1e-5, 0.7, out.data_ptr(), T, H, dv, code, None))
    want = O.unit_rms(a[:, :, 0].double() - lam * a[:, :, 1].double(), 1e-5) * 0.7
    assert rel(out.float().reshape(T, H, dv), want) < (1e-2 if kind == "bf16" else 1e-6)
    o, gate = torch.randn(T, 33, generator=g), torch.randn(T, 50, generator=g)
    out = torch.zeros(T, 33, dtype=tdt(S, code), device="cuda")
    sync_ok(S.lib().b200_sigmoid_gate(dev(o).data_ptr(), dev(gate).data_ptr() + 4 * 9, 50, out.data_ptr(), T, 33, code, None))
    assert rel(out.float(), o.double() * torch.sigmoid(gate[:, 9:42].double())) < (1e-2 if kind == "bf16" else 1e-6)


@pytest.mark.parametrize("taps", [1, 2, 3, 5])
def test_convolution_with_carried_inputs(S, taps):
    """two sequences in portions (two tokens, one token, many), stale ring contents in the slots, against the whole"""
    g, Cn, ld = gen(taps), 37, 45
    lens = {0: 23, 1: 11}
    u = {b: torch.randn(n, ld, generator=g) for b, n in lens.items()}
    w, bias = torch.randn(Cn, taps, generator=g), torch.randn(Cn, generator=g)
    want = {b: O.silu(O.causal_conv(u[b][:, 3: 3 + Cn].double(), w.double(), bias.double())) for b in lens}
    ring = dev(torch.full((2, max(taps - 1, 1), Cn), 55.0))
    plan = [[(0, 2), (1, 1)], [(0, 1), (1, 2)], [(0, 1), (1, 1)], [(0, 19), (1, 7)]]
    at = {0: 0, 1: 0}
    for step in plan:
        rows = [(b, at[b] + i, at[b], at[b] + c) for b, c in step for i in range(c)]
        T = len(rows)
        x = dev(torch.cat([u[b][at[b]: at[b] + c] for b, c in step]))
        slot, pos, start, end = (ints([r[k] for r in rows]) for k in range(4))
        o32, o16 = torch.zeros(T, Cn, device="cuda"), torch.zeros(T, Cn, dtype=torch.bfloat16, device="cuda")
        inline = all(c == 1 for _, c in step)
        a = S.ConvActArgs(x.data_ptr() + 4 * 3, ld, dev(w).data_ptr(), dev(bias).data_ptr(), taps, ring.data_ptr(), o32.data_ptr(), o16.data_ptr(),
                          S.BF16, slot.data_ptr(), pos.data_ptr(), start.data_ptr(), T, Cn, int(inline))
        sync_ok(S.lib().b200_conv_act(C.byref(a), None))
        if not inline:
            sync_ok(S.lib().b200_conv_state_update(x.data_ptr() + 4 * 3, ld, ring.data_ptr(), slot.data_ptr(), pos.data_ptr(), end.data_ptr(), T, Cn,
                                                   taps, None))
        wnt = torch.cat([want[b][at[b]: at[b] + c] for b, c in step])
        assert rel(o32, wnt) < 1e-6 and rel(o16.float(), wnt) < 1e-2, step
        for b, c in step:
            at[b] += c


def plain_scan(x, dt_raw, dt_b, B, Cm, z, A, D):
    Cn, N = A.shape
    S_ = torch.zeros(Cn, N, dtype=torch.float64)
    out = []
    for t in range(len(x)):
        dt = O.softplus(dt_raw[t] + dt_b)
        S_ = torch.exp(dt[:, None] * A) * S_ + (dt * x[t])[:, None] * B[t][None]
        out.append((S_ @ Cm[t] + D * x[t]) * O.silu(z[t]))
    return torch.stack(out), S_


@pytest.mark.parametrize("Cn,N", [(37, 1), (20, 5), (64, 16), (9, 70), (130, 32), (33, 8), (12, 256), (5, 24)])
def test_selective_scan_in_portions_with_a_carried_state(S, Cn, N):
    """two sequences; portions of one, two and hundreds of tokens (the chunk form); a stale state in both slots. State counts
    of 8 per lane with 16-byte aligned B / C rows take the vector-load form of the kernel, the others the predicated one"""
    g = gen(Cn + N)
    lens = {0: 700, 1: 90}
    off = 4 if N % 8 == 0 else 1                      # first B column in the [.. | B | C | ..] rows
    ld_bc, ld_z = 2 * N + off + (4 - off % 4) % 4 + (0 if N % 8 == 0 else 2), Cn + 2
    mk = lambda n, c, s=1.0: torch.randn(n, c, generator=g) * s
    x, dtr, bc, z = ({b: mk(n, c, s) for b, n in lens.items()} for c, s in ((Cn, 1.0), (Cn, 1.0), (ld_bc, 1.0), (ld_z, 1.0)))
    A = -torch.exp(torch.randn(Cn, N, generator=g) * 0.5)
    D, dtb = torch.randn(Cn, generator=g), torch.randn(Cn, generator=g) * 0.5 - 1.5
    want = {b: plain_scan(x[b].double(), dtr[b].double(), dtb.double(), bc[b][:, off: off + N].double(), bc[b][:, off + N: off + 2 * N].double(),
                          z[b][:, 2:].double(), A.double(), D.double()) for b in lens}
    state = dev(torch.full((3, Cn, N), 9.0))
    plan = [[(1, 1), (0, 2)], [(0, 1)], [(0, 1), (1, 2)], [(0, 600), (1, 80)], [(1, 7), (0, 96)]]
    at = {0: 0, 1: 0}
    slot_of = {0: 2, 1: 0}
    for step in plan:
        T = sum(c for _, c in step)
        cat = lambda d: dev(torch.cat([d[b][at[b]: at[b] + c] for b, c in step]))
        dx, ddt, dbc, dz = cat(x), cat(dtr), cat(bc), cat(z)
        ent_row, r = [], 0
        for _, c in step:
            ent_row.append(r)
            r += c
        slot = ints([slot_of[b] for b, c in step for _ in range(c)])
        pos = ints([at[b] + i for b, c in step for i in range(c)])
        out = torch.zeros(T, Cn, device="cuda")
        need = S.lib().b200_selective_scan_workspace_bytes(T, len(step), Cn, N)
        ws = torch.empty(max(need, 16), dtype=torch.uint8, device="cuda")
        a = S.SelectiveScanArgs(dx.data_ptr(), ddt.data_ptr(), dev(dtb).data_ptr(), dbc.data_ptr() + 4 * off, dbc.data_ptr() + 4 * (off + N), ld_bc,
                                dz.data_ptr() + 8, ld_z, dev(A).data_ptr(), dev(D).data_ptr(), state.data_ptr(), out.data_ptr(), S.F32,
                                ints(ent_row).data_ptr(), ints([c for _, c in step]).data_ptr(), slot.data_ptr(), pos.data_ptr(),
                                len(step), T, Cn, N, max(c for _, c in step), ws.data_ptr(), need)
        sync_ok(S.lib().b200_selective_scan(C.byref(a), None))
        wnt = torch.cat([want[b][0][at[b]: at[b] + c] for b, c in step])
        assert rel(out, wnt) < 3e-5, step
        for b, c in step:
            at[b] += c
    for b in lens:
        assert rel(state[slot_of[b]], want[b][1]) < 3e-5
    assert bool((state[1] == 9.0).all())


@pytest.mark.parametrize("kind", ["f32", "bf16"])
def test_router_on_logits_and_routed_squared_relu_experts(S, kind):
    code, g = code_of(S, kind), gen(4)
    T, D, E, top, ff = 50, 40, 6, 3, 24
    bf = (lambda t: t.bfloat16().float()) if kind == "bf16" else (lambda t: t)
    h, wr, br = bf(torch.randn(T, D, generator=g)), torch.randn(E, D, generator=g), torch.randn(E, generator=g)
    up, down = bf(torch.randn(E, ff, D, generator=g) / 6), bf(torch.randn(E, D, ff, generator=g) / 5)
    chosen, weight = torch.zeros(T, top, dtype=torch.int32, device="cuda"), torch.zeros(T, top, device="cuda")
    sync_ok(S.lib().b200_moe_route_logits(dev(h, tdt(S, code)).data_ptr(), code, dev(wr).data_ptr(), dev(br).data_ptr(), T, D, E, top,
                                          chosen.data_ptr(), weight.data_ptr(), None))
    zl = h.double() @ wr.double().T + br.double()
    val, idx = torch.topk(zl, top, dim=-1)
    assert chosen.cpu().tolist() == idx.tolist()
    assert rel(weight, torch.softmax(val, -1)) < 1e-5
    group_off = torch.zeros(E + 1, dtype=torch.int32, device="cuda")
    src_row, dest = torch.zeros(T * top, dtype=torch.int32, device="cuda"), torch.zeros(T, top, dtype=torch.int32, device="cuda")
    sync_ok(S.lib().b200_moe_dispatch(chosen.data_ptr(), T, top, E, group_off.data_ptr(), src_row.data_ptr(), dest.data_ptr(), None))
    act = torch.zeros(T * top, ff, dtype=tdt(S, code), device="cuda")
    eo = torch.zeros(T * top, D, device="cuda")
    dh, dup, ddown = dev(h, tdt(S, code)), dev(up, tdt(S, code)), dev(down, tdt(S, code))
    a = S.GemmGroupedArgs(dh.data_ptr(), dup.data_ptr(), act.data_ptr(), None, src_row.data_ptr(), group_off.data_ptr(), D, D, ff, 0,
                          0, ff * D, 0, 0, T, ff, D, E, 1, S.GG_RELU2, code, code, code)
    sync_ok(S.lib().b200_gemm_grouped(C.byref(a), None))
    a = S.GemmGroupedArgs(act.data_ptr(), ddown.data_ptr(), eo.data_ptr(), None, None, group_off.data_ptr(), ff, ff, D, 0,
                          0, D * ff, 0, 0, T, D, ff, E, 1, S.GG_NONE, code, code, S.F32)
    sync_ok(S.lib().b200_gemm_grouped(C.byref(a), None))
    x = torch.zeros(T, D, device="cuda")
    ra = S.RmsnormResidualArgs(x.data_ptr(), None, 0.0, None, 0.0, eo.data_ptr(), dest.data_ptr(), weight.data_ptr(), top, None, None, None, 0.0,
                               1e-5, None, code, T, D)
    sync_ok(S.lib().b200_rmsnorm_residual(C.byref(ra), None))
    W = {"router": wr.double(), "router.b": br.double()}
    for e in range(E):
        W["e%d.up" % e], W["e%d.down" % e] = up[e].double(), down[e].double()
    want = O.routed_ff(h.double(), dict(router=dict(experts=E, top=top)), W, "")
    assert rel(x, want) < (3e-2 if kind == "bf16" else 2e-5)


@pytest.mark.parametrize("kind", ["f32", "bf16"])
@pytest.mark.parametrize("M,N,K", [(3, 40, 24), (130, 256, 64), (300, 136, 72), (257, 31, 19)])
def test_squared_relu_in_the_gemm_epilogue(S, M, N, K, kind):
    code, g = code_of(S, kind), gen(M + N)
    bf = (lambda t: t.bfloat16().float()) if kind == "bf16" else (lambda t: t)
    x, w = bf(torch.randn(M, K, generator=g)), bf(torch.randn(N, K, generator=g) / math.sqrt(K))
    need = S.lib().b200_linear_ex_workspace_bytes(M, N, K)
    ws = torch.empty(max(need, 16), dtype=torch.uint8, device="cuda")
    for out_code in (code, S.F32):
        y = torch.zeros(M, N, dtype=tdt(S, out_code), device="cuda")
        sync_ok(S.lib().b200_linear_ex(dev(x, tdt(S, code)).data_ptr(), dev(w, tdt(S, code)).data_ptr(), y.data_ptr(), M, N, K, code, out_code,
                                       S.GG_RELU2, ws.data_ptr(), need, None))
        assert rel(y.float(), O.relu2(x.double() @ w.double().T)) < (1e-2 if out_code == S.BF16 else 2e-5)

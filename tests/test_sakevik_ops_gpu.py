"""Each kernel (or kernel option) that the Sakevik family brought to include/b200_serve.h, alone, against the plain
functions of sakevik_oracle.py (or a line of torch): the hashed pair embedding, the residual update with the norm on the
addend, biases and value rotation in the q / k preparation, paged attention with a sliding window and sigmoid weights
(row, group, tile and split forms; keys just inside and just outside the window made to stand out), the turn back of
rotated outputs with head gates, latent attention over rows with a rotated part, a window and no sink, the gated
recurrence with its carried state (direct and chunked), the clamped gated unit as activation kernel and GEMM epilogue."""
import ctypes as C
import math

import numpy as np
import pytest
import torch

import sakevik_oracle as O

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


def rounded(t, kind):
    return t.to(torch.bfloat16).double() if kind == "bf16" else t.float().double()


def tables(S, pos, freqs, amp=1.0):
    """cos / sin [T, n] of the positions through the library's own table kernel"""
    n = len(freqs)
    c, s = torch.zeros(len(pos), n, device="cuda"), torch.zeros(len(pos), n, device="cuda")
    _alive.extend([c, s])
    sync_ok(S.lib().b200_rope_angles_amp(ints(pos).data_ptr(), len(pos), dev(torch.tensor(freqs, dtype=torch.float64)).data_ptr(), n, amp,
                                         c.data_ptr(), s.data_ptr(), None))
    return c, s


# ---------------------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("kind", ["f32", "bf16"])
def test_hashed_pair_embedding(S, kind):
    code, g, V, D, B = code_of(S, kind), gen(1), 50, 24, 13
    table, pair = rounded(torch.randn(V, D, generator=g), "bf16"), rounded(torch.randn(B + 1, D, generator=g), "bf16")
    ids = [3, 49, 0, 17, 17, 2]
    prev = [-1, 3, 49, -1, 17, 48]
    cfg = dict(embedding=dict(scale=2.5, bigram=dict(buckets=B, mul_prev=2000000011, mul_cur=77777)))
    x, h = torch.zeros(6, D, device="cuda"), torch.zeros(6, D, dtype=tdt(S, code), device="cuda")
    sync_ok(S.lib().b200_embed_pair_hash(ints(ids).data_ptr(), ints(prev).data_ptr(), dev(table, tdt(S, code)).data_ptr(), 2.5,
                                         dev(pair, tdt(S, code)).data_ptr(), B, 2000000011, 77777, x.data_ptr(), h.data_ptr(), 6, D, code, None))
    # the oracle on the two sequences [3, 49, 0] and [17, 17]; the last row by hand (products beyond 32 bits)
    want = torch.cat([O.embed(cfg, dict(embed=table, bigram=pair), [3, 49, 0]), O.embed(cfg, dict(embed=table, bigram=pair), [17, 17])])
    assert rel(x[:5], want) < 1e-6
    row = (prev[5] * 2000000011 + 2 * 77777) % B
    assert rel(x[5], table[2] * 2.5 + pair[row]) < 1e-6
    assert rel(h.float(), x.cpu()) < (1e-2 if kind == "bf16" else 1e-7)
    # no pair table: the scaled rows alone
    sync_ok(S.lib().b200_embed_pair_hash(ints(ids).data_ptr(), None, dev(table, tdt(S, code)).data_ptr(), 0.5, None, 0, 0, 0, x.data_ptr(), None, 6, D,
                                         code, None))
    assert rel(x, table[ids] * 0.5) < 1e-6


@pytest.mark.parametrize("kind", ["f32", "bf16"])
@pytest.mark.parametrize("width", [1, 5, 48, 300, 2048, 5000, 9000])
def test_residual_update_with_the_norm_on_the_addend(S, width, kind):
    code, g, T = code_of(S, kind), gen(width), 6
    x, y = torch.randn(T, width, generator=g), torch.randn(T, width, generator=g) * 3
    b, w = torch.randn(width, generator=g), 1 + torch.randn(width, generator=g) * 0.2
    dx, out = dev(x), torch.zeros(T, width, dtype=tdt(S, code), device="cuda")
    a = S.RmsnormResidualArgs()
    a.x, a.y1, a.w, a.w_offset, a.eps, a.out, a.out_dtype = dx.data_ptr(), dev(y).data_ptr(), dev(w).data_ptr(), 0.0, 1e-5, out.data_ptr(), code
    a.n_rows, a.width, a.norm_addend, a.y_bias = T, width, 1, dev(b).data_ptr()
    sync_ok(S.lib().b200_rmsnorm_residual(C.byref(a), None))
    want = x.double() + O.rms_norm(y.double() + b.double(), w.double(), 1e-5)
    assert rel(dx, want) < 2e-6
    assert rel(out.float(), want) < (1e-2 if kind == "bf16" else 2e-6)
    a.y_bias, a.out = None, None          # no bias, nobody reads the row next
    sync_ok(S.lib().b200_rmsnorm_residual(C.byref(a), None))
    assert rel(dx, want + O.rms_norm(y.double(), w.double(), 1e-5)) < 2e-6


def paged(S, code, k, v, PR, perm_seed):
    """k, v: dict slot -> [n, units, d]; scatters them into shuffled pages. Returns pools, page table, max_pages"""
    n_slots, max_pages = len(k), max((len(x) + PR - 1) // PR for x in k.values())
    total = n_slots * max_pages + 3
    order = torch.randperm(total, generator=gen(perm_seed)).tolist()
    table = torch.zeros(n_slots, max_pages, dtype=torch.int32)
    k0, v0 = next(iter(k.values())), next(iter(v.values()))
    kp = torch.full((total * PR, k0.shape[1], k0.shape[2]), 300.0)    # rows nobody owns would dominate if they were read
    vp = torch.full((total * PR, v0.shape[1], v0.shape[2]), -500.0)
    for b in k:
        for i in range((len(k[b]) + PR - 1) // PR):
            pg = order.pop()
            table[b, i] = pg
            n = min(PR, len(k[b]) - i * PR)
            kp[pg * PR: pg * PR + n] = k[b][i * PR: i * PR + n]
            vp[pg * PR: pg * PR + n] = v[b][i * PR: i * PR + n]
    return dev(kp, tdt(S, code)), dev(vp, tdt(S, code)), dev(table), max_pages


def plain_sigmoid_attention(q, k, v, pos, window, scale, hb):
    """q [T, H, d] at positions pos of ONE sequence whose keys k [n, G, d], values v [n, G, dv] start at position 0"""
    T, H, _ = q.shape
    G = k.shape[1]
    out = torch.zeros(T, H, v.shape[2], dtype=torch.float64)
    for i, p in enumerate(pos):
        lo = max(0, p - window + 1) if window else 0
        for h in range(H):
            g = h // (H // G)
            w = torch.sigmoid((k[lo: p + 1, g] @ q[i, h]) * scale + hb[h])
            out[i, h] = w @ v[lo: p + 1, g]
    return out


ATT_SHAPES = [  # heads, kv, dim, vdim, window
    (4, 2, 16, 8, 37),      # row / group kernels
    (3, 3, 10, 6, 5),       # nothing a multiple of 8
    (2, 1, 64, 64, 100),    # tensor-core tiles for prompt portions
    (8, 1, 32, 64, 70),     # values twice as wide as the keys; eight heads on one key head
    (4, 4, 128, 128, 300),  # a window that reaches the split of long contexts
    (2, 2, 64, 64, 0),      # no window
    (1, 1, 4, 2, 1),        # a position that only sees itself
    (6, 2, 16, 8, 400),     # three heads per key head: the row kernel, its long contexts split over CTAs
]


@pytest.mark.parametrize("kind", ["f32", "bf16"])
@pytest.mark.parametrize("shape", ATT_SHAPES)
def test_windowed_sigmoid_attention(S, shape, kind):
    """two sequences in one batch: a prompt portion of 150 tokens behind 330 cached ones, and a single token at position 77.
    For every query the keys just inside and just outside its window are made to stand out (large scores, values of their
    own), as is a key far back: the first must count in full, the others not at all."""
    H, G, d, dv, win = shape
    code, g, PR = code_of(S, kind), gen(sum(shape)), 64
    n0, new0, n1 = 480, 150, 78
    scale = 1.0 / math.sqrt(d)
    k = {0: rounded(torch.randn(n0, G, d, generator=g), kind), 1: rounded(torch.randn(n1, G, d, generator=g), kind)}
    v = {0: rounded(torch.randn(n0, G, dv, generator=g), kind), 1: rounded(torch.randn(n1, G, dv, generator=g), kind)}
    pos = list(range(n0 - new0, n0)) + [n1 - 1]
    slot = [0] * new0 + [1]
    q = rounded(torch.randn(len(pos), H, d, generator=g), kind)
    hb = torch.randn(H, generator=g) - 2.0
    if win:
        # query 100 of the portion (position 430): its own direction in q; the keys at the window's two edges and one far
        # back point the same way, with values +40 / -40 / -40 on one column each
        u = torch.zeros(d, dtype=torch.float64); u[0] = 1.0
        p = pos[100]
        q[100] = rounded(u * 12.0 / scale / 4.0, kind)
        for j, val, col in ((p - win + 1, 40.0, 0), (p - win, -40.0, 1 % dv), (max(p - win - 130, 0), -40.0, 1 % dv)):
            if j >= 0:
                k[0][j] = rounded(u * 4.0, kind)
                v[0][j] = 0.0
                v[0][j, :, col] = val
    kp, vp, table, max_pages = paged(S, code, k, v, PR, 5)
    want = torch.cat([plain_sigmoid_attention(q[:new0], k[0], v[0], pos[:new0], win, scale, hb),
                      plain_sigmoid_attention(q[new0:], k[1], v[1], pos[new0:], win, scale, hb)])
    if win and pos[100] - win + 1 >= 0:
        assert want[100, 0, 0] > 35.0     # the inside edge counts in full (sigmoid(12 + bias) ~ 1); the outside ones would subtract 40

    def run(qq, sl, ps, longest):
        T = len(sl)
        out = torch.empty(T, H * dv, dtype=torch.float32, device="cuda")
        need = S.lib().b200_paged_attention_workspace_bytes(T, H, dv)
        ws = torch.empty(max(need, 16), dtype=torch.uint8, device="cuda")
        _alive.extend([out, ws])
        a = S.PagedAttentionArgs(dev(qq.reshape(T, -1), tdt(S, code)).data_ptr(), out.data_ptr(), kp.data_ptr(), vp.data_ptr(), table.data_ptr(), max_pages,
                                 PR, ints(sl).data_ptr(), ints(ps).data_ptr(), T, H, G, d, dv, scale, 0.0, 0.0, code, longest, max(ps) + 1,
                                 ws.data_ptr(), need, 0, 1, 1, win, 1, dev(hb).data_ptr())
        sync_ok(S.lib().b200_paged_attention(C.byref(a), None))
        return out.reshape(T, H, dv)

    tol = 2e-2 if kind == "bf16" else 2e-5
    assert rel(run(q, slot, pos, new0), want) < tol                       # the mixed batch
    # single tokens (the decode kernels, long contexts split over CTAs): the edge query, the newest one and the short sequence
    pick = [100, new0 - 1, new0]
    assert rel(run(q[pick], [slot[i] for i in pick], [pos[i] for i in pick], 1), want[pick]) < tol


@pytest.mark.parametrize("kind", ["f32", "bf16"])
def test_biases_head_norms_and_rotated_values_reach_the_pages(S, kind):
    code, g, PR = code_of(S, kind), gen(9), 64
    H, G, d, dv, rd, T0 = 4, 2, 12, 10, 8, 70
    nq, nk, nv = H * d, G * d, G * dv
    ld = nq + nk + nv + H
    pos, slot = list(range(60, 60 + T0)), [1] * T0
    proj, bias = torch.randn(T0, ld, generator=g), torch.randn(ld, generator=g)
    qn, kn = 1 + torch.randn(d, generator=g) * 0.2, 1 + torch.randn(d, generator=g) * 0.2
    base = 100.0
    c, s = tables(S, pos, [base ** (-2.0 * i / rd) for i in range(rd // 2)])
    vc, vs = tables(S, pos, [base ** (-2.0 * m / dv) for m in range(dv // 2)])
    table = torch.tensor([[0, 0, 0], [4, 1, 2]], dtype=torch.int32)
    q_out = torch.zeros(T0, nq, dtype=tdt(S, code), device="cuda")
    kp = torch.zeros(5 * PR, G, d, dtype=tdt(S, code), device="cuda")
    vp = torch.zeros(5 * PR, G, dv, dtype=tdt(S, code), device="cuda")
    a = S.QkPrepareArgs()
    a.proj, a.ld_proj, a.q_norm, a.k_norm, a.eps = dev(proj).data_ptr(), ld, dev(qn).data_ptr(), dev(kn).data_ptr(), 1e-5
    a.cos, a.sin, a.rot_dims, a.rot_layout = c.data_ptr(), s.data_ptr(), rd, S.ROPE_HALF
    a.q_out, a.k_pool, a.v_pool = q_out.data_ptr(), kp.data_ptr(), vp.data_ptr()
    a.pages, a.max_pages, a.page_rows = dev(table).data_ptr(), 3, PR
    a.slot, a.pos, a.start = ints(slot).data_ptr(), ints(pos).data_ptr(), ints([60] * T0).data_ptr()
    a.n_tokens, a.heads, a.kv_heads, a.dim, a.dtype = T0, H, G, d, code
    a.v_heads, a.vdim, a.v_off = G, dv, nq + nk
    a.bias, a.v_cos, a.v_sin, a.v_rot_layout = dev(bias).data_ptr(), vc.data_ptr(), vs.data_ptr(), S.ROPE_HALF
    sync_ok(S.lib().b200_qk_prepare(C.byref(a), None))
    pb = (proj + bias).double()
    ang = torch.tensor(pos, dtype=torch.float64)[:, None] * torch.tensor([base ** (-2.0 * i / rd) for i in range(rd // 2)], dtype=torch.float64)
    vang = torch.tensor(pos, dtype=torch.float64)[:, None] * torch.tensor([base ** (-2.0 * m / dv) for m in range(dv // 2)], dtype=torch.float64)
    wq = O.turn(O.rms_norm(pb[:, :nq].view(T0, H, d), qn.double(), 1e-5), ang, "half")
    wk = O.turn(O.rms_norm(pb[:, nq:nq + nk].view(T0, G, d), kn.double(), 1e-5), ang, "half")
    wv = O.turn(pb[:, nq + nk:nq + nk + nv].view(T0, G, dv), vang, "half")
    rows = [int(table[1, p // PR]) * PR + p % PR for p in pos]
    tol = 1e-2 if kind == "bf16" else 1e-5
    assert rel(q_out.float().view(T0, H, d), wq) < tol
    assert rel(kp[rows].float(), wk) < tol
    assert rel(vp[rows].float(), wv) < tol


@pytest.mark.parametrize("layout", ["half", "interleaved"])
@pytest.mark.parametrize("vdim", [2, 10, 48, 7])
def test_outputs_turn_back_and_take_their_head_gate(S, vdim, layout):
    """rotating a value by its position and turning the weighted sum back by the query's leaves a relative rotation: a sum
    with a single weight on the query's own position comes back as the value itself"""
    g, T0, H = gen(vdim), 9, 3
    pos = [0, 1, 5, 64, 1000, 77, 3, 2, 99999]
    fr = [50.0 ** (-2.0 * m / vdim) for m in range(vdim // 2)]
    c, s = tables(S, pos, fr)
    v = torch.randn(T0, H, vdim, generator=g).double()
    ang = torch.tensor(pos, dtype=torch.float64)[:, None] * torch.tensor(fr, dtype=torch.float64)[None]
    turned = O.turn(v, ang, layout)
    gate = torch.randn(T0, H + 2, generator=g)
    code = S.ROPE_HALF if layout == "half" else S.ROPE_INTERLEAVED
    for kind in ("f32", "bf16"):
        out = torch.zeros(T0, H, vdim, dtype=tdt(S, code_of(S, kind)), device="cuda")
        sync_ok(S.lib().b200_unrotate_gate(dev(turned, torch.float32).data_ptr(), c.data_ptr(), s.data_ptr(), code, dev(gate).data_ptr() + 4, H + 2,
                                           out.data_ptr(), T0, H, vdim, code_of(S, kind), None))
        want = v * torch.sigmoid(gate[:, 1:H + 1].double())[:, :, None]
        assert rel(out.float(), want) < (1e-2 if kind == "bf16" else 2e-5)
    out = torch.zeros(T0, H, vdim, device="cuda")
    sync_ok(S.lib().b200_unrotate_gate(dev(turned, torch.float32).data_ptr(), c.data_ptr(), s.data_ptr(), code, None, 0, out.data_ptr(), T0, H, vdim, S.F32, None))
    assert rel(out, v) < 2e-5


LAT_SHAPES = [  # heads, rank, extra, window
    (4, 20, 4, 29),
    (5, 11, 6, 3),
    (8, 64, 32, 200),     # a window long enough for contexts to be split over CTAs
    (16, 128, 64, 0),     # no window
    (1, 3, 2, 1),
    (40, 24, 8, 70),      # more heads than a tile has rows
    (4, 512, 64, 150),    # the widest rows the kernels take
]


@pytest.mark.parametrize("kind", ["f32", "bf16"])
@pytest.mark.parametrize("shape", LAT_SHAPES)
def test_windowed_latent_attention_without_a_sink(S, shape, kind):
    """rows [latent | rotated part] of two sequences; a prompt portion behind cached rows and a single token. The rows at the
    two edges of one query's window stand out by their scores."""
    H, R, X, win = shape
    code, g, PR, W = code_of(S, kind), gen(sum(shape)), 64, R + X
    n0, new0, n1 = 400, 90, 41
    rows = {0: rounded(torch.randn(n0, 1, W, generator=g), kind), 1: rounded(torch.randn(n1, 1, W, generator=g), kind)}
    pos = list(range(n0 - new0, n0)) + [n1 - 1]
    slot = [0] * new0 + [1]
    qa = torch.randn(len(pos), H, W, generator=g).double()
    scale = 1.0 / math.sqrt(W)
    if win > 1:
        p = pos[50]
        u = torch.zeros(W, dtype=torch.float64); u[1] = 1.0
        qa[50] = u * 9.0 / scale / 3.0
        rows[0][p - win + 1, 0] = rounded(u * 3.0, kind)        # just inside: takes nearly all the weight
        rows[0][p - win, 0] = rounded(u * 6.0, kind)            # just outside: would take it all
    pool, _, table, max_pages = paged(S, code, rows, rows, PR, 8)

    def plain(qq, c, ps):
        out = torch.zeros(len(ps), H, W, dtype=torch.float64)
        for i, p in enumerate(ps):
            lo = max(0, p - win + 1) if win else 0
            sc = torch.einsum("hw,jw->hj", rounded(qq[i], kind), c[lo: p + 1, 0]) * scale
            out[i] = torch.softmax(sc, -1) @ c[lo: p + 1, 0]
        return out

    want = torch.cat([plain(qa[:new0], rows[0], pos[:new0]), plain(qa[new0:], rows[1], pos[new0:])])
    if win > 1:
        assert want[50, 0, 1] > 2.5 and want[50, 0, 1] < 3.5

    def run(qq, sl, ps, longest, out_cols=0):
        T = len(sl)
        out = torch.zeros(T, H, W, device="cuda")
        need = S.lib().b200_latent_attention_workspace_bytes(T, H, W)
        ws = torch.empty(max(need, 16), dtype=torch.uint8, device="cuda")
        _alive.extend([out, ws])
        a = S.LatentAttentionArgs(dev(qq, torch.float32).data_ptr(), out.data_ptr(), pool.data_ptr(), table.data_ptr(), max_pages, PR,
                                  ints(sl).data_ptr(), ints(ps).data_ptr(), None, scale, T, H, W, win, code, longest, max(ps) + 1, ws.data_ptr(), need,
                                  out_cols)
        sync_ok(S.lib().b200_latent_attention_ex(C.byref(a), None))
        return out

    tol = 3e-2 if kind == "bf16" else 2e-5
    assert rel(run(qa, slot, pos, new0), want) < tol
    pick = [50, new0 - 1, new0]
    assert rel(run(qa[pick], [slot[i] for i in pick], [pos[i] for i in pick], 1), want[pick]) < tol
    # a caller that only uses the latent columns of the weighted sum
    assert rel(run(qa, slot, pos, new0, R)[:, :, :R], want[:, :, :R]) < tol
    assert rel(run(qa[pick], [slot[i] for i in pick], [pos[i] for i in pick], 1, R)[:, :, :R], want[pick][:, :, :R]) < tol


@pytest.mark.parametrize("kind", ["f32", "bf16"])
def test_latent_rows_with_a_rotated_part_and_the_query_part_beside_the_absorbed_one(S, kind):
    code, g, PR = code_of(S, kind), gen(12), 64
    R, X, T0, H, dq = 11, 6, 20, 3, 5
    rot = dict(dims=X, base=50.0, scaling=dict(factor=4.0, original=32, fast=8.0, slow=1.0))
    pos, slot = list(range(100, 100 + T0)), [0] * T0
    ang, amp = O.ramped_angles(200, rot)
    ang = ang[100:100 + T0]
    freqs = (ang[1] - ang[0]).tolist()
    c, s = tables(S, pos, freqs, amp)
    raw, w = torch.randn(T0, 3 + R + X, generator=g), 1 + torch.randn(R, generator=g) * 0.2
    pool = torch.zeros(3 * PR, R + X, dtype=tdt(S, code), device="cuda")
    table = ints([[2, 0, 1]])
    sync_ok(S.lib().b200_latent_store_rot(dev(raw).data_ptr() + 12, 3 + R + X, dev(w).data_ptr(), 1e-5, pool.data_ptr(), table.data_ptr(), 3, PR,
                                          ints(slot).data_ptr(), ints(pos).data_ptr(), T0, R, X, c.data_ptr(), s.data_ptr(), S.ROPE_INTERLEAVED, code, None))
    rows = [[2, 0, 1][p // PR] * PR + p % PR for p in pos]
    want = torch.cat([O.rms_norm(raw[:, 3:3 + R].double(), w.double(), 1e-5),
                      O.turn(raw[:, 3 + R:].double().view(T0, 1, X), ang, "interleaved", amp).view(T0, X)], 1)
    assert rel(pool[rows].float(), want) < (1e-2 if kind == "bf16" else 1e-5)
    # the heads' rotated query parts behind their absorbed parts
    qp = torch.randn(T0, H * (dq + X) + 2, generator=g)
    qa = torch.zeros(T0, H, R + X, device="cuda")
    sync_ok(S.lib().b200_rotate_part(dev(qp).data_ptr(), H * (dq + X) + 2, dq, dq + X, qa.data_ptr(), H * (R + X), R, R + X, c.data_ptr(), s.data_ptr(),
                                     S.ROPE_INTERLEAVED, T0, H, X, None))
    src = qp[:, :H * (dq + X)].double().view(T0, H, dq + X)[:, :, dq:]
    assert rel(qa[:, :, R:], O.turn(src.contiguous(), ang, "interleaved", amp)) < 1e-5
    assert float(qa[:, :, :R].abs().max()) == 0.0


def plain_recurrence(pre, zb, ub, C_, S0):
    z = torch.sigmoid(pre[:, :C_] + zb)
    u = pre[:, C_:2 * C_] + ub
    cand = torch.where(u >= 0, u + 0.5, torch.sigmoid(u))
    S_, out = S0.clone(), []
    for t in range(pre.shape[0]):
        S_ = (1 - z[t]) * S_ + z[t] * cand[t]
        out.append(S_ * O.silu(pre[t, 2 * C_:3 * C_]))
    return torch.stack(out), S_


@pytest.mark.parametrize("kind", ["f32", "bf16"])
@pytest.mark.parametrize("channels", [1, 40, 300])
def test_gated_recurrence_with_its_carried_state(S, channels, kind):
    """three entries in one batch: 200 tokens from position 0 into a slot that holds someone else's state, one token behind a
    carried state, and 70 tokens behind one; then the long entry goes on for two tokens, and then in one chunked piece"""
    code, g, Cn = code_of(S, kind), gen(channels), channels
    lens, starts, slots = [200, 1, 70], [0, 9, 130], [2, 0, 1]
    T0 = sum(lens)
    pre = torch.randn(T0 + 2 + 150, 3 * Cn + 1, generator=g) * 1.5
    zb, ub = torch.randn(Cn, generator=g), torch.randn(Cn, generator=g) * 0.5
    state = torch.randn(3, Cn, generator=g)
    dstate, dpre = dev(state), dev(pre)
    tol = 1e-2 if kind == "bf16" else 2e-5

    def run(row0, lens_, starts_, slots_):
        T = sum(lens_)
        out = torch.zeros(T, Cn, dtype=tdt(S, code), device="cuda")
        need = S.lib().b200_gated_recurrence_workspace_bytes(T, len(lens_), Cn)
        ws = torch.empty(max(need, 16), dtype=torch.uint8, device="cuda")
        _alive.extend([out, ws])
        ent_row = np.cumsum([0] + lens_[:-1]).tolist()
        a = S.GatedRecurrenceArgs()
        a.pre, a.ld_pre, a.z_off, a.u_off, a.g_off = dpre.data_ptr() + 4 * (row0 * (3 * Cn + 1) + 1), 3 * Cn + 1, 0, Cn, 2 * Cn
        a.z_bias, a.u_bias, a.state, a.out, a.out_dtype = dev(zb).data_ptr(), dev(ub).data_ptr(), dstate.data_ptr(), out.data_ptr(), code
        a.ent_row, a.ent_len = ints(ent_row).data_ptr(), ints(lens_).data_ptr()
        a.slot = ints([s for s, n in zip(slots_, lens_) for _ in range(n)]).data_ptr()
        a.pos = ints([st + i for st, n in zip(starts_, lens_) for i in range(n)]).data_ptr()
        a.n_entries, a.n_tokens, a.channels, a.longest_entry = len(lens_), T, Cn, max(lens_)
        a.workspace, a.workspace_bytes = ws.data_ptr(), need
        sync_ok(S.lib().b200_gated_recurrence(C.byref(a), None))
        return out.float().cpu()

    got = run(0, lens, starts, slots)
    p64 = pre[:, 1:].double()
    want, ends, at = [], {}, 0
    for n, st, sl in zip(lens, starts, slots):
        o, e = plain_recurrence(p64[at: at + n], zb.double(), ub.double(), Cn, state[sl].double() if st > 0 else torch.zeros(Cn, dtype=torch.float64))
        want.append(o); ends[sl] = e; at += n
    assert rel(got, torch.cat(want)) < tol
    for sl in range(3):
        assert rel(dstate[sl], ends[sl]) < 2e-5
    # two single tokens of the long sequence (the direct form), then 150 more in one entry (chunks from a carried state)
    got2 = torch.cat([run(T0, [1], [200], [2]), run(T0 + 1, [1], [201], [2])])
    o2, e2 = plain_recurrence(p64[T0: T0 + 2], zb.double(), ub.double(), Cn, ends[2])
    assert rel(got2, o2) < tol
    got3 = run(T0 + 2, [150], [202], [2])
    o3, e3 = plain_recurrence(p64[T0 + 2:], zb.double(), ub.double(), Cn, e2)
    assert rel(got3, o3) < tol and rel(dstate[2], e3) < 2e-5


@pytest.mark.parametrize("kind", ["f32", "bf16"])
@pytest.mark.parametrize("rows", [3, 300])
def test_clamped_gated_unit_as_kernel_and_as_epilogue(S, rows, kind):
    code, g, K, N, lim = code_of(S, kind), gen(rows), 64, 128, 1.5
    x, W = rounded(torch.randn(rows, K, generator=g), kind), rounded(torch.randn(2 * N, K, generator=g) * 0.4, kind)
    gu = x @ W.T
    want = O.clamped_glu(x, dict(limit=lim), dict(gate=W[:N], up=W[N:], down=torch.eye(N, dtype=torch.float64)), "")
    assert float((gu[:, :N] > lim).double().mean()) > 0.05 and float((gu[:, N:].abs() > lim).double().mean()) > 0.1   # the clamps bite
    out = torch.zeros(rows, N, dtype=tdt(S, code), device="cuda")
    sync_ok(S.lib().b200_glu_act_clamped(dev(gu, torch.float32).data_ptr(), out.data_ptr(), rows, N, lim, code, None))
    assert rel(out.float(), want) < (1e-2 if kind == "bf16" else 1e-5)
    out2 = torch.zeros(rows, N, dtype=tdt(S, code), device="cuda")
    sync_ok(S.lib().b200_linear_ex2(dev(x, tdt(S, code)).data_ptr(), dev(W, tdt(S, code)).data_ptr(), out2.data_ptr(), rows, N, K, code, code,
                                    S.GG_GLU_CLAMP, lim, None, 0, None))
    assert rel(out2.float(), want) < (1e-2 if kind == "bf16" else 1e-5)
    assert S.lib().b200_linear_ex(dev(x, tdt(S, code)).data_ptr(), dev(W, tdt(S, code)).data_ptr(), out2.data_ptr(), rows, N, K, code, code,
                                  S.GG_GLU_CLAMP, None, 0, None) != 0          # the unit needs its limit
    v = torch.randn(1000, generator=g)
    dv_ = dev(v)
    sync_ok(S.lib().b200_scale(dv_.data_ptr(), 1000, 0.3, None))
    assert rel(dv_, v.double() * 0.3) < 1e-6

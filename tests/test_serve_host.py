"""Host side of the model-family layer on a machine without a GPU: the registry, config.json / safetensors parsing
and the error paths that end before any CUDA call."""
import json
import math
import os

import pytest
import torch

import nekodra_oracle as O


@pytest.fixture(scope="module")
def S(pkg):
    if not os.path.exists(pkg.lib_path()):
        pytest.fail(f"{pkg.lib_path()} not built: run __graft_entry__.build()")
    return pkg.serve


def test_registry_lists_the_families(S):
    fams = S.lib().b200_model_families().decode().split(",")
    assert "Nekodra" in fams and "Musilorn" in fams and "Tomalix" in fams and "Sakevik" in fams and "llama" in fams


def test_unknown_architecture_and_broken_config(S, tmp_path):
    with pytest.raises(RuntimeError, match="cannot read"):
        S.Model(tmp_path / "nowhere")
    (tmp_path / "config.json").write_text('{"architecture": "Other", "width": 8}')
    with pytest.raises(RuntimeError, match="no family registered"):
        S.Model(tmp_path)
    (tmp_path / "config.json").write_text('{"architecture": "Nekodra", "width": 8,')
    with pytest.raises(RuntimeError, match="json"):
        S.Model(tmp_path)
    (tmp_path / "config.json").write_text('{"architecture": "Nekodra", "width": 8}')
    with pytest.raises(RuntimeError, match="required"):
        S.Model(tmp_path)


def test_musilorn_configuration_errors_end_before_any_cuda_call(S, tmp_path):
    (tmp_path / "config.json").write_text('{"architecture": "Musilorn", "width": 8, "vocab": 5, "norm": {"eps": 1e-5}, "layers": []}')
    with pytest.raises(RuntimeError, match="required"):
        S.Model(tmp_path)
    (tmp_path / "config.json").write_text('{"architecture": "Musilorn", "width": 8, "vocab": 5, "norm": {"eps": 1e-5}, '
                                          '"layers": [{"type": "attention", "mixer": {}, "mlp": null}]}')
    with pytest.raises(RuntimeError, match="residual_mult"):
        S.Model(tmp_path)


def test_tomalix_configuration_errors_end_before_any_cuda_call(S, tmp_path):
    head = '{"architecture": "Tomalix", "width": 8, "vocab": 5, "norm": {"eps": 1e-5}, '
    (tmp_path / "config.json").write_text(head + '"layers": []}')
    with pytest.raises(RuntimeError, match="required"):
        S.Model(tmp_path)
    (tmp_path / "config.json").write_text(head + '"layers": [{"type": "retention", "mixer": {}, "mlp": null}]}')
    with pytest.raises(RuntimeError, match="not part of this family"):
        S.Model(tmp_path)
    (tmp_path / "config.json").write_text(head + '"layers": [{"type": "attention_2", "mixer": {}, "mlp": {"kind": "glu"}}]}')
    with pytest.raises(RuntimeError, match="feed-forward kind"):
        S.Model(tmp_path)
    (tmp_path / "config.json").write_text(head + '"loop": {"start": 0, "stop": 2, "times": 2}, '
                                          '"layers": [{"type": "attention_2", "mixer": {}, "mlp": null}]}')
    with pytest.raises(RuntimeError, match="loop"):
        S.Model(tmp_path)


def test_tomalix_oracle_pieces_agree_with_closed_forms():
    """the plain implementation of the third family: the offset norm, the three frequency rules, the rotation, the block
    mask, the two-map combination, the convolution, the scan against its unrolled sum, the router, the order of layer runs"""
    import tomalix_oracle as T
    g = torch.Generator().manual_seed(2)
    D = torch.float64
    x = torch.randn(4, 6, generator=g, dtype=D)
    assert torch.allclose(T.rms_norm(x, torch.zeros(6, dtype=D), 0.0), x / x.pow(2).mean(-1, keepdim=True).sqrt())
    assert torch.allclose(T.rms_norm(x, torch.full((6,), 0.5, dtype=D), 0.0), 1.5 * T.unit_rms(x, 0.0))
    rot = dict(base=100.0, dims=8)
    plain, amp0 = T.rot_frequencies(rot, "plain")
    lin, amp1 = T.rot_frequencies(dict(rot, scaling=dict(factor=4.0)), "linear")
    assert amp0 == 1.0 and amp1 == 1.0 and torch.allclose(lin, plain / 4) and float(plain[1]) == pytest.approx(100.0 ** (-2 / 8))
    # the ramp: index where `fast` turns fit into `original` positions -> kept; beyond the index of `slow` -> divided by factor
    sc = dict(factor=2.0, original=64, fast=4.0, slow=0.5)
    ramp, amp = T.rot_frequencies(dict(rot, scaling=sc), "ramp")
    idx = lambda turns: 8 * math.log(64 / (2 * math.pi * turns)) / (2 * math.log(100.0))
    lo, hi = max(math.floor(idx(4.0)), 0), min(math.ceil(idx(0.5)), 7)
    assert (lo, hi) == (0, 3) and amp == pytest.approx(0.1 * math.log(2.0) + 1)
    assert ramp[0] == plain[0] and torch.allclose(ramp[3], plain[3] / 2) and torch.allclose(ramp[1], plain[1] * (1 - 1 / 3) + plain[1] / 2 / 3)
    q = torch.randn(5, 2, 8, generator=g, dtype=D)
    r = T.rotate_half(q, dict(base=100.0, dims=4), "plain")
    a = 3 * 100.0 ** (-2 / 4)
    assert torch.equal(r[..., 4:], q[..., 4:]) and torch.equal(r[0], q[0])
    assert torch.allclose(r[3, 1, 1], q[3, 1, 1] * math.cos(a) - q[3, 1, 3] * math.sin(a))
    assert torch.allclose(r[3, 1, 3], q[3, 1, 3] * math.cos(a) + q[3, 1, 1] * math.sin(a))
    m = T.visible(7, 3)
    assert m[5].tolist() == [False, False, False, True, True, True, False] and m[6].tolist() == [False] * 6 + [True]
    assert T.visible(3).tolist() == [[True, False, False], [True, True, False], [True, True, True]]
    u, w, b = torch.randn(6, 3, generator=g, dtype=D), torch.randn(3, 4, generator=g, dtype=D), torch.randn(3, generator=g, dtype=D)
    y = T.causal_conv(u, w, b)
    assert torch.allclose(y[0], b + w[:, 3] * u[0]) and torch.allclose(y[5], b + (w.T * u[2:6]).sum(0))
    # the scan of one channel and one state is a weighted sum over the past
    W = {"in": torch.tensor([[1.0], [0.5]], dtype=D), "conv": torch.ones(1, 1, dtype=D),
         "conv.b": torch.zeros(1, dtype=D), "x": torch.tensor([[0.3], [1.0], [2.0]], dtype=D), "dt": torch.ones(1, 1, dtype=D),
         "dt.b": torch.zeros(1, dtype=D), "A_log": torch.zeros(1, 1, dtype=D), "D": torch.tensor([0.25], dtype=D), "o": torch.ones(1, 1, dtype=D)}
    h = torch.randn(4, 1, generator=g, dtype=D)
    got = T.selective_scan(h, dict(inner=1, state=1, dt_rank=1, conv=1), W, "")
    xs, z = T.silu(h[:, 0]), 0.5 * h[:, 0]
    dt = torch.log1p(torch.exp(0.3 * xs))
    want = []
    for t in range(4):
        acc = sum(math.exp(-float(dt[j + 1: t + 1].sum())) * float(dt[j] * xs[j]) * float(xs[j]) for j in range(t + 1))
        want.append((acc * 2.0 * float(xs[t]) + 0.25 * float(xs[t])) * float(T.silu(z[t])))
    assert torch.allclose(got[:, 0], torch.tensor(want, dtype=D))
    # router: the two largest biased logits, weights over those two alone
    Wr = {"router": torch.eye(3, dtype=D), "router.b": torch.tensor([0.0, 0.0, -2.0], dtype=D)}
    for e in range(3):
        Wr["e%d.up" % e], Wr["e%d.down" % e] = torch.full((1, 3), float(e + 1), dtype=D), torch.ones(3, 1, dtype=D)
    hh = torch.tensor([[2.0, 1.0, -1.0]], dtype=D)                     # logits 2, 1, -3: experts 0 and 1
    out = T.routed_ff(hh, dict(router=dict(experts=3, top=2)), Wr, "")
    p = torch.softmax(torch.tensor([2.0, 1.0], dtype=D), 0)
    assert torch.allclose(out[0], (p[0] * 2.0 ** 2 + p[1] * 4.0 ** 2).expand(3))
    cfg = dict(layers=[0, 1, 2, 3], loop=dict(start=1, stop=3, times=2))
    assert T.layer_order(cfg) == [(0, None), (1, 0), (2, None), (1, 1), (2, None), (3, None)]
    assert T.layer_order(dict(layers=[0, 1])) == [(0, None), (1, None)]


def test_musilorn_oracle_pieces_agree_with_closed_forms():
    """the plain implementation of the second family: rotation pairings, the convolution, the retention walk against its
    unrolled sum, the softmax with one in the denominator, the order in which a repeated span runs"""
    import musilorn_oracle as M
    g = torch.Generator().manual_seed(1)
    x = torch.randn(5, 2, 8, generator=g, dtype=torch.float64)
    rot = dict(base=100.0, dims=4)
    half, inter = M.rotate(x, rot, "half"), M.rotate(x, rot, "interleaved")
    assert torch.equal(half[..., 4:], x[..., 4:]) and torch.equal(inter[0], x[0])          # beyond dims, and position 0
    a = 3 * 100.0 ** (-2 / 4)                                                                # position 3, second frequency
    assert torch.allclose(half[3, 0, 1], x[3, 0, 1] * math.cos(a) - x[3, 0, 3] * math.sin(a))
    assert torch.allclose(inter[3, 0, 3], x[3, 0, 3] * math.cos(a) + x[3, 0, 2] * math.sin(a))
    assert torch.allclose((half ** 2).sum(-1), (x ** 2).sum(-1))                            # a rotation keeps lengths
    f = M.rot_frequencies(dict(base=10000.0, dims=8, scaling=dict(factor=4.0, low=1.0, high=4.0, original=128)))
    plain = M.rot_frequencies(dict(base=10000.0, dims=8))
    assert f[0] == plain[0] and torch.allclose(f[3], plain[3] / 4) and plain[1] / 4 < f[1] < plain[1]
    u, w = torch.randn(6, 3, generator=g, dtype=torch.float64), torch.randn(3, 4, generator=g, dtype=torch.float64)
    y = M.short_conv(u, w)
    assert torch.allclose(y[0], w[:, 3] * u[0]) and torch.allclose(y[5], (w.T * u[2:6]).sum(0))
    q, k, v = (torch.randn(7, n, generator=g, dtype=torch.float64) for n in (4, 4, 5))
    o = M.retention_state_walk(q, k, v, 0.8)
    assert torch.allclose(o[6], sum(0.8 ** (6 - j) * (q[6] @ k[j]) * v[j] for j in range(7)))
    att = M.capped_sink_attention(q, k, v, 0.7, 2.0)
    s = 2.0 * torch.tanh(k[:3] @ q[2] * 0.7 / 2.0)
    assert torch.allclose(att[2], (torch.exp(s) / (1 + torch.exp(s).sum())) @ v[:3])
    cfg = dict(layers=[0, 1, 2, 3], loop=dict(start=1, stop=3, times=2))
    assert M.layer_runs(cfg) == [(0, False), (1, True), (2, False), (1, True), (2, False), (3, False)]


def test_oracle_pieces_agree_with_torch():
    """the plain implementation itself: its norms and its sink softmax against closed forms"""
    g = torch.Generator().manual_seed(0)
    x, w, b = torch.randn(5, 12, generator=g), torch.randn(12, generator=g), torch.randn(12, generator=g)
    assert torch.allclose(O.layer_norm(x, w, b, 1e-5), torch.nn.functional.layer_norm(x, (12,), w, b, 1e-5), atol=1e-6)
    q, k, v = torch.randn(3, 4, generator=g), torch.randn(6, 4, generator=g), torch.randn(6, 5, generator=g)
    sink = torch.tensor(0.3)
    got = O.sink_attention(q, k, v, 0.5, sink)
    for i in range(3):
        n = 4 + i                                                   # the last three positions of six
        s = torch.cat([(q[i] @ k[:n].T) * 0.5, sink[None]])
        p = torch.softmax(s, 0)[:-1]                                # the sink takes its share and gives nothing back
        assert torch.allclose(got[i], p @ v[:n], atol=1e-6)
    # a very negative sink is plain softmax attention
    plain = O.sink_attention(q, k, v, 0.5, torch.tensor(-1e9))
    assert torch.allclose(plain[2], torch.softmax((q[2] @ k.T) * 0.5, 0) @ v, atol=1e-6)


def test_written_checkpoint_has_the_documented_layout(tmp_path):
    cfg, w = O.random_model(seed=1)
    O.write_model(str(tmp_path), cfg, w)
    raw = (tmp_path / "model.safetensors").read_bytes()
    n = int.from_bytes(raw[:8], "little")
    header = json.loads(raw[8:8 + n])
    assert header["l0.mix.q"]["shape"] == [48, 64] and header["l0.mix.q"]["dtype"] == "BF16"
    assert "l1.mix.dkv" not in header and "l0.mix.dkv" in header    # the second layer reads the first one's rows
    assert json.loads((tmp_path / "config.json").read_text())["layers"][1]["mixer"]["kv_from"] == 0


def test_sakevik_configuration_errors_end_before_any_cuda_call(S, tmp_path):
    head = '{"architecture": "Sakevik", "width": 8, "vocab": 5, "norm": {"eps": 1e-5}, '
    (tmp_path / "config.json").write_text(head + '"layers": []}')
    with pytest.raises(RuntimeError, match="required"):
        S.Model(tmp_path)
    (tmp_path / "config.json").write_text(head + '"layers": [{"type": "retention", "mixer": {}, "mlp": null}]}')
    with pytest.raises(RuntimeError, match="not part of this family"):
        S.Model(tmp_path)
    (tmp_path / "config.json").write_text(head + '"layers": [{"type": "mingru", "mixer": {"width": 4}, "mlp": {"kind": "moe"}}]}')
    with pytest.raises(RuntimeError, match="feed-forward kind"):
        S.Model(tmp_path)
    (tmp_path / "config.json").write_text(head + '"layers": [{"type": "mingru", "mixer": {"width": 4}, "mlp": {"kind": "dense", "ff": 8}}]}')
    with pytest.raises(RuntimeError, match="limit"):
        S.Model(tmp_path)
    (tmp_path / "config.json").write_text(head + '"layers": [{"type": "attention", "mixer": {"heads": 3, "kv_heads": 2, "dim": 4, "vdim": 4, '
                                          '"scale": 0.5}, "mlp": null}]}')
    with pytest.raises(RuntimeError, match="multiple of kv_heads"):
        S.Model(tmp_path)
    (tmp_path / "config.json").write_text(head + '"layers": [{"type": "latent_attention", "mixer": {"heads": 2, "dim": 4, "vdim": 4, "kv_rank": 6, '
                                          '"rot_dim": 4, "rot": {"base": 100.0, "dims": 2}, "scale": 0.5}, "mlp": null}]}')
    with pytest.raises(RuntimeError, match="rot_dim"):
        S.Model(tmp_path)
    (tmp_path / "config.json").write_text(head + '"embedding": {"scale": 1.0, "bigram": {"buckets": 0, "mul_prev": 1, "mul_cur": 1}}, '
                                          '"layers": [{"type": "mingru", "mixer": {"width": 4}, "mlp": null}]}')
    with pytest.raises(RuntimeError, match="buckets"):
        S.Model(tmp_path)


def test_sakevik_oracle_pieces_agree_with_closed_forms():
    """the plain implementation of the fourth family: the norm, the pair rows, both rotation layouts and their inverse, the
    ramp, the window, the recurrence against its unrolled sum, sigmoid weights that do not sum to one, the clamped unit"""
    import sakevik_oracle as K
    g = torch.Generator().manual_seed(3)
    D = torch.float64
    x = torch.randn(4, 6, generator=g, dtype=D)
    assert torch.allclose(K.rms_norm(x, torch.full((6,), 2.0, dtype=D), 0.0), 2 * x / x.pow(2).mean(-1, keepdim=True).sqrt())
    cfg = dict(embedding=dict(scale=3.0, bigram=dict(buckets=5, mul_prev=7, mul_cur=3)))
    W = dict(embed=torch.randn(9, 2, generator=g, dtype=D), bigram=torch.randn(6, 2, generator=g, dtype=D))
    e = K.embed(cfg, W, [4, 8, 8])
    assert torch.allclose(e[0], 3 * W["embed"][4] + W["bigram"][5]) and torch.allclose(e[1], 3 * W["embed"][8] + W["bigram"][(4 * 7 + 8 * 3) % 5])
    assert torch.allclose(e[2], 3 * W["embed"][8] + W["bigram"][(8 * 7 + 8 * 3) % 5])
    q = torch.randn(5, 2, 6, generator=g, dtype=D)
    ang = K.pair_angles(5, 2, 100.0, 4)
    a = 3 * 100.0 ** (-2 / 4)
    r = K.turn(q, ang, "half")
    assert torch.equal(r[..., 4:], q[..., 4:]) and torch.equal(r[0], q[0])
    assert torch.allclose(r[3, 1, 1], q[3, 1, 1] * math.cos(a) - q[3, 1, 3] * math.sin(a))
    assert torch.allclose(r[3, 1, 3], q[3, 1, 3] * math.cos(a) + q[3, 1, 1] * math.sin(a))
    ri = K.turn(q, ang, "interleaved", 1.5)
    assert torch.allclose(ri[3, 0, 2], 1.5 * (q[3, 0, 2] * math.cos(a) - q[3, 0, 3] * math.sin(a)))
    assert torch.allclose(ri[3, 0, 3], 1.5 * (q[3, 0, 3] * math.cos(a) + q[3, 0, 2] * math.sin(a)))
    assert torch.allclose(K.turn(r, -ang, "half"), q)
    rot = dict(base=100.0, dims=8, scaling=dict(factor=2.0, original=64, fast=4.0, slow=0.5))
    angs, amp = K.ramped_angles(3, rot)
    f = angs[1]
    plain = torch.tensor([100.0 ** (-2 * i / 8) for i in range(4)], dtype=D)
    assert amp == pytest.approx(0.1 * math.log(2.0) + 1) and f[0] == plain[0] and torch.allclose(f[3], plain[3] / 2)
    assert torch.allclose(f[1], plain[1] * (1 - 1 / 3) + plain[1] / 2 / 3)
    m = K.window_mask(6, 3)
    assert m[5].tolist() == [False, False, False, True, True, True] and m[1].tolist() == [True, True, False, False, False, False]
    assert K.window_mask(3, 0).tolist() == [[True, False, False], [True, True, False], [True, True, True]]
    # one channel: the state is a weighted sum of the candidates, each weight the product of the later keep factors
    Wg = {"z": torch.tensor([[1.0]], dtype=D), "z.b": torch.tensor([0.3], dtype=D), "x": torch.tensor([[2.0]], dtype=D),
          "x.b": torch.tensor([-0.5], dtype=D), "g": torch.tensor([[1.5]], dtype=D), "o": torch.tensor([[1.0]], dtype=D)}
    h = torch.randn(5, 1, generator=g, dtype=D)
    got = K.mingru(h, Wg, "")
    z = torch.sigmoid(h[:, 0] + 0.3)
    u = 2 * h[:, 0] - 0.5
    cand = [float(v + 0.5) if v >= 0 else 1 / (1 + math.exp(-float(v))) for v in u]
    assert any(v >= 0 for v in u) and any(v < 0 for v in u)
    for t in range(5):
        st = sum(float(z[j]) * cand[j] * math.prod(1 - float(z[i]) for i in range(j + 1, t + 1)) for j in range(t + 1))
        assert float(got[t, 0]) == pytest.approx(st * float(K.silu(1.5 * h[t, 0])))
    # two tokens, one head, no rotation on q and k, unit values: the second output sums two sigmoids and need not be below one
    Wa = {"q": torch.zeros(2, 1, dtype=D), "q.b": torch.tensor([1.0, 0.0], dtype=D), "k": torch.zeros(2, 1, dtype=D), "k.b": torch.tensor([1.0, 0.0], dtype=D),
          "v": torch.zeros(2, 1, dtype=D), "v.b": torch.tensor([1.0, 0.0], dtype=D), "q.norm": torch.ones(2, dtype=D), "k.norm": torch.ones(2, dtype=D),
          "pb": torch.tensor([1.0], dtype=D), "g": torch.zeros(1, 1, dtype=D), "o": torch.eye(2, dtype=D), "o.b": torch.zeros(2, dtype=D)}
    mx = dict(heads=1, kv_heads=1, dim=2, vdim=2, scale=0.5, rot=dict(base=100.0, dims=0))
    out = K.sigmoid_attention(torch.zeros(2, 1, dtype=D), mx, Wa, "", 0.0)
    wgt = 1 / (1 + math.exp(-(2.0 * 0.5 + 1.0)))          # normed q and k are (sqrt 2, 0): their product is 2
    assert float(out[0, 0]) == pytest.approx(0.5 * wgt)
    # the value at position 0 is not turned, the one at position 1 by the angle 1; the sum is turned back by 1
    want1 = 0.5 * (wgt * math.cos(-1.0) + wgt)
    assert float(out[1, 0]) == pytest.approx(want1) and 2 * wgt > 1.0
    assert float(K.sigmoid_attention(torch.zeros(2, 1, dtype=D), dict(mx, mask=dict(size=1)), Wa, "", 0.0)[1, 0]) == pytest.approx(0.5 * wgt)
    Wf = {"gate": torch.tensor([[1.0]], dtype=D), "up": torch.tensor([[1.0]], dtype=D), "down": torch.tensor([[1.0]], dtype=D)}
    hv = torch.tensor([[-5.0], [0.5], [5.0]], dtype=D)
    y = K.clamped_glu(hv, dict(limit=2.0), Wf, "")
    assert float(y[2, 0]) == pytest.approx(2.0 / (1 + math.exp(-1.702 * 2.0)) * 3.0)
    assert float(y[1, 0]) == pytest.approx(0.5 / (1 + math.exp(-1.702 * 0.5)) * 1.5)
    assert float(y[0, 0]) == pytest.approx(-5.0 / (1 + math.exp(1.702 * 5.0)) * -1.0)

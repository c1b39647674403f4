"""The Sakevik family through the library's own entry points (registry -> step function -> paged cache and slot state
-> scheduler) against the plain implementation in sakevik_oracle.py, on small random models of several shapes: whole
prompts with every layer, prefill against token-by-token decoding, prompt portions down to two tokens, unequal batches
against each request alone, pages, slots, states and previous tokens that are freed and used again, window and page
borders in prompts and in decoding, the first tokens of a sequence, long decoding, sizes that are 1 or equal to each
other, and greedy generation through the continuous-batching scheduler."""
import copy

import numpy as np
import pytest
import torch

import sakevik_oracle as O

pytestmark = pytest.mark.gpu

RAMP = dict(factor=4.0, original=48, fast=8.0, slow=1.0)
SHAPES = {
    # every mixer, with and without a feed-forward; windows of 37 and 29 positions, so a page of 64 rows holds window edges
    # at places that are not its own
    "mix": dict(width=48, vocab=61, layers=[
        dict(type="mingru", width=40, ff=None),
        dict(type="attention", heads=4, kv_heads=2, dim=16, vdim=8, window=37, rot_dims=8, base=100.0, ff=(24, 1.5)),
        dict(type="latent_attention", heads=4, dim=8, rot_dim=4, vdim=8, kv_rank=20, window=29, scaling=RAMP, base=50.0, ff=(40, 3.0)),
        dict(type="mingru", width=24, ff=(16, 2.0)),
        dict(type="attention", heads=2, kv_heads=2, dim=8, vdim=12, window=64, ff=None)]),
    # sizes that are 1 or equal; a window of one position (a token only sees itself) and none at all; no rotation on q and k;
    # one key head for six query heads; no pair table; logits as they are; a model that starts with attention
    "odd": dict(width=40, vocab=33, buckets=None, logit_scale=1.0, embed_scale=1.0, layers=[
        dict(type="attention", heads=1, kv_heads=1, dim=4, vdim=2, window=1, rot_dims=0, ff=(8, 0.5)),
        dict(type="latent_attention", heads=1, dim=1, rot_dim=2, vdim=1, kv_rank=3, window=None, ff=None),
        dict(type="mingru", width=1, ff=None),
        dict(type="attention", heads=6, kv_heads=1, dim=6, vdim=10, window=None, rot_dims=4, ff=None),
        dict(type="latent_attention", heads=3, dim=10, rot_dim=6, vdim=6, kv_rank=9, window=1000, scale=0.5, ff=(8, 10.0))]),
    # nothing a multiple of 8
    "plain": dict(width=36, vocab=41, buckets=7, mul_prev=1, mul_cur=0, layers=[
        dict(type="latent_attention", heads=5, dim=6, rot_dim=6, vdim=9, kv_rank=11, window=33, ff=(20, 2.0)),
        dict(type="attention", heads=3, kv_heads=3, dim=10, vdim=6, window=5, rot_dims=10, ff=(12, 1.0)),
        dict(type="mingru", width=13, ff=(28, 2.5))]),
    # heads as wide as the tensor-core tiles take them, group sizes of the decode kernels, windows long enough for the split of
    # long contexts
    "wide": dict(width=64, vocab=50, layers=[
        dict(type="attention", heads=4, kv_heads=2, dim=64, vdim=64, window=100, ff=(128, 2.0)),
        dict(type="latent_attention", heads=8, dim=32, rot_dim=32, vdim=32, kv_rank=64, window=200, scaling=RAMP, ff=None),
        dict(type="mingru", width=128, ff=None),
        dict(type="attention", heads=8, kv_heads=1, dim=32, vdim=64, window=300, rot_dims=16, ff=(64, 4.0)),
        dict(type="attention", heads=2, kv_heads=2, dim=128, vdim=128, window=None, ff=None)]),
}
RTOL = {"f32": 3e-4, "bf16": 6e-2}


@pytest.fixture(scope="module")
def S(pkg):
    if not torch.cuda.is_available():
        pytest.fail("no CUDA device: the library has no CPU path")
    return pkg.serve


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    out = {}
    for i, (name, sh) in enumerate(SHAPES.items()):
        cfg, w = O.random_model(seed=70 + i, **sh)
        folder = tmp_path_factory.mktemp(name)
        O.write_model(str(folder), cfg, w)
        out[name] = (str(folder), O.Oracle(cfg, w), cfg)
    return out


def tokens(n, vocab, seed):
    return torch.randint(0, vocab, (n,), generator=torch.Generator().manual_seed(seed)).tolist()


def row_errors(got, want):
    """per row: rms of the difference with its mean taken off, over the rms of the wanted row"""
    got, want = np.asarray(got, np.float64), np.asarray(want, np.float64)
    d = got - want
    d = d - d.mean(-1, keepdims=True)
    return (np.sqrt((d ** 2).mean(-1)) / np.sqrt((want ** 2).mean(-1))).reshape(-1)


def err(got, want):
    return float(row_errors(got, want).max())


def check(got, want, kind, what=""):
    """fp32: every row within the tolerance. bfloat16: these small models answer a window that is one position off with a
    row error of 0.4 to 0.7 (test_every_mechanism_reaches_the_logits), and the norm on a sublayer's output turns the rounding
    of a small output into a change of its direction; so nine rows in ten have to be within the tolerance, the median well
    inside it, and no row anywhere near a wrong answer."""
    e = row_errors(got, want)
    assert np.all(np.isfinite(e)), what
    if kind == "f32":
        assert e.max() < RTOL[kind], (what, float(e.max()), int(e.argmax()))
    else:
        assert np.quantile(e, 0.9) < RTOL[kind] and np.median(e) < RTOL[kind] / 2 and e.max() < 0.2, \
            (what, float(np.quantile(e, 0.9)), float(np.median(e)), float(e.max()), int(e.argmax()))


def open_model(S, folder, kind, max_tokens=1024, slots=4):
    return S.Model(folder, dtype=S.BF16 if kind == "bf16" else S.F32, max_tokens=max_tokens, max_slots=slots)


@pytest.mark.parametrize("kind", ["f32", "bf16"])
@pytest.mark.parametrize("name", list(SHAPES))
def test_whole_prompt_and_every_layer(S, models, name, kind):
    folder, oracle, cfg = models[name]
    m = open_model(S, folder, kind)
    assert m.family == "Sakevik" and m.vocab == cfg["vocab"] and m.n_layers == len(cfg["layers"])
    toks = tokens(150, cfg["vocab"], 1)
    m.capture_layers(True)
    got = m.step([(0, toks, list(range(150)))])
    want, trail = oracle.forward(toks, return_layers=True)
    layers = m.captured_layers(150)
    for i in range(len(cfg["layers"])):
        check(layers[i], trail[i].numpy(), kind, f"residual after layer {i}")
    check(got, want.numpy(), kind)
    assert m.step_launches > 0
    m.close()


def test_every_mechanism_reaches_the_logits(models):
    """sensitivity of the comparison itself: with a window one position off, the value rotation, the head bias, the gates,
    the pair table, the previous token, the clamp, the candidate's branch or the amplitude changed, the oracle's logits move
    by far more than the tolerance the library is held to"""
    _, oracle, cfg = models["mix"]
    toks = tokens(90, cfg["vocab"], 2)
    base = oracle.forward(toks).numpy()

    def moved(change_cfg=None, change_w=None):
        c, w = copy.deepcopy(cfg), dict(oracle.w)
        if change_cfg:
            change_cfg(c)
        if change_w:
            change_w(w)
        return err(O.Oracle(c, w).forward(toks).numpy(), base)

    def window(c): c["layers"][1]["mixer"]["mask"]["size"] = 36
    def window_latent(c): c["layers"][2]["mixer"]["mask"]["size"] = 30
    def no_window(c): del c["layers"][4]["mixer"]["mask"]
    def value_base(c): c["layers"][1]["mixer"]["rot"]["base"] = 90.0
    def ramp(c): del c["layers"][2]["mixer"]["rot"]["scaling"]
    def ramp_edge(c): c["layers"][2]["mixer"]["rot"]["scaling"]["original"] = 10
    def limit(c): c["layers"][1]["mlp"]["limit"] = 1.4
    def mul(c): c["embedding"]["bigram"]["mul_prev"] = 8
    def scale(c): c["embedding"]["scale"] = 7.0
    def eps(c): c["norm"]["eps"] = 1e-2
    def head_bias(w): w["l1.mix.pb"] = w["l1.mix.pb"] + 0.1
    def gate(w): w["l1.mix.g"] = torch.zeros_like(w["l1.mix.g"])
    def o_bias(w): w["l1.mix.o.b"] = torch.zeros_like(w["l1.mix.o.b"])
    def k_bias(w): w["l4.mix.k.b"] = torch.zeros_like(w["l4.mix.k.b"])
    def k_norm(w): w["l1.mix.k.norm"] = torch.ones_like(w["l1.mix.k.norm"])
    def first_row(w): w["bigram"] = torch.cat([w["bigram"][:-1], torch.zeros_like(w["bigram"][-1:])])
    def z_bias(w): w["l0.mix.z.b"] = torch.zeros_like(w["l0.mix.z.b"])
    def latent_norm(w): w["l2.mix.dkv.norm"] = torch.ones_like(w["l2.mix.dkv.norm"])
    for change in (window, window_latent, no_window, value_base, ramp, ramp_edge, limit, mul, scale, eps):
        assert moved(change_cfg=change) > 10 * RTOL["f32"], change.__name__
    for change in (head_bias, gate, o_bias, k_bias, k_norm, first_row, z_bias, latent_norm):
        assert moved(change_w=change) > 10 * RTOL["f32"], change.__name__


@pytest.mark.parametrize("kind", ["f32", "bf16"])
@pytest.mark.parametrize("name", ["mix", "odd", "plain"])
def test_prefill_against_token_by_token_decoding(S, models, name, kind):
    """70 tokens in one step, then 80 one by one across the page border at 128 and past every window; and a second
    sequence decoded from its very first token (its pair row is the table's last, its states start at zero)"""
    folder, oracle, cfg = models[name]
    toks = tokens(150, cfg["vocab"], 3)
    want = oracle.forward(toks).numpy()
    m = open_model(S, folder, kind)
    got = [m.step([(0, toks[:70], list(range(70)))])]
    for t in range(70, 150):
        got.append(m.step([(0, [toks[t]], [0])]))
    check(np.concatenate(got), want, kind, "prompt then single tokens")
    got = [m.step([(1, [toks[t]], [0])]) for t in range(40)]
    check(np.concatenate(got), want[:40], kind, "single tokens from the first position")
    m.close()


@pytest.mark.parametrize("kind", ["f32", "bf16"])
@pytest.mark.parametrize("name", ["mix", "odd", "wide"])
def test_portions_of_many_sizes(S, models, name, kind):
    """the same prompt cut into portions of 1 .. 64 tokens (ending inside windows, chunks of the recurrence and pages)"""
    folder, oracle, cfg = models[name]
    toks = tokens(200, cfg["vocab"], 4)
    want = oracle.forward(toks).numpy()
    m = open_model(S, folder, kind)
    cuts, at = [2, 3, 2, 37, 5, 2, 64, 1, 1, 2, 29, 31, 2, 19], 0
    got = []
    for c in cuts:
        got.append(m.step([(0, toks[at: at + c], list(range(c)))]))
        at += c
    assert at == 200
    check(np.concatenate(got), want, kind)
    m.close()


@pytest.mark.parametrize("name", ["mix", "plain", "wide"])
def test_a_position_does_not_depend_on_the_cut_or_the_batch(S, models, name):
    """fp32: three unequal requests batched together (portions beside single tokens) against each alone in one step"""
    folder, oracle, cfg = models[name]
    V = cfg["vocab"]
    reqs = [tokens(90, V, 10), tokens(33, V, 11), tokens(140, V, 12)]
    m = open_model(S, folder, "f32")
    alone = []
    for r in reqs:
        alone.append(m.step([(3, r, list(range(len(r))))]))
        m.release(3)
    got = [[], [], []]
    plan = [[(0, 40), (1, 3), (2, 64)], [(0, 1), (1, 2), (2, 2)], [(0, 1), (2, 70)], [(0, 48), (1, 28), (2, 1)], [(2, 1)], [(2, 1)], [(2, 1)]]
    at = [0, 0, 0]
    for stp in plan:
        entries = [(i, reqs[i][at[i]: at[i] + c], list(range(c))) for i, c in stp]
        out = m.step(entries)
        o = 0
        for i, c in stp:
            got[i].append(out[o: o + c])
            o += c
            at[i] += c
    for i in range(3):
        assert at[i] == len(reqs[i])
        assert err(np.concatenate(got[i]), alone[i]) < 2e-5, i
        assert err(alone[i], oracle.forward(reqs[i]).numpy()) < RTOL["f32"]
    m.close()


@pytest.mark.parametrize("kind", ["f32", "bf16"])
def test_pages_slots_states_and_previous_tokens_used_again(S, models, kind):
    """a pool of three pages and two slots: requests follow one another through the same pages, recurrent states and
    previous-token places, which still hold what the previous owner left; an oversized step is refused without side effects"""
    folder, oracle, cfg = models["mix"]
    V = cfg["vocab"]
    m = open_model(S, folder, kind, max_tokens=192, slots=2)
    assert m.pages_total == 3
    for rnd in range(3):
        a, b = tokens(100, V, 20 + rnd), tokens(50, V, 30 + rnd)
        ga = [m.step([(0, a[:60], list(range(60)))])]
        gb = [m.step([(1, b[:10], list(range(10)))])]
        out = m.step([(0, a[60:], list(range(40))), (1, b[10:], list(range(40)))])
        ga.append(out[:40]); gb.append(out[40:])
        check(np.concatenate(ga), oracle.forward(a).numpy(), kind, f"turn {rnd}, first request")
        check(np.concatenate(gb), oracle.forward(b).numpy(), kind, f"turn {rnd}, second request")
        free = m.pages_free
        with pytest.raises(RuntimeError):
            m.step([(1, tokens(80, V, 1), [0])])          # 50 + 80 tokens need a third page for slot 1: none left
        assert m.pages_free == free and m.slot_length(1) == 50
        m.release(0)
        m.release(1)
        assert m.pages_free == 3
    m.close()


@pytest.mark.parametrize("kind", ["f32", "bf16"])
@pytest.mark.parametrize("name", ["mix", "wide"])
def test_long_decoding(S, models, name, kind):
    folder, oracle, cfg = models[name]
    n = 330 if name == "mix" else 420
    toks = tokens(n, cfg["vocab"], 5)
    want = oracle.forward(toks).numpy()
    m = open_model(S, folder, kind)
    got = [m.step([(0, toks[:10], list(range(10)))])]
    for t in range(10, n):     # the same single-token shape again and again: graph replay, windows that slide, page borders
        got.append(m.step([(0, [toks[t]], [0])]))
    check(np.concatenate(got), want, kind)
    m.close()


def test_long_prompt_in_one_step_and_in_portions(S, models):
    """700 tokens: the recurrence's chunk form, attention tiles over many key tiles, windows far from the sequence's start,
    against the same prompt in odd portions"""
    folder, oracle, cfg = models["wide"]
    toks = tokens(700, cfg["vocab"], 6)
    want = oracle.forward(toks).numpy()
    for kind in ("f32", "bf16"):
        m = open_model(S, folder, kind, max_tokens=2048)
        whole = m.step([(0, toks, list(range(700)))])
        check(whole, want, kind, "one step")
        got, at = [], 0
        for c in [301, 257, 2, 140]:
            got.append(m.step([(1, toks[at: at + c], list(range(c)))]))
            at += c
        check(np.concatenate(got), want, kind, "portions")
        if kind == "f32":
            assert err(np.concatenate(got), whole) < 2e-5
        m.close()


def test_a_key_at_the_window_edge_decides_the_logits(S, models, tmp_path):
    """one attention layer whose head bias shuts every key out (weights near zero) except the key of the token `mark`, which
    every later query opens. The logits at a position change by far
    more than the tolerance when `mark` moves from the last position inside the window to the first outside; the library has
    to follow the oracle on both sides, for prompt rows and for single tokens."""
    cfg, w = O.random_model(seed=5, width=32, vocab=30, buckets=None, layers=[
        dict(type="attention", heads=2, kv_heads=1, dim=8, vdim=8, window=20, rot_dims=0, pb=-9.0, ff=None)])
    mark = 7
    # every query is e0 after its head norm; a key is (r, 8 - r, 0, ...) before its norm with r = 8 for the marked token and
    # |r| of about one for the others: after the norm only the marked token's key lies along e0
    unit = w["embed"][mark] / (w["embed"][mark] ** 2).sum()
    w["l0.mix.q"] = torch.zeros_like(w["l0.mix.q"]); w["l0.mix.k"] = torch.zeros_like(w["l0.mix.k"])
    w["l0.mix.q.b"] = torch.zeros(16, dtype=O.DT); w["l0.mix.q.b"][0] = 1.0; w["l0.mix.q.b"][8] = 1.0
    w["l0.mix.k.b"] = torch.zeros(8, dtype=O.DT); w["l0.mix.k.b"][1] = 8.0
    w["l0.mix.k"][0] = unit * 8.0
    w["l0.mix.k"][1] = -unit * 8.0
    w["l0.mix.q.norm"] = torch.ones(8, dtype=O.DT); w["l0.mix.k.norm"] = torch.ones(8, dtype=O.DT)
    w["l0.mix.pb"] = torch.full((2,), -9.0, dtype=O.DT)
    w = {k: v.to(torch.bfloat16).to(O.DT) for k, v in w.items()}
    cfg["layers"][0]["mixer"]["scale"] = 2.0
    cfg["embedding"]["scale"] = 1.0
    O.write_model(str(tmp_path), cfg, w)
    oracle = O.Oracle(cfg, w)
    base = [t for t in tokens(60, 30, 9)]
    base = [t if t != mark else mark + 1 for t in base]
    inside, outside = list(base), list(base)
    inside[59 - 19] = mark        # position 40: the last one position 59 still sees
    outside[59 - 20] = mark       # position 39: the first one it does not
    wi, wo = oracle.forward(inside).numpy(), oracle.forward(outside).numpy()
    assert err(wi[59:], wo[59:]) > 0.2
    for kind in ("f32", "bf16"):
        m = open_model(S, str(tmp_path), kind)
        for seq, want in ((inside, wi), (outside, wo)):
            got = m.step([(0, seq, [58, 59])])
            check(got, want[58:], kind, "prompt rows")
            m.release(0)
            m.step([(0, seq[:59], [])])
            got = m.step([(0, seq[59:], [0])])
            check(got, want[59:], kind, "single token")
            m.release(0)
        m.close()


def test_refused_configurations(S, models, tmp_path):
    folder, oracle, cfg = models["odd"]
    def refused(change, text):
        c = copy.deepcopy(cfg)
        change(c)
        O.write_model(str(tmp_path), c, oracle.w)
        with pytest.raises(RuntimeError, match=text):
            S.Model(str(tmp_path), dtype=S.F32, max_tokens=64, max_slots=1)
    refused(lambda c: c["layers"][1].update(type="retention"), "not part of this family")
    refused(lambda c: c["layers"][0]["mlp"].update(kind="moe"), "not part of this family")
    refused(lambda c: c["layers"][3]["mixer"].update(kv_heads=4), "multiple of kv_heads")
    refused(lambda c: c["layers"][1]["mixer"]["rot"].update(dims=4), "rot_dim")
    refused(lambda c: c["layers"][2]["mixer"].update(width=3), "shape")


def test_greedy_generation_through_the_scheduler(S, models):
    """six requests on two slots with an end token, prompts fed in portions of 16 beside the others' single tokens,
    against greedy decoding with the oracle"""
    folder, oracle, cfg = models["mix"]
    V = cfg["vocab"]
    prompts = [tokens(n, V, 40 + i) for i, n in enumerate([5, 40, 17, 1, 33, 70])]
    max_new, eos = 12, 7
    want = []
    for p in prompts:
        seq, outp = list(p), []
        for k in range(max_new):
            nxt = int(oracle.forward(seq)[-1].argmax())
            if k > 0 and nxt == eos:
                break
            outp.append(nxt)
            seq.append(nxt)
        want.append(outp)
    m = open_model(S, folder, "f32", max_tokens=64 * 6, slots=2)
    outs, steps = m.generate(prompts, max_new=max_new, eos_id=eos, chunk=16)
    assert steps > max_new
    assert outs == want
    assert m.pages_free == m.pages_total
    m.close()

"""The Tomalix family through the library's own entry points (registry -> step function -> paged cache and slot state
-> scheduler) against the plain implementation in tomalix_oracle.py, on small random models of several shapes: whole
prompts with every layer run, prefill against token-by-token decoding, prompt portions down to two tokens (shorter than
the convolution), unequal batches against each request alone, pages, slots and carried state that are freed and used
again, block and page borders, long decoding, sizes that are 1 or equal to each other, layer spans that repeat, and
greedy generation through the continuous-batching scheduler."""
import copy

import numpy as np
import pytest
import torch

import tomalix_oracle as O

pytestmark = pytest.mark.gpu

RAMP = dict(factor=4.0, original=48, fast=8.0, slow=1.0)
SHAPES = {
    # every mixer and both feed-forwards; the span [differential, parallel] runs twice; blocks of 7 positions, so a page
    # of 64 rows holds block borders at places that are not its own
    "mix": dict(width=48, vocab=61, loop=(1, 3, 2), layers=[
        dict(type="parallel", heads=4, kv_heads=2, dim=16, vdim=8, chunk=7, rot_dims=8, base=100.0, inner=40, state=6, dt_rank=5,
             conv=3, left_scale=1.3, right_scale=0.7, ff=(24, 6, 2)),
        dict(type="attention", heads=2, kv_heads=1, dim=8, vdim=16, diff=0.25, scaling=dict(factor=4.0), ff=40),
        dict(type="parallel", heads=2, kv_heads=2, dim=8, vdim=8, chunk=64, inner=24, state=16, dt_rank=8, conv=4, ff=None),
        dict(type="attention_2", heads=4, kv_heads=2, dim=12, vdim=6, scaling=RAMP, base=50.0, ff=(16, 4, 4))]),
    # sizes that are 1 or equal; a one-tap convolution; one state; no rotation; one key head for six query heads; a span
    # of one layer at the start that runs three times; top = 1; no logit cap; blocks of one page and of one position
    "odd": dict(width=40, vocab=33, loop=(0, 1, 3), logit_softcap=None, layers=[
        dict(type="parallel", heads=1, kv_heads=1, dim=4, vdim=4, chunk=1, rot_dims=0, inner=10, state=1, dt_rank=1, conv=1, ff=8),
        dict(type="attention_2", heads=6, kv_heads=1, dim=6, vdim=10, rot_dims=4, ff=(8, 3, 1)),
        dict(type="attention", heads=1, kv_heads=1, dim=6, vdim=4, rot_dims=2, diff=0.6, ff=None),
        dict(type="parallel", heads=3, kv_heads=1, dim=10, vdim=6, chunk=130, rot_dims=10, scale=0.5, inner=7, state=9, dt_rank=3,
             conv=5, left_scale=1.0, right_scale=1.0, ff=None)]),
    # no span; nothing a multiple of 8; attention without any frequency change; more states than one lane holds
    "plain": dict(width=36, vocab=41, layers=[
        dict(type="attention_2", heads=3, kv_heads=3, dim=10, vdim=7, ff=20),
        dict(type="attention", heads=5, kv_heads=5, dim=6, vdim=9, rot_dims=4, ff=(12, 5, 3)),
        dict(type="parallel", heads=2, kv_heads=1, dim=14, vdim=18, chunk=33, inner=20, state=70, dt_rank=2, conv=2, ff=28)]),
    # heads as wide as the tensor-core tiles take them, group sizes of the decode kernel, a span that ends the model
    "wide": dict(width=64, vocab=50, loop=(1, 3, 2), layers=[
        dict(type="attention_2", heads=4, kv_heads=2, dim=64, vdim=64, scaling=RAMP, ff=128),
        dict(type="parallel", heads=8, kv_heads=1, dim=32, vdim=32, chunk=100, inner=128, state=16, dt_rank=8, conv=4, ff=None),
        dict(type="attention", heads=2, kv_heads=1, dim=64, vdim=128, scaling=dict(factor=2.0), ff=(64, 8, 2))]),
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
        cfg, w = O.random_model(seed=90 + i, **sh)
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
    """fp32: every row within the tolerance. bfloat16: the unit RMS of a differential head whose two maps nearly cancel
    turns a rounding error into a large relative change of that head, which moves the row by more than rounding does
    elsewhere; so nine rows in ten have to be within the tolerance, the median well inside it, and no row anywhere near a
    wrong answer."""
    e = row_errors(got, want)
    assert np.all(np.isfinite(e)), what
    if kind == "f32":
        assert e.max() < RTOL[kind], (what, float(e.max()))
    else:
        assert np.quantile(e, 0.9) < RTOL[kind] and np.median(e) < RTOL[kind] / 2 and e.max() < 0.6, \
            (what, float(np.quantile(e, 0.9)), float(np.median(e)), float(e.max()))


def open_model(S, folder, kind, max_tokens=1024, slots=4):
    return S.Model(folder, dtype=S.BF16 if kind == "bf16" else S.F32, max_tokens=max_tokens, max_slots=slots)


@pytest.mark.parametrize("kind", ["f32", "bf16"])
@pytest.mark.parametrize("name", list(SHAPES))
def test_whole_prompt_and_every_layer_run(S, models, name, kind):
    folder, oracle, cfg = models[name]
    m = open_model(S, folder, kind)
    runs = O.layer_order(cfg)
    assert m.family == "Tomalix" and m.vocab == cfg["vocab"] and m.n_layers == len(runs)
    toks = tokens(150, cfg["vocab"], 1)
    m.capture_layers(True)
    got = m.step([(0, toks, list(range(150)))])
    want, trail = oracle.forward(toks, return_layers=True)
    layers = m.captured_layers(150)
    for i in range(len(runs)):
        check(layers[i], trail[i].numpy(), kind, f"residual after layer run {i} (layer {runs[i][0]})")
    check(got, want.numpy(), kind)
    assert m.step_launches > 0
    m.close()


def test_every_mechanism_reaches_the_logits(models):
    """sensitivity of the comparison itself: with the block mask, the second score map, the frequency changes, the gate,
    the scan's history, the router's bias, the pass vectors or the embedding added back changed, the oracle's logits move
    by far more than the tolerance the library is held to"""
    _, oracle, cfg = models["mix"]
    toks = tokens(60, cfg["vocab"], 2)
    base = oracle.forward(toks).numpy()

    def moved(change_cfg=None, change_w=None):
        c, w = copy.deepcopy(cfg), dict(oracle.w)
        if change_cfg:
            change_cfg(c)
        if change_w:
            change_w(w)
        return err(O.Oracle(c, w).forward(toks).numpy(), base)

    def block(c): c["layers"][0]["mixer"]["left"]["mask"]["size"] = 8
    def no_block(c): del c["layers"][0]["mixer"]["left"]["mask"]
    def diff(c): c["layers"][1]["mixer"]["diff"] = 0.3
    def linear(c): del c["layers"][1]["mixer"]["rot"]["scaling"]
    def ramp(c): del c["layers"][3]["mixer"]["rot"]["scaling"]
    def ramp_edge(c): c["layers"][3]["mixer"]["rot"]["scaling"]["slow"] = 0.25
    def times(c): c["loop"]["times"] = 1
    def weights(c): c["layers"][0]["mixer"]["left_scale"] = 1.0
    def top(c): c["layers"][0]["mlp"]["router"]["top"] = 1
    def cap(c): c["logit_softcap"] = 80.0
    def lam(w): w["l1.mix.lq2"] = w["l1.mix.lq2"] * 0.5
    def gate(w): w["l0.mix.left.g"] = torch.zeros_like(w["l0.mix.left.g"])
    def conv(w): w["l0.mix.right.conv"] = torch.cat([torch.zeros_like(w["l0.mix.right.conv"][:, :1]), w["l0.mix.right.conv"][:, 1:]], 1)
    def decay(w): w["l2.mix.right.A_log"] = w["l2.mix.right.A_log"] + 1.0
    def skip(w): w["l0.mix.right.D"] = torch.zeros_like(w["l0.mix.right.D"])
    def router_bias(w): w["l0.mlp.router.b"] = torch.zeros_like(w["l0.mlp.router.b"])
    def pass_vector(w): w["loop.step"] = torch.cat([w["loop.step"][:1], torch.zeros_like(w["loop.step"][1:])], 0)
    def norm_offset(w): w["l1.norm1"] = w["l1.norm1"] - 1.0
    for change in (block, no_block, diff, linear, ramp, ramp_edge, times, weights, top, cap):
        assert moved(change_cfg=change) > 10 * RTOL["f32"], change.__name__
    for change in (lam, gate, conv, decay, skip, router_bias, pass_vector, norm_offset):
        assert moved(change_w=change) > 10 * RTOL["f32"], change.__name__


@pytest.mark.parametrize("kind", ["f32", "bf16"])
@pytest.mark.parametrize("name", ["mix", "odd", "plain"])
def test_prefill_against_token_by_token_decoding(S, models, name, kind):
    """70 tokens in one step, then 80 one by one across the page border at 128 and many block borders; and a second
    sequence decoded from its very first token"""
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
    """the same prompt cut into portions of 2 .. 37 tokens (shorter than the convolution, ending inside blocks and pages)"""
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
def test_pages_slots_and_states_used_again(S, models, kind):
    """a pool of three pages and two slots: requests follow one another through the same pages, rings and scan states,
    which still hold what the previous owner left; an oversized step is refused without side effects"""
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
def test_long_decoding(S, models, kind):
    folder, oracle, cfg = models["mix"]
    toks = tokens(330, cfg["vocab"], 5)
    want = oracle.forward(toks).numpy()
    m = open_model(S, folder, kind)
    got = [m.step([(0, toks[:10], list(range(10)))])]
    for t in range(10, 330):     # the same single-token shape again and again: graph replay, growing contexts, five page borders
        got.append(m.step([(0, [toks[t]], [0])]))
    check(np.concatenate(got), want, kind)
    m.close()


def test_long_prompt_in_one_step_and_in_portions(S, models):
    """700 tokens: the scan's chunk form, attention tiles over many key tiles, against the same prompt in odd portions"""
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


def test_prompt_long_enough_for_dense_expert_products(S, models):
    """1100 tokens in one step: in bfloat16 the routed experts run as dense products per expert on side streams (from 1024
    tokens on); the same prompt in portions below that stays on the grouped kernel. Both against the oracle, and against
    each other"""
    folder, oracle, cfg = models["wide"]
    toks = tokens(1100, cfg["vocab"], 8)
    want = oracle.forward(toks).numpy()
    m = open_model(S, folder, "bf16", max_tokens=2560)
    whole = m.step([(0, toks, list(range(1100)))])
    check(whole, want, "bf16", "one step")
    got, at = [], 0
    for c in [500, 598, 2]:
        got.append(m.step([(1, toks[at: at + c], list(range(c)))]))
        at += c
    parts = np.concatenate(got)
    check(parts, want, "bf16", "portions")
    e = row_errors(whole, parts)
    assert np.median(e) < 2e-2 and np.quantile(e, 0.9) < RTOL["bf16"], (float(np.median(e)), float(e.max()))
    m.release(0)
    again = m.step([(2, toks, list(range(1100)))])          # the side streams once more, pages in another order
    assert err(again, whole) < 1e-6
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
    refused(lambda c: c["layers"][0]["mlp"].update(kind="glu"), "not part of this family")
    refused(lambda c: c["loop"].update(stop=9), "loop")
    refused(lambda c: c["layers"][1]["mixer"].update(kv_heads=4), "multiple of kv_heads")
    refused(lambda c: c["layers"][2]["mixer"].update(dim=8), "lq1|shape")


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

"""Prefill and decode throughput of a model family served through include/b200_serve.h, beside the LLaMA engine at
equal size (same width, heads, layers, vocabulary and the same feed-forward width per token), random weights.
Called by bench.py --workload nekodra | musilorn; prints one JSON line."""
import json
import os
import tempfile
import time

SIZES = {
    # width, heads, dim, vdim, kv_rank, experts, ff, top, identity, shared_ff, layers, vocab
    "s": dict(width=1024, heads=8, dim=128, vdim=128, kv_rank=256, experts=8, ff=512, top=2, identity=2, shared_ff=1024,
              n_layers=4, vocab=32000),
    "m": dict(width=2048, heads=16, dim=128, vdim=128, kv_rank=512, experts=16, ff=1024, top=4, identity=2, shared_ff=2048,
              n_layers=4, vocab=32000),
}


MUSILORN_SIZES = {
    # attention layers with a dense feed-forward; the last layer is a retention layer without one
    "s": dict(width=1024, heads=8, kv_heads=4, dim=128, ff=4096, n_layers=4, vocab=32000, retention_every=4, ret_heads=4, ret_dim=128,
              ret_vdim=256),
    "m": dict(width=2048, heads=16, kv_heads=8, dim=128, ff=8192, n_layers=4, vocab=32000, retention_every=4, ret_heads=8, ret_dim=128,
              ret_vdim=256),
}


def tomalix_layers(width, heads, kv_heads, dim, ff, chunk, **_):
    """four layers: block-masked gated attention beside a scan with a dense feed-forward; plain attention with routed experts
    (four of sixteen, the same feed-forward width per token); differential attention (half the heads, two maps each, values
    twice as wide); plain attention with a dense feed-forward"""
    return [
        dict(type="parallel", heads=heads, kv_heads=kv_heads, dim=dim, vdim=dim, chunk=chunk, inner=2 * width, state=16,
             dt_rank=width // 16, conv=4, ff=ff),
        dict(type="attention_2", heads=heads, kv_heads=kv_heads, dim=dim, vdim=dim, ff=(ff // 4, 16, 4)),
        dict(type="attention", heads=heads // 2, kv_heads=kv_heads // 2, dim=dim, vdim=2 * dim, ff=ff),
        dict(type="attention_2", heads=heads, kv_heads=kv_heads, dim=dim, vdim=dim, ff=ff),
    ]


TOMALIX_SIZES = {
    "s": dict(width=1024, heads=8, kv_heads=4, dim=128, ff=4096, chunk=1024, n_layers=4, vocab=32000),
    "m": dict(width=2048, heads=16, kv_heads=8, dim=128, ff=8192, chunk=1024, n_layers=4, vocab=32000),
}


def sakevik_layers(width, heads, kv_heads, dim, ff, window, kv_rank, rot_dim, **_):
    """four layers: a gated recurrence twice as wide as the model, without a feed-forward; windowed sigmoid attention with
    rotated values; windowed latent attention with a rotated key part; the sigmoid attention again; the last three with a
    clamped gated feed-forward"""
    return [
        dict(type="mingru", width=2 * width, ff=None),
        dict(type="attention", heads=heads, kv_heads=kv_heads, dim=dim, vdim=dim, window=window, ff=(ff, 7.0)),
        dict(type="latent_attention", heads=heads, dim=dim, rot_dim=rot_dim, vdim=dim, kv_rank=kv_rank, window=window, ff=(ff, 7.0)),
        dict(type="attention", heads=heads, kv_heads=kv_heads, dim=dim, vdim=dim, window=window, ff=(ff, 7.0)),
    ]


# ff: a gated unit holds three matrices where the squared-relu unit of Tomalix holds two, so two thirds of its hidden width
# (rounded to 128) give the same feed-forward weights per layer
SAKEVIK_SIZES = {
    "s": dict(width=1024, heads=8, kv_heads=4, dim=128, ff=2688, window=1024, kv_rank=256, rot_dim=64, n_layers=4, vocab=32000),
    "m": dict(width=2048, heads=16, kv_heads=8, dim=128, ff=5504, window=1024, kv_rank=512, rot_dim=64, n_layers=4, vocab=32000),
}


def timed(fn, steps, warmup):
    import torch
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    for _ in range(steps):
        fn()
    torch.cuda.synchronize()
    return (time.perf_counter() - t0) / steps


def run(pkg, size="m", prompt=2048, batch=8, context=1024, steps=10, warmup=3, dtype="bfloat16", family="nekodra"):
    import numpy as np
    import torch

    S, E, capi = pkg.serve, pkg.engine, pkg.capi
    if family == "tomalix":
        return run_tomalix(pkg, size, prompt, batch, context, steps, warmup, dtype)
    if family == "sakevik":
        return run_sakevik(pkg, size, prompt, batch, context, steps, warmup, dtype)
    sz = (MUSILORN_SIZES if family == "musilorn" else SIZES)[size]
    rng = np.random.default_rng(0)
    out = {"workload": family, "size": size, "shape": sz, "prompt": prompt, "decode_batch": batch, "decode_context": context,
           "dtype": dtype, "data": "synthetic ids, random weights", "timing": "host clock around synchronous steps (each step ends "
           "with the device-to-host copy of its results), after warm-up"}
    with tempfile.TemporaryDirectory() as folder:
        if family == "musilorn":
            cfg, w = S.random_musilorn(**sz)
        else:
            cfg, w = S.random_nekodra(max_positions=max(prompt, context + steps + warmup + 8) + 64, **sz)
        S.write_checkpoint(folder, cfg, w)
        del w
        PR = 64
        need = max(prompt + PR, batch * (context + steps + warmup + PR + 8))
        m = S.Model(folder, dtype=S.BF16 if dtype == "bfloat16" else S.F32, max_tokens=need, max_slots=batch)
    V = sz["vocab"]
    ids = rng.integers(0, V, prompt).tolist()

    def prefill():
        m.step([(0, ids, [prompt - 1])], logits=False, ids=True)
        m.release(0)
    t = timed(prefill, steps, warmup)
    out["prefill"] = {"tokens_per_s": prompt / t, "ms": t * 1e3, "launches": m.step_launches}
    for b in range(batch):
        m.step([(b, rng.integers(0, V, context).tolist(), [])], logits=False)
    tok = rng.integers(0, V, batch).tolist()

    def decode():
        m.step([(b, [tok[b]], [0]) for b in range(batch)], logits=False, ids=True)
    t = timed(decode, steps, warmup)
    out["decode"] = {"tokens_per_s": batch / t, "ms": t * 1e3, "launches": m.step_launches}
    m.close()

    # the closest existing model: the LLaMA engine with the same width, heads, layers and vocabulary, and the
    # feed-forward width a Nekodra token actually uses (its chosen experts + the shared one); fp16
    # (Musilorn: the same grouped heads and feed-forward width; its retention layer stands against one more attention layer)
    inter = sz["ff"] if family == "musilorn" else sz["top"] * sz["ff"] + sz["shared_ff"]
    shape = dict(num_layers=sz["n_layers"], head_num=sz["heads"], kv_head_num=sz.get("kv_heads", sz["heads"]), head_size=sz["dim"],
                 inter_size=inter, vocab_size=V)
    ll = {"shape": shape, "dtype": "fp16"}
    try:
        eng = E.Engine(1, prompt + 8, dtype=capi.F16, **shape)
        eng.init_random(seed=1, std=0.02)
        pid = rng.integers(0, V, (1, prompt)).astype(np.int32)

        def ll_prefill():
            eng.reset()
            eng.prefill(pid)
        t = timed(ll_prefill, steps, warmup)
        ll["prefill"] = {"tokens_per_s": prompt / t, "ms": t * 1e3}
        eng.close()
        eng = E.Engine(batch, context + steps + warmup + 16, dtype=capi.F16, **shape)
        eng.init_random(seed=1, std=0.02)
        eng.fill_kv_random(context, seed=2, amp=0.5)
        did = rng.integers(0, V, batch).astype(np.int32)
        t = timed(lambda: eng.decode_step_host(did), steps, warmup)
        ll["decode"] = {"tokens_per_s": batch / t, "ms": t * 1e3, "launches": eng.launches_per_step}
        eng.close()
    except Exception as ex:   # the comparison must not take the family's own numbers down
        ll["failed"] = f"{type(ex).__name__}: {ex}"
    out["llama_equal_size"] = ll
    return out


def serve_family(S, cfg, w, prompt, batch, context, steps, warmup, dtype, vocab):
    """prefill of one prompt and decode steps of `batch` sequences at `context` tokens through b200_model_step"""
    import numpy as np

    rng = np.random.default_rng(0)
    with tempfile.TemporaryDirectory() as folder:
        S.write_checkpoint(folder, cfg, w)
        PR = 64
        need = max(prompt + PR, batch * (context + steps + warmup + PR + 8))
        m = S.Model(folder, dtype=S.BF16 if dtype == "bfloat16" else S.F32, max_tokens=need, max_slots=batch)
    ids = rng.integers(0, vocab, prompt).tolist()
    out = {}

    def prefill():
        m.step([(0, ids, [prompt - 1])], logits=False, ids=True)
        m.release(0)
    t = timed(prefill, steps, warmup)
    out["prefill"] = {"tokens_per_s": prompt / t, "ms": t * 1e3, "launches": m.step_launches}
    for b in range(batch):
        m.step([(b, rng.integers(0, vocab, context).tolist(), [])], logits=False)
    tok = rng.integers(0, vocab, batch).tolist()

    def decode():
        m.step([(b, [tok[b]], [0]) for b in range(batch)], logits=False, ids=True)
    t = timed(decode, steps, warmup)
    out["decode"] = {"tokens_per_s": batch / t, "ms": t * 1e3, "launches": m.step_launches}
    m.close()
    return out


def run_tomalix(pkg, size, prompt, batch, context, steps, warmup, dtype):
    """The Tomalix family beside the closest existing one, Musilorn (the same serving layer, paged attention, a recurrent
    layer with carried state, fp32 residual), at equal width, heads, feed-forward width per token, layer count and vocabulary."""
    S = pkg.serve
    sz = TOMALIX_SIZES[size]
    out = {"workload": "tomalix", "size": size, "shape": sz, "prompt": prompt, "decode_batch": batch, "decode_context": context,
           "dtype": dtype, "data": "synthetic ids, random weights", "timing": "host clock around synchronous steps (each step ends "
           "with the device-to-host copy of its results), after warm-up"}
    cfg, w = S.random_tomalix(sz["width"], sz["vocab"], tomalix_layers(**sz))
    out.update(serve_family(S, cfg, w, prompt, batch, context, steps, warmup, dtype, sz["vocab"]))
    del w
    mu = dict(MUSILORN_SIZES[size])
    try:
        cfg, w = S.random_musilorn(**mu)
        res = serve_family(S, cfg, w, prompt, batch, context, steps, warmup, dtype, mu["vocab"])
        res["shape"] = mu
        out["musilorn_equal_size"] = res
    except Exception as ex:   # the comparison must not take the family's own numbers down
        out["musilorn_equal_size"] = {"failed": f"{type(ex).__name__}: {ex}"}
    return out


def run_sakevik(pkg, size, prompt, batch, context, steps, warmup, dtype):
    """The Sakevik family beside the closest existing one, Tomalix (the same serving layer and fp32 residual; gated attention
    with a mask, a recurrence with carried state, dense feed-forwards), at equal width, heads, head size, layer count,
    vocabulary and feed-forward weights per layer."""
    S = pkg.serve
    sz = SAKEVIK_SIZES[size]
    out = {"workload": "sakevik", "size": size, "shape": sz, "prompt": prompt, "decode_batch": batch, "decode_context": context,
           "dtype": dtype, "data": "synthetic ids, random weights", "timing": "host clock around synchronous steps (each step ends "
           "with the device-to-host copy of its results), after warm-up"}
    cfg, w = S.random_sakevik(sz["width"], sz["vocab"], sakevik_layers(**sz))
    out.update(serve_family(S, cfg, w, prompt, batch, context, steps, warmup, dtype, sz["vocab"]))
    del w
    tx = dict(TOMALIX_SIZES[size])
    try:
        cfg, w = S.random_tomalix(tx["width"], tx["vocab"], tomalix_layers(**tx))
        res = serve_family(S, cfg, w, prompt, batch, context, steps, warmup, dtype, tx["vocab"])
        res["shape"] = tx
        out["tomalix_equal_size"] = res
    except Exception as ex:   # the comparison must not take the family's own numbers down
        out["tomalix_equal_size"] = {"failed": f"{type(ex).__name__}: {ex}"}
    return out

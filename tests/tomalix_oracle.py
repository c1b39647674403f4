"""Plain, slow statement of the Tomalix decoder, one function per mechanism (torch on the CPU, float64 by default).

Shares no code with the product path: the tests build small random models, run them through the library and compare
with these functions. Every function sees a WHOLE sequence from position 0; nothing is cached.

Design: pre-norm layers x <- x + mixer(N1 x), x <- x + ff(N2 x) with N x = x / rms(x) * (1 + w). Three mixers:
"attention" (differential: two score maps per head over shared values, combined as a1 - lambda a2, unit RMS, rotary
positions with linearly stretched frequencies), "parallel" (a sigmoid-gated attention that only looks inside its own
chunk of positions, beside a selective-scan recurrence; their outputs are added with two weights) and "attention_2"
(plain grouped-query attention with the ramped frequency interpolation and its amplitude factor). Feed-forwards: dense
squared-relu, or a routed mixture of such experts (top-k on the logits, softmax over the chosen). A span of layers
runs several times; each pass adds a per-pass vector (and, from the second pass on, the embedding output) to x.
The logits are tanh-capped.

A model is (config dict as in config.json, dict name -> tensor).
"""
import math

import torch

DT = torch.float64


def rms_norm(x, w, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps) * (1 + w)


def unit_rms(x, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def relu2(z):
    return torch.relu(z) ** 2


def silu(z):
    return z * torch.sigmoid(z)


def softplus(z):
    return torch.where(z > 30, z, torch.log1p(torch.exp(torch.clamp(z, max=30))))


def rot_frequencies(rot, kind):
    """(frequencies [dims/2], amplitude). kind 'plain': base^(-2i/dims); 'linear': those divided by scaling.factor;
    'ramp': blended between f and f / factor by a ramp over the index, amplitude 0.1 ln(factor) + 1."""
    d, base = rot["dims"], rot["base"]
    f = [base ** (-2.0 * i / d) for i in range(d // 2)]
    sc = rot.get("scaling")
    amp = 1.0
    if kind == "linear" and sc:
        f = [fi / sc["factor"] for fi in f]
    elif kind == "ramp" and sc:
        def index_of(turns):
            return d * math.log(sc["original"] / (2 * math.pi * turns)) / (2 * math.log(base))
        lo = max(math.floor(index_of(sc["fast"])), 0)
        hi = min(math.ceil(index_of(sc["slow"])), d - 1)
        out = []
        for i, fi in enumerate(f):
            r = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
            out.append(fi / sc["factor"] * r + fi * (1 - r))
        f = out
        amp = 0.1 * math.log(sc["factor"]) + 1.0
    return torch.tensor(f, dtype=DT), amp


def rotate_half(x, rot, kind):
    """x [T, heads, dim], positions 0..T-1: the first rot['dims'] dimensions of every head, i paired with i + dims/2"""
    if not rot or not rot.get("dims"):
        return x
    T, d = x.shape[0], rot["dims"]
    f, amp = rot_frequencies(rot, kind)
    ang = torch.arange(T, dtype=DT)[:, None] * f[None, :]
    c, s = (amp * torch.cos(ang))[:, None, :], (amp * torch.sin(ang))[:, None, :]
    out = x.clone()
    u, v = x[..., : d // 2], x[..., d // 2: d]
    out[..., : d // 2] = u * c - v * s
    out[..., d // 2: d] = v * c + u * s
    return out


def visible(T, chunk=None):
    """[T, T] bool: row i sees column j <= i (and, with chunk, only inside i's own block of `chunk` positions)"""
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    m = j <= i
    if chunk:
        m = m & (i // chunk == j // chunk)
    return m


def softmax_attention(q, k, v, scale, mask):
    """q [T, H, d], k [T, H, d], v [T, H, dv] (one key / value head per query head already) -> [T, H, dv]"""
    s = torch.einsum("ihd,jhd->hij", q, k) * scale
    s = s.masked_fill(~mask[None], float("-inf"))
    p = torch.softmax(s, dim=-1)
    return torch.einsum("hij,jhd->ihd", p, v)


def expand_groups(t, heads):
    """[T, G, d] -> [T, heads, d]: query head h reads group h // (heads / G)"""
    G = t.shape[1]
    return t.repeat_interleave(heads // G, dim=1)


def plain_attention(h, mx, W, pre, eps):
    """mixer 'attention_2'"""
    T, H, G, d, dv = h.shape[0], mx["heads"], mx["kv_heads"], mx["dim"], mx["vdim"]
    q = (h @ W[pre + "q"].T).reshape(T, H, d)
    k = (h @ W[pre + "k"].T).reshape(T, G, d)
    v = (h @ W[pre + "v"].T).reshape(T, G, dv)
    q, k = rotate_half(q, mx.get("rot"), "ramp"), rotate_half(k, mx.get("rot"), "ramp")
    o = softmax_attention(q, expand_groups(k, H), expand_groups(v, H), mx["scale"], visible(T))
    return o.reshape(T, H * dv) @ W[pre + "o"].T


def differential_attention(h, mx, W, pre, eps):
    """mixer 'attention': per head two maps [q1 | q2], [k1 | k2] over the same values"""
    T, H, G, d, dv = h.shape[0], mx["heads"], mx["kv_heads"], mx["dim"], mx["vdim"]
    q = (h @ W[pre + "q"].T).reshape(T, H, 2, d)
    k = (h @ W[pre + "k"].T).reshape(T, G, 2, d)
    v = expand_groups((h @ W[pre + "v"].T).reshape(T, G, dv), H)
    maps = []
    for m in range(2):
        qm, km = rotate_half(q[:, :, m], mx.get("rot"), "linear"), rotate_half(k[:, :, m], mx.get("rot"), "linear")
        maps.append(softmax_attention(qm, expand_groups(km, H), v, mx["scale"], visible(T)))
    lam = torch.exp((W[pre + "lq1"] * W[pre + "lk1"]).sum()) - torch.exp((W[pre + "lq2"] * W[pre + "lk2"]).sum()) + mx["diff"]
    o = unit_rms(maps[0] - lam * maps[1], eps) * (1 - mx["diff"])
    return o.reshape(T, H * dv) @ W[pre + "o"].T


def gated_chunk_attention(h, mx, W, pre):
    """left half of 'parallel': keys only from the query's own block of mask.size positions; sigmoid output gate"""
    T, H, G, d, dv = h.shape[0], mx["heads"], mx["kv_heads"], mx["dim"], mx["vdim"]
    q = (h @ W[pre + "q"].T).reshape(T, H, d)
    k = (h @ W[pre + "k"].T).reshape(T, G, d)
    v = (h @ W[pre + "v"].T).reshape(T, G, dv)
    q, k = rotate_half(q, mx.get("rot"), "plain"), rotate_half(k, mx.get("rot"), "plain")
    o = softmax_attention(q, expand_groups(k, H), expand_groups(v, H), mx["scale"], visible(T, (mx.get("mask") or {}).get("size")))
    o = o.reshape(T, H * dv) * torch.sigmoid(h @ W[pre + "g"].T)
    return o @ W[pre + "o"].T


def causal_conv(u, w, b):
    """u [T, C], w [C, taps], b [C]: y_t = b + sum_j w[:, j] u_(t - taps + 1 + j), zeros before the start"""
    T, taps = u.shape[0], w.shape[1]
    y = b.expand(T, -1).clone()
    for j in range(taps):
        back = taps - 1 - j
        if back < T:
            y[back:] += w[:, j] * u[: T - back]
    return y


def selective_scan(h, mx, W, pre):
    """right half of 'parallel'"""
    T, C, N, R = h.shape[0], mx["inner"], mx["state"], mx["dt_rank"]
    xz = h @ W[pre + "in"].T
    x, z = xz[:, :C], xz[:, C:]
    x = silu(causal_conv(x, W[pre + "conv"], W[pre + "conv.b"]))
    p = x @ W[pre + "x"].T
    dt = softplus(p[:, :R] @ W[pre + "dt"].T + W[pre + "dt.b"])    # [T, C]
    B, Cm = p[:, R: R + N], p[:, R + N: R + 2 * N]
    A = -torch.exp(W[pre + "A_log"])                                # [C, N]
    S = torch.zeros(C, N, dtype=h.dtype)
    y = torch.zeros(T, C, dtype=h.dtype)
    for t in range(T):
        S = torch.exp(dt[t][:, None] * A) * S + (dt[t] * x[t])[:, None] * B[t][None, :]
        y[t] = S @ Cm[t] + W[pre + "D"] * x[t]
    return (y * silu(z)) @ W[pre + "o"].T


def parallel_mixer(h, mx, W, pre):
    return mx["left_scale"] * gated_chunk_attention(h, mx["left"], W, pre + "left.") + \
        mx["right_scale"] * selective_scan(h, mx["right"], W, pre + "right.")


def dense_ff(h, W, pre):
    return relu2(h @ W[pre + "up"].T) @ W[pre + "down"].T


def routed_ff(h, ml, W, pre):
    E, top = ml["router"]["experts"], ml["router"]["top"]
    z = h @ W[pre + "router"].T + W[pre + "router.b"]
    val, idx = torch.topk(z, top, dim=-1)
    wt = torch.softmax(val, dim=-1)
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for j in range(top):
            e = int(idx[t, j])
            out[t] += wt[t, j] * dense_ff(h[t: t + 1], W, pre + "e%d." % e)[0]
    return out


def layer_order(cfg):
    """[(layer index, pass number or None)]: which layer runs when; a pass number marks the first layer of a pass"""
    n = len(cfg["layers"])
    lp = cfg.get("loop")
    if not lp:
        return [(i, None) for i in range(n)]
    order = [(i, None) for i in range(lp["start"])]
    for t in range(lp["times"]):
        order += [(i, t if i == lp["start"] else None) for i in range(lp["start"], lp["stop"])]
    return order + [(i, None) for i in range(lp["stop"], n)]


def forward(cfg, W, tokens, keep_layers=False, dtype=DT):
    """logits [T, vocab] of a whole sequence (and the residual stream after every layer run)"""
    W = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in W.items()}
    eps = cfg["norm"]["eps"]
    x = W["embed"][torch.as_tensor(tokens, dtype=torch.long)]
    x0 = x.clone()
    kept = []
    for i, pass_no in layer_order(cfg):
        lj, pre = cfg["layers"][i], "l%d." % i
        if pass_no is not None:
            if pass_no > 0:
                x = x + x0
            x = x + W["loop.step"][pass_no]
        h = rms_norm(x, W[pre + "norm1"], eps)
        mx = lj["mixer"]
        if lj["type"] == "attention":
            x = x + differential_attention(h, mx, W, pre + "mix.", eps)
        elif lj["type"] == "attention_2":
            x = x + plain_attention(h, mx, W, pre + "mix.", eps)
        elif lj["type"] == "parallel":
            x = x + parallel_mixer(h, mx, W, pre + "mix.")
        else:
            raise ValueError(lj["type"])
        ml = lj.get("mlp")
        if ml:
            h = rms_norm(x, W[pre + "norm2"], eps)
            x = x + (dense_ff(h, W, pre + "mlp.") if ml["kind"] == "dense" else routed_ff(h, ml, W, pre + "mlp."))
        if keep_layers:
            kept.append(x.clone())
    logits = rms_norm(x, W["final.norm"], eps) @ W["head"].T
    cap = cfg.get("logit_softcap")
    if cap:
        logits = cap * torch.tanh(logits / cap)
    return (logits, torch.stack(kept)) if keep_layers else logits


class Oracle:
    def __init__(self, cfg, w):
        self.cfg, self.w = cfg, w

    def forward(self, tokens, return_layers=False):
        return forward(self.cfg, self.w, tokens, keep_layers=return_layers)


# ---------------------------------------------------------------------------------------------------------------
# small random models for the tests (weights rounded to bfloat16, as a checkpoint stores them)
# ---------------------------------------------------------------------------------------------------------------
def random_model(seed, width, vocab, layers, loop=None, logit_softcap=8.0, eps=1e-5):
    """layers: dicts with type 'attention' | 'parallel' | 'attention_2', the attention's heads, kv_heads, dim, vdim and
    optionally rot_dims, base, scale, scaling, chunk (parallel), diff (attention); the scan's inner, state, dt_rank, conv
    and the two weights left_scale, right_scale (parallel); ff = None | int (dense) | (ff, experts, top)."""
    g = torch.Generator().manual_seed(seed)

    def rnd(*shape, s=None):
        return (torch.randn(*shape, generator=g) * (s if s is not None else 1.0 / math.sqrt(shape[-1]))).to(torch.bfloat16).to(DT)

    cfg = dict(architecture="Tomalix", vocab=vocab, width=width, norm=dict(eps=eps), layers=[])
    if logit_softcap:
        cfg["logit_softcap"] = logit_softcap
    w = {"embed": rnd(vocab, width, s=1.0), "head": rnd(vocab, width), "final.norm": rnd(width, s=0.1)}
    if loop:
        cfg["loop"] = dict(start=loop[0], stop=loop[1], times=loop[2])
        w["loop.step"] = rnd(loop[2], width, s=0.3)

    def attention(sp, pre, gate):
        H, G, d, dv = sp["heads"], sp["kv_heads"], sp["dim"], sp["vdim"]
        maps = 2 if sp["type"] == "attention" else 1
        mx = dict(heads=H, kv_heads=G, dim=d, vdim=dv, scale=sp.get("scale", 1.0 / math.sqrt(d)))
        rd = sp.get("rot_dims", d)
        if rd:
            mx["rot"] = dict(base=sp.get("base", 10000.0), dims=rd)
            if sp.get("scaling"):
                mx["rot"]["scaling"] = dict(sp["scaling"])
        w[pre + "q"], w[pre + "k"], w[pre + "v"] = rnd(H * maps * d, width), rnd(G * maps * d, width), rnd(G * dv, width)
        w[pre + "o"] = rnd(width, H * dv)
        if gate:
            w[pre + "g"] = rnd(H * dv, width)
        return mx

    for i, sp in enumerate(layers):
        pre = "l%d." % i
        w[pre + "norm1"] = rnd(width, s=0.1)
        if sp["type"] == "parallel":
            left = attention(sp, pre + "mix.left.", True)
            if sp.get("chunk"):
                left["mask"] = dict(size=sp["chunk"])
            C, N, R, taps = sp["inner"], sp["state"], sp["dt_rank"], sp["conv"]
            rp = pre + "mix.right."
            w[rp + "in"], w[rp + "conv"], w[rp + "conv.b"] = rnd(2 * C, width), rnd(C, taps, s=0.5), rnd(C, s=0.2)
            w[rp + "x"], w[rp + "dt"] = rnd(R + 2 * N, C), rnd(C, R)
            w[rp + "dt.b"] = (torch.randn(C, generator=g) * 0.7 - 2.0).to(torch.bfloat16).to(DT)
            w[rp + "A_log"] = torch.log(torch.rand(C, N, generator=g) * 3 + 0.05).to(torch.bfloat16).to(DT)
            w[rp + "D"], w[rp + "o"] = rnd(C, s=1.0), rnd(width, C)
            mx = dict(left=left, right=dict(inner=C, state=N, dt_rank=R, conv=taps), left_scale=sp.get("left_scale", 1.0),
                      right_scale=sp.get("right_scale", 1.0))
        else:
            mx = attention(sp, pre + "mix.", False)
            if sp["type"] == "attention":
                mx["diff"] = sp.get("diff", 0.3)
                for nm in ("lq1", "lk1", "lq2", "lk2"):
                    w[pre + "mix." + nm] = rnd(sp["dim"], s=0.4)
        ff = sp.get("ff")
        if ff is None:
            ml = None
        else:
            w[pre + "norm2"] = rnd(width, s=0.1)
            if isinstance(ff, int):
                ml = dict(kind="dense", ff=ff)
                w[pre + "mlp.up"], w[pre + "mlp.down"] = rnd(ff, width), rnd(width, ff)
            else:
                f, E, top = ff
                ml = dict(kind="moe", expert=dict(ff=f), router=dict(experts=E, top=top))
                for e in range(E):
                    w[pre + "mlp.e%d.up" % e], w[pre + "mlp.e%d.down" % e] = rnd(f, width), rnd(width, f)
                w[pre + "mlp.router"], w[pre + "mlp.router.b"] = rnd(E, width, s=1.0), rnd(E, s=0.5)
        cfg["layers"].append(dict(type=sp["type"], mixer=mx, mlp=ml))
    return cfg, w


def write_model(folder, cfg, w):
    """config.json + model.safetensors with every tensor as bfloat16"""
    import json
    import os
    import struct

    os.makedirs(folder, exist_ok=True)
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(cfg, f)
    header, blobs, off = {}, [], 0
    for name, t in w.items():
        raw = t.to(torch.bfloat16).contiguous().view(torch.int16).numpy().tobytes()
        header[name] = dict(dtype="BF16", shape=list(t.shape), data_offsets=[off, off + len(raw)])
        blobs.append(raw)
        off += len(raw)
    hj = json.dumps(header).encode()
    hj += b" " * (-len(hj) % 8)
    with open(os.path.join(folder, "model.safetensors"), "wb") as f:
        f.write(struct.pack("<Q", len(hj)))
        f.write(hj)
        for b in blobs:
            f.write(b)

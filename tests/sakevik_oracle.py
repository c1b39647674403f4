"""Plain, slow statement of the Sakevik decoder, one function per mechanism (torch on the CPU, float64 by default).

Shares no code with the product path: the tests build small random models, run them through the library and compare
with these functions. Every function sees a WHOLE sequence from position 0; nothing is cached.

Design: the norm sits on a sublayer's OUTPUT, x <- x + N1(mixer(x)), x <- x + N2(ff(x)), N y = y / rms(y) * w, and the
sublayers read x itself. The embedding is scaled and a hashed embedding of the (previous token, token) pair is added.
Three mixers: "mingru" (an element-wise gated recurrence whose gate and candidate read only the current token),
"attention" (grouped heads with biases, a per-head norm of q and k, rotary positions, values that are rotated by their
own position and outputs that are turned back by the query's, a sliding window, sigmoid weights that are not normalised
over the keys, one output gate per head) and "latent_attention" (keys and values expanded from a cached, normed latent
row plus one rotary key part shared by the heads, interleaved rotary pairs with ramped frequency interpolation, a sliding
window, softmax). The feed-forward is a clamped gated unit. The logits are scaled.

A model is (config dict as in config.json, dict name -> tensor).
"""
import math

import torch

DT = torch.float64


def rms_norm(y, w, eps):
    return y / torch.sqrt((y * y).mean(-1, keepdim=True) + eps) * w


def silu(z):
    return z * torch.sigmoid(z)


def embed(cfg, W, tokens):
    """scaled token rows plus the row of the pair table: (prev * mul_prev + cur * mul_cur) mod buckets, the row behind the
    buckets for a sequence's first token"""
    e = cfg["embedding"]
    ids = torch.tensor(tokens, dtype=torch.long)
    x = W["embed"][ids] * e["scale"]
    bg = e.get("bigram")
    if bg:
        rows = [bg["buckets"]] + [(tokens[t - 1] * bg["mul_prev"] + tokens[t] * bg["mul_cur"]) % bg["buckets"] for t in range(1, len(tokens))]
        x = x + W["bigram"][torch.tensor(rows, dtype=torch.long)]
    return x


def pair_angles(T, n_pairs, base, span):
    """[T, n_pairs]: position * base^(-2m/span)"""
    f = torch.tensor([base ** (-2.0 * m / span) for m in range(n_pairs)], dtype=DT)
    return torch.arange(T, dtype=DT)[:, None] * f[None, :]


def turn(x, ang, layout, amp=1.0):
    """x [T, heads, n]: the first 2 * ang.shape[1] dimensions of each head turned by ang [T, pairs]; layout 'half' pairs m
    with m + pairs, 'interleaved' 2m with 2m + 1"""
    P = ang.shape[1]
    c, s = (amp * torch.cos(ang))[:, None, :], (amp * torch.sin(ang))[:, None, :]
    out = x.clone()
    if layout == "half":
        u, v = x[..., :P], x[..., P:2 * P]
        out[..., :P] = u * c - v * s
        out[..., P:2 * P] = v * c + u * s
    else:
        u, v = x[..., 0:2 * P:2], x[..., 1:2 * P:2]
        out[..., 0:2 * P:2] = u * c - v * s
        out[..., 1:2 * P:2] = v * c + u * s
    return out


def ramped_angles(T, rot):
    """([T, dims/2] angles, amplitude) of a rotation with ramped frequency interpolation (or none)"""
    d, base = rot["dims"], rot["base"]
    f = [base ** (-2.0 * i / d) for i in range(d // 2)]
    amp = 1.0
    sc = rot.get("scaling")
    if sc:
        def index_of(turns):
            return d * math.log(sc["original"] / (2 * math.pi * turns)) / (2 * math.log(base))
        lo = max(math.floor(index_of(sc["fast"])), 0)
        hi = min(math.ceil(index_of(sc["slow"])), d - 1)
        g = []
        for i, fi in enumerate(f):
            r = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
            g.append(fi / sc["factor"] * r + fi * (1 - r))
        f = g
        amp = 0.1 * math.log(sc["factor"]) + 1.0
    return torch.arange(T, dtype=DT)[:, None] * torch.tensor(f, dtype=DT)[None, :], amp


def window_mask(T, size):
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    ok = j <= i
    if size:
        ok = ok & (i - j < size)
    return ok


def mingru(h, W, pre):
    """S_t = (1 - z_t) S_(t-1) + z_t c_t from S = 0; out = W_o (S_t * silu(W_g h_t))"""
    z = torch.sigmoid(h @ W[pre + "z"].T + W[pre + "z.b"])
    u = h @ W[pre + "x"].T + W[pre + "x.b"]
    cand = torch.where(u >= 0, u + 0.5, torch.sigmoid(u))
    S = torch.zeros(z.shape[1], dtype=DT)
    states = []
    for t in range(h.shape[0]):
        S = (1 - z[t]) * S + z[t] * cand[t]
        states.append(S)
    return (torch.stack(states) * silu(h @ W[pre + "g"].T)) @ W[pre + "o"].T


def sigmoid_attention(h, mx, W, pre, eps):
    T = h.shape[0]
    H, G, d, dv = mx["heads"], mx.get("kv_heads", mx["heads"]), mx["dim"], mx["vdim"]
    q = (h @ W[pre + "q"].T + W[pre + "q.b"]).view(T, H, d)
    k = (h @ W[pre + "k"].T + W[pre + "k.b"]).view(T, G, d)
    v = (h @ W[pre + "v"].T + W[pre + "v.b"]).view(T, G, dv)
    q = rms_norm(q, W[pre + "q.norm"], eps)
    k = rms_norm(k, W[pre + "k.norm"], eps)
    rot = mx.get("rot")
    if rot and rot.get("dims"):
        ang = pair_angles(T, rot["dims"] // 2, rot["base"], rot["dims"])
        q, k = turn(q, ang, "half"), turn(k, ang, "half")
    base = rot["base"] if rot else 10000.0
    vang = pair_angles(T, dv // 2, base, dv)
    v = turn(v, vang, "half")
    ok = window_mask(T, (mx.get("mask") or {}).get("size", 0))
    out = torch.zeros(T, H, dv, dtype=DT)
    for hd in range(H):
        g = hd // (H // G)
        s = (q[:, hd] @ k[:, g].T) * mx["scale"] + W[pre + "pb"][hd]
        p = torch.where(ok, torch.sigmoid(s), torch.zeros((), dtype=DT))
        out[:, hd] = p @ v[:, g]
    out = turn(out, -vang, "half")
    gate = torch.sigmoid(h @ W[pre + "g"].T)          # [T, H]
    out = out * gate[:, :, None]
    return out.reshape(T, H * dv) @ W[pre + "o"].T + W[pre + "o.b"]


def latent_attention(h, mx, W, pre, eps):
    T = h.shape[0]
    H, d, dr, dv, R = mx["heads"], mx["dim"], mx["rot_dim"], mx["vdim"], mx["kv_rank"]
    q = (h @ W[pre + "q"].T).view(T, H, d + dr)
    ckv = h @ W[pre + "dkv"].T
    c = rms_norm(ckv[:, :R], W[pre + "dkv.norm"], eps)
    kr = ckv[:, R:].view(T, 1, dr)
    ang, amp = ramped_angles(T, mx["rot"])
    qr = turn(q[..., d:].contiguous(), ang, "interleaved", amp)
    kr = turn(kr, ang, "interleaved", amp)
    kn = (c @ W[pre + "uk"].T).view(T, H, d)
    v = (c @ W[pre + "uv"].T).view(T, H, dv)
    ok = window_mask(T, (mx.get("mask") or {}).get("size", 0))
    out = torch.zeros(T, H, dv, dtype=DT)
    for hd in range(H):
        s = (q[:, hd, :d] @ kn[:, hd].T + qr[:, hd] @ kr[:, 0].T) * mx["scale"]
        s = s.masked_fill(~ok, float("-inf"))
        out[:, hd] = torch.softmax(s, -1) @ v[:, hd]
    return out.reshape(T, H * dv) @ W[pre + "o"].T


def clamped_glu(h, ml, W, pre):
    lim = ml["limit"]
    g = torch.clamp(h @ W[pre + "gate"].T, max=lim)
    u = torch.clamp(h @ W[pre + "up"].T, -lim, lim)
    return (g * torch.sigmoid(1.702 * g) * (u + 1)) @ W[pre + "down"].T


def forward(cfg, W, tokens, keep_layers=False):
    eps = cfg["norm"]["eps"]
    x = embed(cfg, W, tokens)
    kept = []
    for i, lj in enumerate(cfg["layers"]):
        pre = "l%d." % i
        mx = lj["mixer"]
        if lj["type"] == "mingru":
            y = mingru(x, W, pre + "mix.")
        elif lj["type"] == "attention":
            y = sigmoid_attention(x, mx, W, pre + "mix.", eps)
        else:
            y = latent_attention(x, mx, W, pre + "mix.", eps)
        x = x + rms_norm(y, W[pre + "norm1"], eps)
        if lj.get("mlp"):
            x = x + rms_norm(clamped_glu(x, lj["mlp"], W, pre + "mlp."), W[pre + "norm2"], eps)
        if keep_layers:
            kept.append(x.clone())
    logits = rms_norm(x, W["final.norm"], eps) @ W["head"].T * cfg.get("logit_scale", 1.0)
    return (logits, torch.stack(kept)) if keep_layers else logits


class Oracle:
    def __init__(self, cfg, w):
        self.cfg, self.w = cfg, w

    def forward(self, tokens, return_layers=False):
        return forward(self.cfg, self.w, tokens, keep_layers=return_layers)


# ---------------------------------------------------------------------------------------------------------------
# small random models for the tests (weights rounded to bfloat16, as a checkpoint stores them)
# ---------------------------------------------------------------------------------------------------------------
def random_model(seed, width, vocab, layers, buckets=53, mul_prev=7, mul_cur=3, embed_scale=None, logit_scale=0.5, eps=1e-5):
    """layers: dicts with type 'mingru' (width) | 'attention' (heads, kv_heads, dim, vdim, optionally rot_dims, base, scale,
    window, pb) | 'latent_attention' (heads, dim, rot_dim, vdim, kv_rank, optionally base, scale, window, scaling);
    ff = None | (ff, limit)."""
    g = torch.Generator().manual_seed(seed)

    def rnd(*shape, s=None):
        return (torch.randn(*shape, generator=g) * (s if s is not None else 1.0 / math.sqrt(shape[-1]))).to(torch.bfloat16).to(DT)

    cfg = dict(architecture="Sakevik", vocab=vocab, width=width, norm=dict(eps=eps), logit_scale=logit_scale,
               embedding=dict(scale=embed_scale if embed_scale is not None else math.sqrt(width)), layers=[])
    w = {"embed": rnd(vocab, width, s=1.0 / math.sqrt(width)), "head": rnd(vocab, width), "final.norm": 1 + rnd(width, s=0.1)}
    if buckets:
        cfg["embedding"]["bigram"] = dict(buckets=buckets, mul_prev=mul_prev, mul_cur=mul_cur)
        w["bigram"] = rnd(buckets + 1, width, s=0.5)
    for i, sp in enumerate(layers):
        pre = "l%d." % i
        mp = pre + "mix."
        w[pre + "norm1"] = 1 + rnd(width, s=0.1)
        if sp["type"] == "mingru":
            C = sp["width"]
            mx = dict(width=C)
            w[mp + "z"], w[mp + "x"], w[mp + "g"], w[mp + "o"] = rnd(C, width, s=2.0 / math.sqrt(width)), rnd(C, width, s=2.0 / math.sqrt(width)), rnd(C, width), rnd(width, C)
            w[mp + "z.b"], w[mp + "x.b"] = rnd(C, s=1.0), rnd(C, s=0.5)
        elif sp["type"] == "attention":
            H, G, d, dv = sp["heads"], sp["kv_heads"], sp["dim"], sp["vdim"]
            mx = dict(heads=H, kv_heads=G, dim=d, vdim=dv, scale=sp.get("scale", 1.0 / math.sqrt(d)))
            rd = sp.get("rot_dims", d)
            mx["rot"] = dict(base=sp.get("base", 10000.0), dims=rd)
            if sp.get("window"):
                mx["mask"] = dict(size=sp["window"])
            for nm, rows in (("q", H * d), ("k", G * d), ("v", G * dv)):
                w[mp + nm], w[mp + nm + ".b"] = rnd(rows, width), rnd(rows, s=0.3)
            w[mp + "q.norm"], w[mp + "k.norm"] = 1 + rnd(d, s=0.2), 1 + rnd(d, s=0.2)
            w[mp + "pb"] = torch.full((H,), float(sp.get("pb", -2.0)), dtype=DT) + rnd(H, s=0.5)
            w[mp + "g"], w[mp + "o"], w[mp + "o.b"] = rnd(H, width), rnd(width, H * dv), rnd(width, s=0.3)
        else:
            H, d, dr, dv, R = sp["heads"], sp["dim"], sp["rot_dim"], sp["vdim"], sp["kv_rank"]
            mx = dict(heads=H, dim=d, rot_dim=dr, vdim=dv, kv_rank=R, scale=sp.get("scale", 1.0 / math.sqrt(d + dr)),
                      rot=dict(base=sp.get("base", 10000.0), dims=dr))
            if sp.get("scaling"):
                mx["rot"]["scaling"] = dict(sp["scaling"])
            if sp.get("window"):
                mx["mask"] = dict(size=sp["window"])
            w[mp + "q"], w[mp + "dkv"], w[mp + "dkv.norm"] = rnd(H * (d + dr), width, s=2.0 / math.sqrt(width)), rnd(R + dr, width), 1 + rnd(R, s=0.2)
            w[mp + "uk"], w[mp + "uv"], w[mp + "o"] = rnd(H * d, R, s=2.0 / math.sqrt(R)), rnd(H * dv, R), rnd(width, H * dv)
        ff = sp.get("ff")
        if ff is None:
            ml = None
        else:
            f, lim = ff
            ml = dict(kind="dense", ff=f, limit=lim)
            w[pre + "norm2"] = 1 + rnd(width, s=0.1)
            w[pre + "mlp.gate"], w[pre + "mlp.up"], w[pre + "mlp.down"] = rnd(f, width, s=2.0 / math.sqrt(width)), rnd(f, width, s=2.0 / math.sqrt(width)), rnd(width, f)
        cfg["layers"].append(dict(type=sp["type"], mixer=mx, mlp=ml))
    return cfg, {k: v.to(torch.bfloat16).to(DT) for k, v in w.items()}     # weights around one are sums: rounded once more


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

"""ctypes plumbing for ``include/b200_serve.h``: the model-family layer (registry, step function, paged sequence
cache, continuous-batching scheduler) and the kernels it brings. Tests and the bench call the library through this
module; the product path is the C ABI itself and ``bin/b200_serve``."""
import ctypes as C

import numpy as np

from . import capi

F32, BF16 = 0, 2
GG_NONE, GG_SIGMOID_MUL, GG_GLU, GG_GLU_GELU, GG_RELU2, GG_BIAS_SOFTPLUS, GG_GLU_CLAMP = 0, 1, 2, 3, 4, 5, 6
ROPE_HALF, ROPE_INTERLEAVED = 0, 1
_vp, _i, _f, _sz, _ll = C.c_void_p, C.c_int, C.c_float, C.c_size_t, C.c_longlong


class GemmGroupedArgs(C.Structure):
    """mirror of ``b200_gemm_grouped_args``"""
    _fields_ = [("A", _vp), ("W", _vp), ("C", _vp), ("aux", _vp), ("a_rows", _vp), ("group_off", _vp),
                ("lda", _ll), ("ldw", _ll), ("ldc", _ll), ("ld_aux", _ll),
                ("stride_a", _ll), ("stride_w", _ll), ("stride_c", _ll), ("stride_aux", _ll),
                ("M", _i), ("N", _i), ("K", _i), ("batch", _i), ("trans_b", _i), ("epi", _i),
                ("a_dtype", _i), ("w_dtype", _i), ("c_dtype", _i), ("epi_param", _f)]


class QkPrepareArgs(C.Structure):
    """mirror of ``b200_qk_prepare_args``"""
    _fields_ = [("proj", _vp), ("ld_proj", _ll), ("conv_w", _vp), ("taps", _i), ("conv_state", _vp),
                ("q_norm", _vp), ("k_norm", _vp), ("eps", _f), ("cos", _vp), ("sin", _vp), ("rot_dims", _i), ("rot_layout", _i),
                ("q_out", _vp), ("k_pool", _vp), ("v_pool", _vp), ("v_from_conv", _i),
                ("pages", _vp), ("max_pages", _i), ("page_rows", _i), ("slot", _vp), ("pos", _vp), ("start", _vp),
                ("n_tokens", _i), ("heads", _i), ("kv_heads", _i), ("dim", _i), ("dtype", _i), ("update_state_inline", _i),
                ("v_heads", _i), ("vdim", _i), ("v_off", _ll),
                ("bias", _vp), ("v_cos", _vp), ("v_sin", _vp), ("v_rot_layout", _i)]


class PagedAttentionArgs(C.Structure):
    """mirror of ``b200_paged_attention_args``"""
    _fields_ = [("q", _vp), ("out", _vp), ("k_pool", _vp), ("v_pool", _vp), ("pages", _vp), ("max_pages", _i), ("page_rows", _i),
                ("slot", _vp), ("pos", _vp), ("n_tokens", _i), ("heads", _i), ("kv_heads", _i), ("dim", _i), ("vdim", _i),
                ("scale", _f), ("softcap", _f), ("denom_bias", _f), ("dtype", _i), ("longest_entry", _i),
                ("longest_context", _i), ("workspace", _vp), ("workspace_bytes", _sz),
                ("chunk", _i), ("maps", _i), ("out_f32", _i),
                ("window", _i), ("sigmoid_weights", _i), ("head_bias", _vp)]


class RmsnormResidualArgs(C.Structure):
    """mirror of ``b200_rmsnorm_residual_args``"""
    _fields_ = [("x", _vp), ("y1", _vp), ("s1", _f), ("y2", _vp), ("s2", _f),
                ("expert_out", _vp), ("dest", _vp), ("weight", _vp), ("top", _i), ("bcast", _vp), ("rows", _vp),
                ("w", _vp), ("w_offset", _f), ("eps", _f), ("out", _vp), ("out_dtype", _i), ("n_rows", _i), ("width", _i),
                ("norm_addend", _i), ("y_bias", _vp)]


class ConvActArgs(C.Structure):
    """mirror of ``b200_conv_act_args``"""
    _fields_ = [("u", _vp), ("ld_u", _ll), ("w", _vp), ("bias", _vp), ("taps", _i), ("conv_state", _vp),
                ("out32", _vp), ("out", _vp), ("out_dtype", _i), ("slot", _vp), ("pos", _vp), ("start", _vp),
                ("n_tokens", _i), ("channels", _i), ("update_state_inline", _i)]


class SelectiveScanArgs(C.Structure):
    """mirror of ``b200_selective_scan_args``"""
    _fields_ = [("x", _vp), ("dt_raw", _vp), ("dt_bias", _vp), ("B", _vp), ("C", _vp), ("ld_bc", _ll), ("z", _vp), ("ld_z", _ll),
                ("A", _vp), ("D", _vp), ("state", _vp), ("out", _vp), ("out_dtype", _i),
                ("ent_row", _vp), ("ent_len", _vp), ("slot", _vp), ("pos", _vp),
                ("n_entries", _i), ("n_tokens", _i), ("channels", _i), ("n_state", _i), ("longest_entry", _i),
                ("workspace", _vp), ("workspace_bytes", _sz), ("dt_ready", _i)]


class RetentionArgs(C.Structure):
    """mirror of ``b200_retention_args``"""
    _fields_ = [("proj", _vp), ("ld_proj", _ll), ("q_off", _i), ("k_off", _i), ("v_off", _i),
                ("cos", _vp), ("sin", _vp), ("rot_dims", _i), ("rot_layout", _i), ("decay", _vp), ("k_scale", _f),
                ("state", _vp), ("out", _vp), ("ent_row", _vp), ("ent_len", _vp), ("slot", _vp), ("pos", _vp),
                ("n_entries", _i), ("n_tokens", _i), ("heads", _i), ("dim", _i), ("vdim", _i), ("longest_entry", _i),
                ("workspace", _vp), ("workspace_bytes", _sz)]


class LatentAttentionArgs(C.Structure):
    """mirror of ``b200_latent_attention_args``"""
    _fields_ = [("qa", _vp), ("out", _vp), ("pool", _vp), ("pages", _vp), ("max_pages", _i), ("page_rows", _i),
                ("slot", _vp), ("pos", _vp), ("sink", _vp), ("scale", _f), ("n_tokens", _i), ("heads", _i), ("rank", _i),
                ("window", _i), ("dtype", _i), ("longest_entry", _i), ("longest_context", _i),
                ("workspace", _vp), ("workspace_bytes", _sz), ("out_cols", _i)]


class GatedRecurrenceArgs(C.Structure):
    """mirror of ``b200_gated_recurrence_args``"""
    _fields_ = [("pre", _vp), ("ld_pre", _ll), ("z_off", _i), ("u_off", _i), ("g_off", _i), ("z_bias", _vp), ("u_bias", _vp),
                ("state", _vp), ("out", _vp), ("out_dtype", _i), ("ent_row", _vp), ("ent_len", _vp), ("slot", _vp), ("pos", _vp),
                ("n_entries", _i), ("n_tokens", _i), ("channels", _i), ("longest_entry", _i),
                ("workspace", _vp), ("workspace_bytes", _sz)]


class ModelOptions(C.Structure):
    """mirror of ``b200_model_options``"""
    _fields_ = [("dtype", _i), ("max_tokens", _i), ("max_slots", _i), ("max_step_tokens", _i)]


_ip = C.POINTER(C.c_int)
SERVE_PROTOTYPES = {
    "b200_embed_positions": (_i, [_vp, _vp, _vp, _vp, _vp, _i, _i, _i, _vp]),
    "b200_layernorm_pair": (_i, [_vp, _vp, _i, _i, _f, _vp, _vp, _vp, _vp, _vp, _vp, _i, _vp]),
    "b200_gemm_grouped": (_i, [C.POINTER(GemmGroupedArgs), _vp]),
    "b200_linear_ex_workspace_bytes": (_sz, [_i, _i, _i]),
    "b200_linear_ex": (_i, [_vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _vp, _sz, _vp]),
    "b200_latent_store": (_i, [_vp, _ll, _vp, _f, _vp, _vp, _i, _i, _vp, _vp, _i, _i, _i, _vp]),
    "b200_latent_attention_workspace_bytes": (_sz, [_i, _i, _i]),
    "b200_latent_attention": (_i, [_vp, _vp, _vp, _vp, _i, _i, _vp, _vp, _vp, _f, _i, _i, _i, _i, _i, _i, _vp, _sz, _vp]),
    "b200_moe_route": (_i, [_vp, _i, _vp, _vp, _i, _i, _i, _i, _f, _vp, _vp, _vp]),
    "b200_moe_dispatch": (_i, [_vp, _i, _i, _i, _vp, _vp, _vp, _vp]),
    "b200_residual_combine": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _vp]),
    "b200_layernorm_residual": (_i, [_vp, _vp, _i, _i, _f, _f, _vp, _vp, _vp, _vp, _vp, _i, _vp]),
    "b200_concat_cast": (_i, [_vp, _vp, _vp, _i, _i, _i, _vp]),
    "b200_softcap": (_i, [_vp, _sz, _f, _vp]),
    "b200_glu_act": (_i, [_vp, _vp, _i, _i, _i, _i, _vp]),
    "b200_rope_angles": (_i, [_vp, _i, _vp, _i, _vp, _vp, _vp]),
    "b200_qk_prepare": (_i, [C.POINTER(QkPrepareArgs), _vp]),
    "b200_conv_state_update": (_i, [_vp, _ll, _vp, _vp, _vp, _vp, _i, _i, _i, _vp]),
    "b200_paged_attention_workspace_bytes": (_sz, [_i, _i, _i]),
    "b200_paged_attention": (_i, [C.POINTER(PagedAttentionArgs), _vp]),
    "b200_retention_workspace_bytes": (_sz, [_i, _i, _i, _i, _i]),
    "b200_retention": (_i, [C.POINTER(RetentionArgs), _vp]),
    "b200_unit_rms_gate": (_i, [_vp, _vp, _ll, _vp, _i, _i, _i, _f, _i, _vp]),
    "b200_gather_rows": (_i, [_vp, _vp, _vp, _i, _i, _i, _vp]),
    "b200_moe_route_logits": (_i, [_vp, _i, _vp, _vp, _i, _i, _i, _i, _vp, _vp, _vp]),
    "b200_rmsnorm_residual": (_i, [C.POINTER(RmsnormResidualArgs), _vp]),
    "b200_rope_angles_amp": (_i, [_vp, _i, _vp, _i, C.c_double, _vp, _vp, _vp]),
    "b200_diff_combine": (_i, [_vp, _f, _f, _f, _vp, _i, _i, _i, _i, _vp]),
    "b200_sigmoid_gate": (_i, [_vp, _vp, _ll, _vp, _i, _i, _i, _vp]),
    "b200_conv_act": (_i, [C.POINTER(ConvActArgs), _vp]),
    "b200_selective_scan_workspace_bytes": (_sz, [_i, _i, _i, _i]),
    "b200_selective_scan": (_i, [C.POINTER(SelectiveScanArgs), _vp]),
    "b200_linear_ex2": (_i, [_vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _f, _vp, _sz, _vp]),
    "b200_latent_attention_ex": (_i, [C.POINTER(LatentAttentionArgs), _vp]),
    "b200_latent_store_rot": (_i, [_vp, _ll, _vp, _f, _vp, _vp, _i, _i, _vp, _vp, _i, _i, _i, _vp, _vp, _i, _i, _vp]),
    "b200_rotate_part": (_i, [_vp, _ll, _ll, _ll, _vp, _ll, _ll, _ll, _vp, _vp, _i, _i, _i, _i, _vp]),
    "b200_unrotate_gate": (_i, [_vp, _vp, _vp, _i, _vp, _ll, _vp, _i, _i, _i, _i, _vp]),
    "b200_gated_recurrence_workspace_bytes": (_sz, [_i, _i, _i]),
    "b200_gated_recurrence": (_i, [C.POINTER(GatedRecurrenceArgs), _vp]),
    "b200_embed_pair_hash": (_i, [_vp, _vp, _vp, _f, _vp, _i, _i, _i, _vp, _vp, _i, _i, _i, _vp]),
    "b200_scale": (_i, [_vp, _sz, _f, _vp]),
    "b200_glu_act_clamped": (_i, [_vp, _vp, _i, _i, _f, _i, _vp]),
    "b200_serve_last_error": (C.c_char_p, []),
    "b200_model_families": (C.c_char_p, []),
    "b200_model_open": (_vp, [C.c_char_p, C.POINTER(ModelOptions)]),
    "b200_model_close": (None, [_vp]),
    "b200_model_family": (C.c_char_p, [_vp]),
    "b200_model_vocab": (_i, [_vp]),
    "b200_model_width": (_i, [_vp]),
    "b200_model_layer_count": (_i, [_vp]),
    "b200_model_max_positions": (_i, [_vp]),
    "b200_model_page_rows": (_i, [_vp]),
    "b200_model_pages_total": (_i, [_vp]),
    "b200_model_pages_free": (_i, [_vp]),
    "b200_model_slot_length": (_i, [_vp, _i]),
    "b200_model_slot_pages": (_i, [_vp, _i, _vp, _i]),
    "b200_model_step": (_i, [_vp, _i, _vp, _vp, _vp, _vp, _vp, _vp, _vp]),
    "b200_model_release": (_i, [_vp, _i]),
    "b200_model_capture_layers": (_i, [_vp, _i]),
    "b200_model_captured_layers": (_i, [_vp, _vp, _sz]),
    "b200_model_step_launches": (_i, [_vp]),
    "b200_model_generate": (_i, [_vp, _i, _vp, _vp, _i, _i, _i, _vp, _vp]),
    "b200_session_create": (_vp, [_vp]),
    "b200_session_destroy": (None, [_vp]),
    "b200_session_slot": (_i, [_vp, C.c_char_p]),
    "b200_session_end": (_i, [_vp, C.c_char_p]),
}

_bound = False


def lib():
    global _bound
    handle = capi.lib()
    if not _bound:
        for name, (res, args) in SERVE_PROTOTYPES.items():
            fn = getattr(handle, name)
            fn.restype = res
            fn.argtypes = args
        _bound = True
    return handle


def last_error():
    return lib().b200_serve_last_error().decode()


def _ints(a):
    a = np.ascontiguousarray(np.asarray(a, dtype=np.int32))
    return a, a.ctypes.data_as(_vp)


class Model:
    """A checkpoint folder opened through the registry (``b200_model_open``)."""

    def __init__(self, folder, dtype=BF16, max_tokens=1024, max_slots=4):
        opt = ModelOptions(dtype, max_tokens, max_slots, 0)
        self._h = lib().b200_model_open(str(folder).encode(), C.byref(opt))
        if not self._h:
            raise RuntimeError("[b200][ERROR] model_open: " + last_error())
        L = lib()
        self.family = L.b200_model_family(self._h).decode()
        self.vocab, self.width = L.b200_model_vocab(self._h), L.b200_model_width(self._h)
        self.n_layers, self.page_rows = L.b200_model_layer_count(self._h), L.b200_model_page_rows(self._h)
        self.pages_total = L.b200_model_pages_total(self._h)

    def close(self):
        if getattr(self, "_h", None):
            lib().b200_model_close(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:   # interpreter shutdown: the module globals may be gone already
            pass

    @property
    def pages_free(self):
        return lib().b200_model_pages_free(self._h)

    def slot_length(self, slot):
        return lib().b200_model_slot_length(self._h, slot)

    def slot_pages(self, slot):
        buf = np.zeros(4096, np.int32)
        n = lib().b200_model_slot_pages(self._h, slot, buf.ctypes.data_as(_vp), len(buf))
        return buf[:n].tolist()

    def step(self, entries, logits=True, ids=False):
        """entries: list of (slot, tokens, want). Returns logits [sum want, vocab] (and greedy ids when ids=True)."""
        slots, _s = _ints([e[0] for e in entries])
        counts, _c = _ints([len(e[1]) for e in entries])
        toks, _t = _ints([t for e in entries for t in e[1]] or [0])
        nw, _nw = _ints([len(e[2]) for e in entries])
        want, _w = _ints([w for e in entries for w in e[2]] or [0])
        total = int(nw.sum())
        out = np.zeros((max(total, 1), self.vocab), np.float32)
        picks = np.zeros(max(total, 1), np.int32)
        rc = lib().b200_model_step(self._h, len(entries), _s, _c, _t, _nw, _w,
                                   out.ctypes.data_as(_vp) if logits else None, picks.ctypes.data_as(_vp) if ids else None)
        if rc != 0:
            raise RuntimeError(f"[b200][ERROR] model_step rc={rc}: {last_error()}")
        return (out[:total], picks[:total]) if ids else out[:total]

    def release(self, slot):
        return lib().b200_model_release(self._h, slot)

    def capture_layers(self, on=True):
        lib().b200_model_capture_layers(self._h, int(on))

    def captured_layers(self, n_tokens):
        out = np.zeros((self.n_layers, n_tokens, self.width), np.float32)
        rc = lib().b200_model_captured_layers(self._h, out.ctypes.data_as(_vp), out.size)
        if rc != n_tokens:
            raise RuntimeError(f"[b200][ERROR] captured_layers rc={rc}")
        return out

    @property
    def step_launches(self):
        return lib().b200_model_step_launches(self._h)

    def generate(self, prompts, max_new, eos_id=-1, chunk=0):
        ids, _p = _ints([t for p in prompts for t in p])
        lens, _l = _ints([len(p) for p in prompts])
        out = np.zeros((len(prompts), max_new), np.int32)
        made = np.zeros(len(prompts), np.int32)
        rc = lib().b200_model_generate(self._h, len(prompts), _p, _l, max_new, eos_id, chunk, out.ctypes.data_as(_vp),
                                       made.ctypes.data_as(_vp))
        if rc < 0:
            raise RuntimeError(f"[b200][ERROR] model_generate rc={rc}: {last_error()}")
        return [out[i, :made[i]].tolist() for i in range(len(prompts))], rc


def write_checkpoint(folder, config, tensors):
    """config.json + model.safetensors (bfloat16) from a dict name -> torch tensor: random-weight models for the bench
    and for trying a configuration out."""
    import json
    import os
    import struct

    import torch

    os.makedirs(folder, exist_ok=True)
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(config, f)
    header, off = {}, 0
    for name, t in tensors.items():
        n = t.numel() * 2
        header[name] = dict(dtype="BF16", shape=list(t.shape), data_offsets=[off, off + n])
        off += n
    hj = json.dumps(header).encode()
    hj += b" " * (-len(hj) % 8)
    with open(os.path.join(folder, "model.safetensors"), "wb") as f:
        f.write(struct.pack("<Q", len(hj)))
        f.write(hj)
        for t in tensors.values():
            f.write(t.to(torch.bfloat16).contiguous().view(torch.int16).numpy().tobytes())


def random_nekodra(width, heads, dim, vdim, kv_rank, experts, ff, top, identity, shared_ff, n_layers, vocab, max_positions,
                   share_every=2, seed=0):
    """(config, tensors) of a random Nekodra model; every `share_every`-th layer reads the previous layer's cached rows"""
    import math

    import torch

    g = torch.Generator().manual_seed(seed)

    def rnd(*shape, s=None):
        return (torch.randn(*shape, generator=g) * (s if s is not None else 1.0 / math.sqrt(shape[-1]))).to(torch.bfloat16)

    cfg = dict(architecture="Nekodra", vocab=vocab, width=width, max_positions=max_positions, norm=dict(eps=1e-5), layers=[])
    w = {"embed": rnd(vocab, width, s=1.0), "pos": rnd(max_positions, width, s=0.3), "head": rnd(vocab, width),
         "final.norm": torch.ones(width), "final.norm.b": torch.zeros(width)}
    for i in range(n_layers):
        pre = f"l{i}."
        mx = dict(heads=heads, dim=dim, vdim=vdim, kv_rank=kv_rank, scale=1.0 / math.sqrt(dim))
        shares = share_every > 0 and i % share_every == share_every - 1 and i > 0
        for n in ("norm1", "norm2"):
            w[pre + n], w[pre + n + ".b"] = torch.ones(width), torch.zeros(width)
        w[pre + "mix.q"], w[pre + "mix.g"] = rnd(heads * dim, width), rnd(heads * vdim, width)
        if shares:
            mx["kv_from"] = i - 1
        else:
            w[pre + "mix.dkv"], w[pre + "mix.dkv.norm"] = rnd(kv_rank, width), torch.ones(kv_rank)
        w[pre + "mix.uk"], w[pre + "mix.uv"] = rnd(heads * dim, kv_rank), rnd(heads * vdim, kv_rank)
        w[pre + "mix.sink"], w[pre + "mix.o"] = torch.zeros(heads), rnd(width, heads * vdim)
        for e in range(experts):
            w[pre + f"mlp.e{e}.gate"], w[pre + f"mlp.e{e}.up"] = rnd(ff, width), rnd(ff, width)
            w[pre + f"mlp.e{e}.down"] = rnd(width, ff)
        w[pre + "mlp.router"], w[pre + "mlp.correction"] = rnd(experts + identity, width), torch.zeros(experts + identity)
        w[pre + "mlp.shared.gate"], w[pre + "mlp.shared.up"] = rnd(shared_ff, width), rnd(shared_ff, width)
        w[pre + "mlp.shared.down"] = rnd(width, shared_ff)
        cfg["layers"].append(dict(type="latent_attention", mixer=mx,
                                  mlp=dict(kind="moe", expert=dict(ff=ff), shared=dict(ff=shared_ff),
                                           router=dict(experts=experts, identity=identity, top=top, scale=1.0))))
    return cfg, w


def random_musilorn(width, heads, kv_heads, dim, ff, n_layers, vocab, retention_every=0, ret_heads=0, ret_dim=0, ret_vdim=0,
                    conv=4, loop=None, seed=0):
    """(config, tensors) of a random Musilorn model: attention layers with a dense feed-forward; every
    `retention_every`-th layer is a retention layer without one; `loop` = (start, stop, times) or None"""
    import math

    import torch

    g = torch.Generator().manual_seed(seed)

    def rnd(*shape, s=None):
        return (torch.randn(*shape, generator=g) * (s if s is not None else 1.0 / math.sqrt(shape[-1]))).to(torch.bfloat16)

    cfg = dict(architecture="Musilorn", vocab=vocab, width=width, norm=dict(eps=1e-5), residual_mult=0.5, logit_softcap=25.0, layers=[])
    w = {"embed": rnd(vocab, width, s=1.0), "head": rnd(vocab, width), "final.norm": torch.ones(width), "final.norm.b": torch.zeros(width)}
    if loop:
        cfg["loop"] = dict(start=loop[0], stop=loop[1], times=loop[2])
        w["loop.in"] = rnd(width, 2 * width)
    for i in range(n_layers):
        pre = f"l{i}."
        retention = retention_every > 0 and i % retention_every == retention_every - 1
        for n in ("norm1", "norm1b") + (() if retention else ("norm2", "norm2b")):
            w[pre + n], w[pre + n + ".b"] = torch.ones(width), torch.zeros(width)
        if retention:
            mx = dict(heads=ret_heads, dim=ret_dim, vdim=ret_vdim, rot=dict(base=10000.0, dims=ret_dim),
                      decay=[1 - 2.0 ** (-5 - 5 * h / max(1, ret_heads - 1)) for h in range(ret_heads)])
            w[pre + "mix.q"], w[pre + "mix.k"] = rnd(ret_heads * ret_dim, width), rnd(ret_heads * ret_dim, width)
            w[pre + "mix.v"], w[pre + "mix.g"] = rnd(ret_heads * ret_vdim, width), rnd(ret_heads * ret_vdim, width)
            w[pre + "mix.o"] = rnd(width, ret_heads * ret_vdim)
            cfg["layers"].append(dict(type="retention", mixer=mx, mlp=None))
            continue
        mx = dict(heads=heads, kv_heads=kv_heads, dim=dim, vdim=dim, conv=conv, scale=1.0 / math.sqrt(dim), softcap=50.0,
                  rot=dict(base=500000.0, dims=dim, scaling=dict(factor=8.0, low=1.0, high=4.0, original=8192)))
        w[pre + "mix.q"], w[pre + "mix.k"] = rnd(heads * dim, width), rnd(kv_heads * dim, width)
        w[pre + "mix.q.conv"], w[pre + "mix.k.conv"] = rnd(heads * dim, conv, s=0.5), rnd(kv_heads * dim, conv, s=0.5)
        w[pre + "mix.q.norm"], w[pre + "mix.k.norm"] = torch.ones(dim), torch.ones(dim)
        w[pre + "mix.o"] = rnd(width, heads * dim)
        w[pre + "mlp.gate"], w[pre + "mlp.up"], w[pre + "mlp.down"] = rnd(ff, width), rnd(ff, width), rnd(width, ff)
        cfg["layers"].append(dict(type="attention", mixer=mx, mlp=dict(kind="dense", ff=ff)))
    return cfg, w


def random_tomalix(width, vocab, layers, loop=None, seed=0):
    """(config, tensors) of a random Tomalix model. layers: dicts with type 'attention' (differential) | 'parallel' |
    'attention_2', heads, kv_heads, dim, vdim, optionally chunk (parallel) and the scan's inner, state, dt_rank, conv;
    ff = None | int (dense) | (ff, experts, top); `loop` = (start, stop, times) or None"""
    import math

    import torch

    g = torch.Generator().manual_seed(seed)

    def rnd(*shape, s=None):
        return (torch.randn(*shape, generator=g) * (s if s is not None else 1.0 / math.sqrt(shape[-1]))).to(torch.bfloat16)

    cfg = dict(architecture="Tomalix", vocab=vocab, width=width, norm=dict(eps=1e-5), logit_softcap=30.0, layers=[])
    w = {"embed": rnd(vocab, width, s=1.0), "head": rnd(vocab, width), "final.norm": torch.zeros(width)}
    if loop:
        cfg["loop"] = dict(start=loop[0], stop=loop[1], times=loop[2])
        w["loop.step"] = rnd(loop[2], width, s=0.1)
    for i, sp in enumerate(layers):
        pre = f"l{i}."
        H, G, d, dv = sp["heads"], sp["kv_heads"], sp["dim"], sp["vdim"]
        kind = sp["type"]
        maps = 2 if kind == "attention" else 1
        ap = pre + ("mix.left." if kind == "parallel" else "mix.")
        att = dict(heads=H, kv_heads=G, dim=d, vdim=dv, scale=1.0 / math.sqrt(d), rot=dict(base=500000.0, dims=d))
        w[ap + "q"], w[ap + "k"], w[ap + "v"] = rnd(H * maps * d, width), rnd(G * maps * d, width), rnd(G * dv, width)
        w[ap + "o"] = rnd(width, H * dv)
        w[pre + "norm1"] = torch.zeros(width)
        if kind == "parallel":
            w[ap + "g"] = rnd(H * dv, width)
            if sp.get("chunk"):
                att["mask"] = dict(size=sp["chunk"])
            C_, N, R, taps = sp["inner"], sp["state"], sp["dt_rank"], sp["conv"]
            rp = pre + "mix.right."
            w[rp + "in"], w[rp + "conv"], w[rp + "conv.b"] = rnd(2 * C_, width), rnd(C_, taps, s=0.5), torch.zeros(C_)
            w[rp + "x"], w[rp + "dt"] = rnd(R + 2 * N, C_), rnd(C_, R)
            w[rp + "dt.b"] = torch.full((C_,), -3.0)
            w[rp + "A_log"] = torch.log(torch.arange(1, N + 1, dtype=torch.float32)).repeat(C_, 1)
            w[rp + "D"], w[rp + "o"] = torch.ones(C_), rnd(width, C_)
            mx = dict(left=att, right=dict(inner=C_, state=N, dt_rank=R, conv=taps), left_scale=1.0, right_scale=1.0)
        else:
            mx = att
            if kind == "attention":
                mx["diff"] = 0.3
                mx["rot"]["scaling"] = dict(factor=4.0)
                for nm in ("lq1", "lk1", "lq2", "lk2"):
                    w[pre + "mix." + nm] = rnd(d, s=0.1)
            else:
                mx["rot"]["scaling"] = dict(factor=8.0, original=8192, fast=32.0, slow=1.0)
        ff = sp.get("ff")
        if ff is None:
            ml = None
        else:
            w[pre + "norm2"] = torch.zeros(width)
            if isinstance(ff, int):
                ml = dict(kind="dense", ff=ff)
                w[pre + "mlp.up"], w[pre + "mlp.down"] = rnd(ff, width), rnd(width, ff)
            else:
                f, E, top = ff
                ml = dict(kind="moe", expert=dict(ff=f), router=dict(experts=E, top=top))
                for e in range(E):
                    w[pre + f"mlp.e{e}.up"], w[pre + f"mlp.e{e}.down"] = rnd(f, width), rnd(width, f)
                w[pre + "mlp.router"], w[pre + "mlp.router.b"] = rnd(E, width), torch.zeros(E)
        cfg["layers"].append(dict(type=kind, mixer=mx, mlp=ml))
    return cfg, w


def random_sakevik(width, vocab, layers, buckets=65521, seed=0):
    """(config, tensors) of a random Sakevik model. layers: dicts with type 'mingru' (width) | 'attention' (heads, kv_heads,
    dim, vdim, window) | 'latent_attention' (heads, dim, rot_dim, vdim, kv_rank, window); ff = None | (ff, limit)"""
    import math

    import torch

    g = torch.Generator().manual_seed(seed)

    def rnd(*shape, s=None):
        return (torch.randn(*shape, generator=g) * (s if s is not None else 1.0 / math.sqrt(shape[-1]))).to(torch.bfloat16)

    cfg = dict(architecture="Sakevik", vocab=vocab, width=width, norm=dict(eps=1e-6), logit_scale=0.5,
               embedding=dict(scale=math.sqrt(width), bigram=dict(buckets=buckets, mul_prev=31, mul_cur=17)), layers=[])
    w = {"embed": rnd(vocab, width), "bigram": rnd(buckets + 1, width, s=0.5), "head": rnd(vocab, width), "final.norm": torch.ones(width)}
    for i, sp in enumerate(layers):
        pre, mp = f"l{i}.", f"l{i}.mix."
        w[pre + "norm1"] = torch.ones(width)
        if sp["type"] == "mingru":
            C_ = sp["width"]
            mx = dict(width=C_)
            w[mp + "z"], w[mp + "x"], w[mp + "g"], w[mp + "o"] = rnd(C_, width), rnd(C_, width), rnd(C_, width), rnd(width, C_)
            w[mp + "z.b"], w[mp + "x.b"] = torch.zeros(C_), torch.zeros(C_)
        elif sp["type"] == "attention":
            H, G, d, dv = sp["heads"], sp["kv_heads"], sp["dim"], sp["vdim"]
            mx = dict(heads=H, kv_heads=G, dim=d, vdim=dv, scale=1.0 / math.sqrt(d), rot=dict(base=10000.0, dims=d))
            if sp.get("window"):
                mx["mask"] = dict(size=sp["window"])
            for nm, rows in (("q", H * d), ("k", G * d), ("v", G * dv)):
                w[mp + nm], w[mp + nm + ".b"] = rnd(rows, width), torch.zeros(rows)
            w[mp + "q.norm"], w[mp + "k.norm"], w[mp + "pb"] = torch.ones(d), torch.ones(d), torch.full((H,), -4.0)
            w[mp + "g"], w[mp + "o"], w[mp + "o.b"] = rnd(H, width), rnd(width, H * dv), torch.zeros(width)
        else:
            H, d, dr, dv, R = sp["heads"], sp["dim"], sp["rot_dim"], sp["vdim"], sp["kv_rank"]
            mx = dict(heads=H, dim=d, rot_dim=dr, vdim=dv, kv_rank=R, scale=1.0 / math.sqrt(d + dr),
                      rot=dict(base=500000.0, dims=dr, scaling=dict(factor=8.0, original=8192, fast=32.0, slow=1.0)))
            if sp.get("window"):
                mx["mask"] = dict(size=sp["window"])
            w[mp + "q"], w[mp + "dkv"], w[mp + "dkv.norm"] = rnd(H * (d + dr), width), rnd(R + dr, width), torch.ones(R)
            w[mp + "uk"], w[mp + "uv"], w[mp + "o"] = rnd(H * d, R), rnd(H * dv, R), rnd(width, H * dv)
        ff = sp.get("ff")
        if ff is None:
            ml = None
        else:
            f, lim = ff
            ml = dict(kind="dense", ff=f, limit=lim)
            w[pre + "norm2"] = torch.ones(width)
            w[pre + "mlp.gate"], w[pre + "mlp.up"], w[pre + "mlp.down"] = rnd(f, width), rnd(f, width), rnd(width, f)
        cfg["layers"].append(dict(type=sp["type"], mixer=mx, mlp=ml))
    return cfg, w

"""Python front end of the layer-list host (``libpegainfer_qwen3_host.so``, csrc/host/layered_host.cpp): ctypes mirrors of its
configuration structs and the model surface every design served by it shares -- build from a checkpoint folder or a tensor
dict, allocate requests, run ``step`` over a ragged batch (portions of prompts beside single decoded tokens), greedy
``generate``.  Compute runs in the sm_100a kernels behind the C ABI; there is no fallback path.
"""
from __future__ import annotations

import ctypes as C
import json
import os

import torch

from . import ffi
from .model import host_lib


# ---------------------------------------------------------------- host binding
class LayerCfg(C.Structure):
    _fields_ = [(n, C.c_int) for n in ("heads", "dim", "rot_dim", "vdim", "kv_rank", "kv_from", "rot_dims")] + \
               [("rot_base", C.c_float), ("scale", C.c_float), ("has_scaling", C.c_int)] + \
               [(n, C.c_float) for n in ("s_factor", "s_original", "s_fast", "s_slow")] + \
               [(n, C.c_int) for n in ("mlp_kind", "ff", "experts", "top", "groups", "keep")] + \
               [("route_scale", C.c_float), ("expert_ff", C.c_int), ("shared_ff", C.c_int)] + \
               [(n, C.c_int) for n in ("mixer_kind", "kv_heads", "chunk", "conv", "rot_interleaved")] + [("gate_cap", C.c_float)] + \
               [(n, C.c_int) for n in ("router_kind", "expert_act", "window")] + [("softcap", C.c_float), ("slope_log2", C.c_float)] + \
               [(n, C.c_int) for n in ("value_norm", "sink_kind", "out_gate", "proj_bias", "keep_first", "qk_norm")] + \
               [("q_temp_coef", C.c_float)] + \
               [(n, C.c_int) for n in ("q_temp_every", "values_are_keys", "scaling_kind", "ssm_heads", "ssm_vdim", "ssm_state", "ssm_groups",
                                       "ssm_norm_groups")] + \
               [(n, C.c_float) for n in ("act_limit", "act_slope", "shared_limit")] + [("weights_of", C.c_int)]


class ModelCfg(C.Structure):
    _fields_ = [("vocab", C.c_int), ("width", C.c_int), ("n_layers", C.c_int), ("eps", C.c_float)] + \
               [(n, C.c_int) for n in ("f32", "page_size", "num_pages", "max_requests", "device", "enable_pdl", "block_kind")] + \
               [("embed_scale", C.c_float), ("logit_scale", C.c_float), ("norm_groups", C.c_int), ("residual_mult", C.c_float),
                ("gated_residual", C.c_int), ("logit_softcap", C.c_float)]


def typed_host():
    h = host_lib()
    if getattr(h, "_pv_typed", False):
        return h
    vp, i32 = C.c_void_p, C.c_int
    h.pv_create_error.restype = C.c_char_p
    h.pv_create.restype = vp
    h.pv_create.argtypes = [C.POINTER(ModelCfg), C.POINTER(LayerCfg), C.c_char_p]
    h.pv_destroy.argtypes = [vp]
    h.pv_last_error.restype = C.c_char_p
    h.pv_last_error.argtypes = [vp]
    h.pv_load_tensor.argtypes = [vp, C.c_char_p, vp, i32, i32, i32]
    h.pv_finalize.argtypes = [vp]
    h.pv_request_alloc.argtypes = [vp]
    h.pv_request_free.argtypes = [vp, i32]
    h.pv_seq_len.argtypes = [vp, i32]
    h.pv_available_pages.argtypes = [vp]
    h.pv_page_size.argtypes = [vp]
    h.pv_request_pages.argtypes = [vp, i32, vp, i32]
    h.pv_step.argtypes = [vp, i32, vp, vp, vp, i32, vp, i32, vp, vp]
    h.pv_keep_trail.argtypes = [vp, i32]
    h.pv_use_graph.argtypes = [vp, i32]
    h.pv_graph_count.argtypes = [vp]
    h.pv_copy_trail.argtypes = [vp, vp]
    h.pv_launch_count.restype = C.c_int64
    h.pv_launch_count.argtypes = [vp, i32]
    h.pv_generate.argtypes = [vp, vp, i32, i32, vp, vp, vp]
    h._pv_typed = True
    return h


PAGE_SIZE = 16


def pages_for(max_tokens: int, page_size: int = PAGE_SIZE) -> int:
    """Pool pages for ``max_tokens`` live tokens (every request's share already rounded up to whole pages by the caller)."""
    return (int(max_tokens) + page_size - 1) // page_size


class LayeredModel:
    """A decoder served by the layer-list host.  A design subclasses it with its configuration class (``config_class`` with
    ``from_dict``), its checkpoint naming (``weight_shapes``) and the mapping of its configuration onto the host's structs
    (``layer_struct`` / ``model_struct``)."""
    architecture = ""
    config_class = None

    @staticmethod
    def weight_shapes(cfg) -> dict:
        raise NotImplementedError

    @staticmethod
    def layer_struct(layer) -> "LayerCfg":
        raise NotImplementedError

    @staticmethod
    def model_struct(cfg, mc: "ModelCfg") -> "ModelCfg":
        return mc

    def __init__(self, cfg, weights, dtype: torch.dtype = torch.bfloat16, max_tokens: int = 0, max_requests: int = 4,
                 device_ordinal: int = 0, enable_pdl: bool = True, kernel_lib: str | None = None):
        """``weights``: dict or iterable of (checkpoint name, tensor).  ``dtype``: bfloat16 (serving precision) or float32 (every
        product in true fp32).  ``max_tokens``: cache pool size in tokens, 0 = a share of free memory."""
        if not torch.cuda.is_available():
            raise RuntimeError("pegainfer_b200 needs a CUDA device (there is no CPU path)")
        if dtype not in (torch.bfloat16, torch.float32):
            raise ValueError("dtype must be torch.bfloat16 or torch.float32")
        self.cfg, self.dtype, self._h = cfg, dtype, typed_host()
        f32 = int(dtype == torch.float32)
        lcs = (LayerCfg * len(cfg.layers))()
        for i, l in enumerate(cfg.layers):
            lcs[i] = self.layer_struct(l)
        mc = self.model_struct(cfg, ModelCfg(vocab=cfg.vocab, width=cfg.width, n_layers=len(cfg.layers), eps=cfg.eps, f32=f32, page_size=PAGE_SIZE,
                                             num_pages=pages_for(max_tokens) if max_tokens > 0 else 0, max_requests=max_requests, device=device_ordinal,
                                             enable_pdl=int(enable_pdl), block_kind=0, embed_scale=1.0, logit_scale=1.0, norm_groups=1,
                                             residual_mult=1.0, gated_residual=0, logit_softcap=0.0))
        torch.cuda.set_device(device_ordinal)
        self._m = self._h.pv_create(C.byref(mc), lcs, (kernel_lib or ffi.KERNEL_LIB_PATH).encode())
        if not self._m:
            raise RuntimeError("pv_create: " + self._h.pv_create_error().decode())
        shapes = self.weight_shapes(cfg)
        seen = set()
        for name, t in (weights.items() if isinstance(weights, dict) else weights):
            if name not in shapes:  # nothing in the configuration uses it: leave it out, loudly
                import warnings
                warnings.warn(f"{name}: not a tensor of this configuration, ignored")
                continue
            if tuple(t.shape) != tuple(shapes[name]):
                raise ValueError(f"{name}: shape {tuple(t.shape)} != {tuple(shapes[name])} from the configuration")
            if t.is_cuda:
                torch.cuda.current_stream().synchronize()
            t = t.to(dtype).contiguous()
            rows, cols = (t.shape[0], t.shape[1]) if t.dim() == 2 else (1, t.numel())
            self._ck(self._h.pv_load_tensor(self._m, name.encode(), t.data_ptr(), rows, cols, f32))
            seen.add(name)
        missing = [n for n in shapes if n not in seen]
        if missing:
            raise KeyError(f"checkpoint misses {missing[:4]}{' ...' if len(missing) > 4 else ''}")
        self._ck(self._h.pv_finalize(self._m))

    @classmethod
    def from_pretrained(cls, model_path: str, **kw):
        """``config.json`` + ``model.safetensors`` (or a sharded index) of a checkpoint of this design."""
        from safetensors import safe_open
        from .weights import load_shard_info
        with open(os.path.join(model_path, "config.json")) as f:
            cfg = cls.config_class.from_dict(json.load(f), os.path.basename(os.path.normpath(model_path)) or "custom")
        files, _ = load_shard_info(model_path)

        def tensors():
            for p in files:
                with safe_open(p, framework="pt", device="cpu") as h:
                    for name in h.keys():
                        yield name, h.get_tensor(name)
        return cls(cfg, tensors(), **kw)

    def _ck(self, rc):
        if rc != 0:
            raise RuntimeError(self._h.pv_last_error(self._m).decode())

    def close(self):
        if getattr(self, "_m", None):
            self._h.pv_destroy(self._m)
            self._m = None

    __del__ = close

    # -- request state
    def alloc_request(self) -> int:
        rid = self._h.pv_request_alloc(self._m)
        if rid < 0:
            raise RuntimeError(self._h.pv_last_error(self._m).decode())
        return rid

    def drop_request(self, rid: int) -> None:
        self._h.pv_request_free(self._m, rid)

    def seq_len(self, rid: int) -> int:
        return self._h.pv_seq_len(self._m, rid)

    def available_pages(self) -> int:
        return self._h.pv_available_pages(self._m)

    def request_pages(self, rid: int) -> list[int]:
        buf = (C.c_int * 65536)()
        n = self._h.pv_request_pages(self._m, rid, buf, 65536)
        return list(buf[:max(n, 0)])

    # -- one engine step
    def step(self, entries, want=None, sample: bool = False, logits: bool = True):
        """``entries``: [(request id, [token, ...]), ...] -- each request's next tokens (a portion of its prompt or one decoded
        token); all entries run as one batch.  ``want``: per entry the offsets inside its tokens whose logits are wanted
        (default: the last one).  Returns fp32 logits [rows, vocab] on the host in entry order (and greedy tokens with ``sample``);
        ``logits=False`` leaves the logits on the device and returns ``None`` in their place (a generation loop needs the tokens only)."""
        n = len(entries)
        flat, lens, rids, rows, base = [], [], [], [], 0
        for i, (rid, toks) in enumerate(entries):
            w = [len(toks) - 1] if want is None else want[i]
            rows += [base + int(k) for k in w]
            flat += [int(t) for t in toks]
            lens.append(len(toks))
            rids.append(int(rid))
            base += len(toks)
        out = torch.empty((len(rows), self.cfg.vocab), dtype=torch.float32) if logits else None
        sampled = (C.c_int * max(len(rows), 1))()
        self._ck(self._h.pv_step(self._m, n, (C.c_int * len(flat))(*flat), (C.c_int * n)(*lens), (C.c_int * n)(*rids), len(rows),
                                 (C.c_int * max(len(rows), 1))(*rows), int(sample), out.data_ptr() if logits and len(rows) else None, sampled))
        return (out, list(sampled)[:len(rows)]) if sample else out

    def generate(self, prompt: list[int], max_tokens: int):
        """Greedy generation of one request: (tokens, ttft_ms, step_ms[])."""
        out = (C.c_int * max_tokens)()
        ttft = C.c_double()
        steps = (C.c_double * max(1, max_tokens - 1))()
        self._ck(self._h.pv_generate(self._m, (C.c_int * len(prompt))(*prompt), len(prompt), max_tokens, out, C.byref(ttft), steps))
        return list(out), ttft.value, list(steps)[:max_tokens - 1]

    # -- bring-up aid: residual stream after every layer of the last step, [layers, tokens, width]
    def keep_trail(self, on: bool = True) -> None:
        self._h.pv_keep_trail(self._m, int(on))

    def trail(self, tokens: int) -> torch.Tensor:
        out = torch.empty((len(self.cfg.layers), tokens, self.cfg.width), dtype=torch.float32)
        self._ck(self._h.pv_copy_trail(self._m, out.data_ptr()))
        return out

    def use_graph(self, on: bool = True) -> None:
        """Decode steps (one token per entry) replay a captured launch sequence from their second occurrence on; off = always eager."""
        self._h.pv_use_graph(self._m, int(on))

    def graph_count(self) -> int:
        return int(self._h.pv_graph_count(self._m))

    def launch_count(self, reset: bool = False) -> int:
        return int(self._h.pv_launch_count(self._m, int(reset)))

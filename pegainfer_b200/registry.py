"""Model registry: which class serves a checkpoint folder, decided from its ``config.json``.

A checkpoint names its design either with the key ``architecture`` (a string) or, as HF checkpoints do, with
``architectures`` (a list) / ``model_type``.  ``load_model`` builds the model with that class's own loader.
"""
from __future__ import annotations

import json
import os

import torch

DTYPES = {"bfloat16": torch.bfloat16, "float32": torch.float32}


def _load_vamadra(path, dtype, max_tokens, max_requests, **kw):
    from .vamadra import VamadraModel
    return VamadraModel.from_pretrained(path, dtype=dtype, max_tokens=max_tokens, max_requests=max_requests, **kw)


def _load_risolorn(path, dtype, max_tokens, max_requests, **kw):
    from .risolorn import RisolornModel
    return RisolornModel.from_pretrained(path, dtype=dtype, max_tokens=max_tokens, max_requests=max_requests, **kw)


def _load_nagosun(path, dtype, max_tokens, max_requests, **kw):
    from .nagosun import NagosunModel
    return NagosunModel.from_pretrained(path, dtype=dtype, max_tokens=max_tokens, max_requests=max_requests, **kw)


def _load_goguzen(path, dtype, max_tokens, max_requests, **kw):
    from .goguzen import GoguzenModel
    return GoguzenModel.from_pretrained(path, dtype=dtype, max_tokens=max_tokens, max_requests=max_requests, **kw)


def _load_qwen3(path, dtype, max_tokens, max_requests, **kw):
    from .config import PAGE_SIZE
    from .model import ModelRuntimeConfig, Qwen3Model
    if dtype != torch.bfloat16:
        raise ValueError("the Qwen3 path computes in bfloat16 only")
    rt = ModelRuntimeConfig(num_pages=(max_tokens + PAGE_SIZE - 1) // PAGE_SIZE + 1 if max_tokens > 0 else 0, max_batch=max_requests, **kw)
    return Qwen3Model.from_safetensors(path, rt)


# design name (as a checkpoint spells it) -> loader
ARCHITECTURES = {
    "Vamadra": _load_vamadra,
    "Risolorn": _load_risolorn,
    "Nagosun": _load_nagosun,
    "Goguzen": _load_goguzen,
    "Qwen3ForCausalLM": _load_qwen3,
    "qwen3": _load_qwen3,
}
# designs whose kernels run with every product in fp32 as well
FLOAT32_CAPABLE = {"Vamadra", "Risolorn", "Nagosun", "Goguzen"}


def architecture_of(model_path: str) -> str:
    with open(os.path.join(model_path, "config.json")) as f:
        raw = json.load(f)
    names = [raw.get("architecture")] + list(raw.get("architectures") or []) + [raw.get("model_type")]
    for n in names:
        if n in ARCHITECTURES:
            return n
    raise KeyError(f"no model class for {[n for n in names if n]} (known: {sorted(ARCHITECTURES)})")


def load_model(model_path: str, dtype: str | torch.dtype = "bfloat16", max_tokens: int = 0, max_requests: int = 4, **kw):
    """Build the model class that ``config.json`` names.  ``max_tokens``: size of the cache pool in tokens (0: a share of free memory)."""
    dt = DTYPES[dtype] if isinstance(dtype, str) else dtype
    return ARCHITECTURES[architecture_of(model_path)](model_path, dt, max_tokens, max_requests, **kw)

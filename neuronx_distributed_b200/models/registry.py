"""Model registry for serving: ``config.json`` of a model directory names the family (``architecture`` for the framework's own
checkpoint layouts, ``model_type`` for Hugging Face ones) and the family's loader returns a ready serving model — an object with
``context_encoding`` / ``token_generation`` / ``generate`` (and, for models that keep per-sequence state in slots,
``forward_step`` / ``logits`` / ``states``)."""
from __future__ import annotations

import json
import os
from typing import Any, Callable, Dict

import torch

_LOADERS: Dict[str, Callable[..., Any]] = {}


def register_family(name: str, loader: Callable[..., Any]) -> None:
    _LOADERS[name.lower()] = loader


def family_of(config: Dict[str, Any]) -> str:
    name = config.get("architecture") or config.get("model_type") or ""
    if not name and config.get("architectures"):
        name = str(config["architectures"][0]).replace("ForCausalLM", "")
    return str(name).lower()


def families():
    return sorted(_LOADERS)


def load_for_serving(model_dir: str, dtype: torch.dtype = torch.bfloat16, device=None, max_seq_len: int = 2048, batch_size: int = 1, **kw):
    with open(os.path.join(model_dir, "config.json")) as f:
        fam = family_of(json.load(f))
    if fam not in _LOADERS:
        raise ValueError(f"no serving model registered for {fam!r} (known: {', '.join(families())})")
    return _LOADERS[fam](model_dir, dtype=dtype, device=device, max_seq_len=max_seq_len, batch_size=batch_size, **kw)


def _load_naguzen(model_dir, dtype, device, max_seq_len, batch_size, **kw):
    from .naguzen import NaguzenForInference

    return NaguzenForInference.from_pretrained(model_dir, dtype=dtype, device=device, max_seq_len=max_seq_len, batch_size=batch_size, **kw)


def _load_pinirax(model_dir, dtype, device, max_seq_len, batch_size, **kw):
    from .pinirax import PiniraxForInference

    return PiniraxForInference.from_pretrained(model_dir, dtype=dtype, device=device, max_seq_len=max_seq_len, batch_size=batch_size, **kw)


def _load_pulenex(model_dir, dtype, device, max_seq_len, batch_size, **kw):
    from .pulenex import PulenexForInference

    return PulenexForInference.from_pretrained(model_dir, dtype=dtype, device=device, max_seq_len=max_seq_len, batch_size=batch_size, **kw)


def _load_noresun(model_dir, dtype, device, max_seq_len, batch_size, **kw):
    from .noresun import NoresunForInference

    return NoresunForInference.from_pretrained(model_dir, dtype=dtype, device=device, max_seq_len=max_seq_len, batch_size=batch_size, **kw)


def _load_hf_decoder(model_dir, dtype, device, max_seq_len, batch_size, **kw):
    """Llama / Mistral / Mixtral / DBRX checkpoints (model-parallel state must be initialised by the caller)."""
    from . import hf_compat
    from .llama_inference import LlamaForInference

    cfg = hf_compat.config_from_hf(model_dir, dtype=dtype, device=device, max_position_embeddings=max_seq_len)
    lm_cls = None
    if hasattr(cfg, "num_local_experts"):
        from .mixtral import MixtralForCausalLM as lm_cls
    model = LlamaForInference(cfg, batch_size=batch_size, max_seq_len=max_seq_len, lm_cls=lm_cls, **kw).eval()
    hf_compat.load_hf_checkpoint(model, model_dir)
    return model


register_family("naguzen", _load_naguzen)
register_family("pinirax", _load_pinirax)
register_family("pulenex", _load_pulenex)
register_family("noresun", _load_noresun)
for _name in ("llama", "mistral", "qwen2", "mixtral", "dbrx"):
    register_family(_name, _load_hf_decoder)

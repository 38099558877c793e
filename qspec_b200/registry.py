"""Model registry: the architecture named in a checkpoint folder's config.json selects the model class.

`load_model(path)` reads `config.json`, looks the architecture up (`"architecture"`, or the first entry of the
Hugging Face style `"architectures"` list) and calls the registered loader. New designs register a loader with
`register`; the scheduler (`scheduler.Scheduler`) serves whatever the loader returns.
"""
from __future__ import annotations

import json
import os
from typing import Callable, Dict

_LOADERS: Dict[str, Callable] = {}
SEQUENCE_DESIGNS = ("Mutusun", "Pitudra", "Repepel", "Kinanex")      # served by the sequence-mixer library alone, bfloat16 / float32
_DTYPES = {"bfloat16": "bfloat16", "bf16": "bfloat16", "float32": "float32", "fp32": "float32", "float16": "float16", "fp16": "float16"}


def register(architecture: str, loader: Callable) -> None:
    """loader(path, config_dict, dtype_name, device, **kw) -> model"""
    _LOADERS[architecture] = loader


def architectures():
    return sorted(_LOADERS)


def read_config(path: str) -> dict:
    with open(os.path.join(path, "config.json")) as f:
        return json.load(f)


def architecture_of(cfg: dict) -> str:
    arch = cfg.get("architecture") or (cfg.get("architectures") or [None])[0]
    if not arch:
        raise ValueError("config.json names no architecture")
    return arch


def supports_dtype(architecture: str, dtype: str) -> bool:
    dtype = _DTYPES.get(dtype, dtype)
    if architecture in SEQUENCE_DESIGNS:
        return dtype in ("bfloat16", "float32")
    return dtype == "float16"          # the int4 decoders run float16 activations only


def load_model(path: str, dtype: str = None, device="cuda", **kw):
    cfg = read_config(path)
    arch = architecture_of(cfg)
    if arch not in _LOADERS:
        raise ValueError(f"unknown architecture {arch!r}; known: {', '.join(architectures())}")
    return _LOADERS[arch](path, cfg, _DTYPES.get(dtype, dtype), device, **kw)


def _load_mutusun(path, cfg, dtype, device, n_slots: int = 8, max_step_tokens: int = 2048, **_):
    import torch
    from .mutusun import MutusunModel
    dt = {"bfloat16": torch.bfloat16, "float32": torch.float32, None: torch.bfloat16}.get(dtype)
    if dt is None:
        raise ValueError(f"Mutusun runs in bfloat16 or float32, not {dtype}")
    return MutusunModel.from_pretrained(path, dtype=dt, device=device, n_slots=n_slots, max_step_tokens=max_step_tokens)


def _load_pitudra(path, cfg, dtype, device, n_slots: int = 8, max_step_tokens: int = 2048, max_seq_tokens=None, **_):
    import torch
    from .pitudra import PitudraModel
    dt = {"bfloat16": torch.bfloat16, "float32": torch.float32, None: torch.bfloat16}.get(dtype)
    if dt is None:
        raise ValueError(f"Pitudra runs in bfloat16 or float32, not {dtype}")
    return PitudraModel.from_pretrained(path, dtype=dt, device=device, n_slots=n_slots, max_step_tokens=max_step_tokens,
                                        max_seq_tokens=max_seq_tokens)


def _load_repepel(path, cfg, dtype, device, n_slots: int = 8, max_step_tokens: int = 2048, max_seq_tokens=None, **_):
    import torch
    from .repepel import RepepelModel
    dt = {"bfloat16": torch.bfloat16, "float32": torch.float32, None: torch.bfloat16}.get(dtype)
    if dt is None:
        raise ValueError(f"Repepel runs in bfloat16 or float32, not {dtype}")
    return RepepelModel.from_pretrained(path, dtype=dt, device=device, n_slots=n_slots, max_step_tokens=max_step_tokens,
                                        max_seq_tokens=max_seq_tokens)


def _load_kinanex(path, cfg, dtype, device, n_slots: int = 8, max_step_tokens: int = 2048, max_seq_tokens=None, **_):
    import torch
    from .kinanex import KinanexModel
    dt = {"bfloat16": torch.bfloat16, "float32": torch.float32, None: torch.bfloat16}.get(dtype)
    if dt is None:
        raise ValueError(f"Kinanex runs in bfloat16 or float32, not {dtype}")
    return KinanexModel.from_pretrained(path, dtype=dt, device=device, n_slots=n_slots, max_step_tokens=max_step_tokens,
                                        max_seq_tokens=max_seq_tokens)


def _load_qspec_llama(path, cfg, dtype, device, n_slots: int = 8, max_step_tokens: int = 256, **_):
    """The int4 dual-mode decoder (Llama-3 / Qwen2.5 shapes) from a Hugging Face style config.json; weights from the
    folder's QuaRot-format safetensors shards if there are any, random otherwise."""
    import glob
    from .checkpoint import load_qspec_checkpoint
    from .model import QSpecLlamaConfig, QSpecLlamaModel
    if dtype not in (None, "float16"):
        raise ValueError(f"the int4 decoders run float16 activations, not {dtype}")
    qwen = "qwen" in architecture_of(cfg).lower()
    base = QSpecLlamaConfig.qwen25_14b if qwen else QSpecLlamaConfig.llama3_8b
    heads = cfg["num_attention_heads"]
    c = base(hidden_size=cfg["hidden_size"], intermediate_size=cfg["intermediate_size"], num_attention_heads=heads,
             num_key_value_heads=cfg.get("num_key_value_heads", heads), head_dim=cfg.get("head_dim", cfg["hidden_size"] // heads),
             num_hidden_layers=cfg["num_hidden_layers"], vocab_size=cfg["vocab_size"], rms_norm_eps=cfg.get("rms_norm_eps", 1e-5),
             rope_theta=cfg.get("rope_theta", 500000.0), max_seq_len=cfg.get("max_position_embeddings", 1024))
    model = QSpecLlamaModel(c, max_batch=n_slots, max_tokens=max_step_tokens, device=device)
    if glob.glob(os.path.join(path, "*.safetensors")):
        load_qspec_checkpoint(model, path)
    return model


register("Mutusun", _load_mutusun)
register("Pitudra", _load_pitudra)
register("Repepel", _load_repepel)
register("Kinanex", _load_kinanex)
register("LlamaForCausalLM", _load_qspec_llama)
register("Qwen2ForCausalLM", _load_qspec_llama)

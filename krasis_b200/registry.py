"""Model registry: which class serves a checkpoint directory, chosen by its config.json.

A design with its own config.json layout announces itself with the key "architecture"; Hugging Face checkpoints are recognised
by "architectures" / "model_type" and go to the MoE prefill model."""
import json
import os
from typing import Callable, Dict

import torch

_REGISTRY: Dict[str, Callable] = {}
_HF_MOE = ("qwen3_next", "qwen3_5_moe", "qwen3_5_moe_text", "qwen3_moe", "deepseek_v2", "deepseek_v3")


def register(name: str, factory: Callable) -> None:
    """factory(model_dir, dtype=..., device=..., **kw) -> model"""
    _REGISTRY[name] = factory


def _vofelix(model_dir, dtype=torch.bfloat16, device=0, **kw):
    from .build import build_seq
    build_seq()                                     # only the sequence-operator library; a no-op when it is current
    from .vofelix import VofelixModel
    return VofelixModel.from_pretrained(model_dir, dtype=dtype, device=device, **kw)


def _megolorn(model_dir, dtype=torch.bfloat16, device=0, **kw):
    from .build import build_seq
    build_seq()
    from .megolorn import MegolornModel
    return MegolornModel.from_pretrained(model_dir, dtype=dtype, device=device, **kw)


def _gurozen(model_dir, dtype=torch.bfloat16, device=0, **kw):
    from .build import build_seq
    build_seq()
    from .gurozen import GurozenModel
    return GurozenModel.from_pretrained(model_dir, dtype=dtype, device=device, **kw)


def _zaronex(model_dir, dtype=torch.bfloat16, device=0, **kw):
    from .build import build_seq
    build_seq()
    from .zaronex import ZaronexModel
    return ZaronexModel.from_pretrained(model_dir, dtype=dtype, device=device, **kw)


def _hf_moe(model_dir, dtype=torch.bfloat16, device=0, **kw):
    if dtype != torch.bfloat16:
        raise ValueError("the MoE prefill models run in bfloat16 only")
    from .build import build
    build()
    from .model import KrasisModel
    return KrasisModel.from_pretrained(model_dir, device=device, **kw)


register("Vofelix", _vofelix)
register("Megolorn", _megolorn)
register("Gurozen", _gurozen)
register("Zaronex", _zaronex)
for _name in _HF_MOE:
    register(_name, _hf_moe)


def architecture_of(model_dir: str) -> str:
    raw = json.load(open(os.path.join(model_dir, "config.json")))
    if "architecture" in raw:
        return raw["architecture"]
    cfg = raw.get("text_config", raw)
    if cfg.get("model_type") in _REGISTRY:
        return cfg["model_type"]
    for a in raw.get("architectures", []):
        if a in _REGISTRY:
            return a
    raise ValueError(f"{model_dir}: no registered model for this config.json "
                     f"(architecture={raw.get('architecture')!r}, model_type={cfg.get('model_type')!r})")


def load_model(model_dir: str, dtype=torch.bfloat16, device=0, **kw):
    return _REGISTRY[architecture_of(model_dir)](model_dir, dtype=dtype, device=device, **kw)

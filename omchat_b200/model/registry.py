"""Which model class serves which configuration.

`load_model(path)` reads config.json (checkpoint.config_from_dict picks the configuration class from "model_type" /
"architecture"), looks the model class up here and loads the weights. Model modules are imported lazily: a process pays only for
the model it runs.
"""
from __future__ import annotations

import json
import os
from typing import Optional

import torch

from ..config import FofisunConfig, OmChatQwen2Config, OmChatQwen2MoeConfig, TifisunConfig, VefunexConfig, VoduzenConfig

# configuration class -> (module, class name)
MODEL_CLASSES = {
    VefunexConfig: ("omchat_b200.model.vefunex", "VefunexForCausalLM"),
    FofisunConfig: ("omchat_b200.model.fofisun", "FofisunForCausalLM"),
    TifisunConfig: ("omchat_b200.model.tifisun", "TifisunForCausalLM"),
    VoduzenConfig: ("omchat_b200.model.voduzen", "VoduzenForCausalLM"),
    OmChatQwen2MoeConfig: ("omchat_b200.model.moe", "OmChatQwen2MoeForCausalLM"),
    OmChatQwen2Config: ("omchat_b200.model.omchat", "OmChatQwen2ForCausalLM"),
}


def model_class_for(config):
    for cfg_cls, (mod, name) in MODEL_CLASSES.items():      # subclasses are listed before their bases
        if isinstance(config, cfg_cls):
            import importlib
            return getattr(importlib.import_module(mod), name)
    raise ValueError(f"no model class is registered for {type(config).__name__}")


def read_config(path: str):
    from .checkpoint import config_from_dict
    cj = os.path.join(path, "config.json") if os.path.isdir(path) else os.path.join(os.path.dirname(path), "config.json")
    with open(cj) as fh:
        return config_from_dict(json.load(fh))


def load_model(path: str, device="cuda", dtype: Optional[torch.dtype] = None):
    """The model of the checkpoint folder `path`. dtype: compute dtype for models that offer a choice (Voduzen: bfloat16 or
    float32; Tifisun, Fofisun and Vefunex likewise); the OmChat models are bfloat16 only and refuse anything else."""
    cfg = read_config(path)
    cls = model_class_for(cfg)
    if isinstance(cfg, (VoduzenConfig, TifisunConfig, FofisunConfig, VefunexConfig)):
        return cls.from_pretrained(path, config=cfg, device=device, dtype=dtype or torch.bfloat16)
    if dtype not in (None, torch.bfloat16):
        raise ValueError(f"{cls.__name__} computes in bfloat16 only")
    return cls.from_pretrained(path, config=cfg, device=device)

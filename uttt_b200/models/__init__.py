"""Model registry: ``model_type`` -> causal-LM class (the counterpart of the reference's
``AutoModelForCausalLM`` registration in uttt_llm/flame/custom_models/__init__.py:15-34)."""
from __future__ import annotations

from typing import Callable, Dict

from ..config import LMConfig, config_from_dict, load_config

_REGISTRY: Dict[str, Callable] = {}


def register_model(model_type: str):
    def deco(cls):
        _REGISTRY[model_type] = cls
        return cls
    return deco


def _populate() -> None:
    if _REGISTRY:
        return
    from .uttt_moe import UTTTMoEForCausalLM, TTTMoEForCausalLM
    _REGISTRY["uttt_moe"] = UTTTMoEForCausalLM
    _REGISTRY["ttt_moe_lb"] = TTTMoEForCausalLM
    _REGISTRY["ttt_moe_no_lb"] = TTTMoEForCausalLM
    try:
        from .uttt_dense import UTTTDenseForCausalLM, TTTDenseForCausalLM, LaCTForCausalLM
        _REGISTRY["uttt_dense"] = UTTTDenseForCausalLM
        _REGISTRY["ttt_dense"] = TTTDenseForCausalLM
        _REGISTRY["lact_swiglu"] = LaCTForCausalLM
    except ImportError:
        pass
    try:
        from .baselines import TransformerForCausalLM, SWAMixerForCausalLM
        _REGISTRY["transformer"] = TransformerForCausalLM
        for name in ("deltanet_swa", "gated_deltanet_swa", "kda_swa", "mamba2_swa", "mom_swa"):
            _REGISTRY[name] = SWAMixerForCausalLM
    except ImportError:
        pass


def model_class_for(model_type: str):
    _populate()
    if model_type not in _REGISTRY:
        raise KeyError(f"no model registered for model_type {model_type!r}; known: {sorted(_REGISTRY)}")
    return _REGISTRY[model_type]


def build_model(config: LMConfig):
    """Instantiate the causal LM for a config (random init)."""
    return model_class_for(config.model_type)(config)


def registered_model_types():
    _populate()
    return sorted(_REGISTRY)

"""Architecture configs for the language models (HF-style JSON schema).

The field names and validation rules follow the reference's
``PretrainedConfig`` subclasses so that its JSON files load unchanged:

* base fields ........ uttt_llm/flame/custom_models/uttt_moe/configuration_recurrent_lact_base.py:11-240
* uTTT-MoE fields .... uttt_llm/flame/custom_models/uttt_moe/configuration_recurrent_lact.py:9-230
* uTTT-Dense fields .. uttt_llm/flame/custom_models/uttt_dense/configuration_recurrent_lact.py:28-301
* TTT-MoE fields ..... uttt_llm/flame/custom_models/ttt_moe_lb/configuration_recurrent_lact.py:12-27

The classes here are plain Python (no ``transformers`` dependency): a config is
a validated attribute bag with ``from_json`` / ``to_dict`` / ``save_pretrained``.
"""
from __future__ import annotations

import copy
import json
import os
from typing import Any, Dict, Optional, Type

_COMPOSE_MODES = {"reuse", "attn-proj", "shared", "ttt-proj"}


class LMConfig:
    """Fields shared by every recurrent fast-weight language model."""

    model_type = "uttt_base"

    _BASE_DEFAULTS: Dict[str, Any] = dict(
        hidden_size=2048,
        num_hidden_layers=24,
        num_heads=32,
        num_kv_heads=None,
        qkv_bias=False,
        qk_norm=False,
        window_size=None,
        rope_theta=10000.0,
        max_position_embeddings=2048,
        hidden_ratio=4,
        intermediate_size=None,
        hidden_act="swish",
        initializer_range=0.02,
        elementwise_affine=True,
        norm_eps=1e-6,
        use_cache=True,
        pad_token_id=None,
        bos_token_id=1,
        eos_token_id=2,
        tie_word_embeddings=False,
        fuse_norm=True,
        fuse_swiglu=True,
        fuse_cross_entropy=True,
        fuse_linear_cross_entropy=False,
        use_l2warp=False,
        vocab_size=32000,
        chunk_size=1024,
        memory_v_gap=None,
        memory_k_gap=None,
        attention_v_gap=None,
        attention_k_gap=None,
        shared_kv_cache=False,
        memory_shared_kv_cache=False,
        memory_reuse_kv_cache=False,
        memory_perlayer_k_share_v=False,
        memory_perlayer_k_reuse_v=False,
        memory_k_compose_mode=None,
        memory_v_compose_mode=None,
        use_memory_block=False,
        fw_num_heads=None,
        fw_inter_multi=2.0,
        base_lr=0.01,
        per_head_lr=False,
        repeat_function="repeat",
        w0_w2_low_rank=-1,
        fw_init_gain=0.5,
        memory_kv_mode="to_kv",
        memory_kv_feature="x_memory_in",
        memory_kv_proj="ttt_kv_proj",
        memory_qkv_silu=False,
        memory_qk_norm=False,
        memory_qk_norm_type="l2",
        memory_norm_type="rms",
        memory_v_norm=False,
        memory_qk_rescale=False,
        learnable_ttt_scale=False,
        ttt_prenorm=False,
        same_rope=False,
        last_layer_fuse_norm=True,
        ttt_rope_theta=0.0,
        use_momentum=False,
        use_moun=False,
        enable_memory_output_proj=False,
        enable_attention_output_proj=False,
        enable_attention_memory_output_proj=False,
        residual_style="parallel",
        memory_adaLN_modulation_enabled=False,
    )

    # subclasses add their own defaults here
    _EXTRA_DEFAULTS: Dict[str, Any] = {}

    def __init__(self, **kwargs: Any):
        kwargs = dict(kwargs)
        kwargs.pop("model_type", None)
        kwargs.pop("native_reference_impl", None)
        removed = [k for k in kwargs if k.endswith("_reference_impl")]
        if removed:
            raise ValueError(f"Removed config key(s): {', '.join(removed)}")
        defaults = {**self._BASE_DEFAULTS, **self._all_extra_defaults()}
        for key, default in defaults.items():
            setattr(self, key, kwargs.pop(key, copy.deepcopy(default)))
        # unknown keys (attention_bias, transformers_version, ...) are kept verbatim
        self.extra: Dict[str, Any] = kwargs
        self._validate_base()
        self._validate()

    @classmethod
    def _all_extra_defaults(cls) -> Dict[str, Any]:
        merged: Dict[str, Any] = {}
        for klass in reversed(cls.__mro__):
            merged.update(getattr(klass, "_EXTRA_DEFAULTS", {}))
        return merged

    # ------------------------------------------------------------------ derived
    @property
    def head_dim(self) -> int:
        return self.hidden_size // self.num_heads

    @property
    def kv_heads(self) -> int:
        return self.num_kv_heads if self.num_kv_heads is not None else self.num_heads

    @property
    def fw_heads(self) -> int:
        return self.fw_num_heads if self.fw_num_heads is not None else self.kv_heads

    @property
    def fw_head_dim(self) -> int:
        return self.hidden_size // self.fw_heads

    @property
    def fw_inter_dim(self) -> int:
        return int(self.fw_head_dim * self.fw_inter_multi)

    @property
    def mlp_intermediate_size(self) -> int:
        if self.intermediate_size is not None:
            return int(self.intermediate_size)
        ratio = self.hidden_ratio if self.hidden_ratio is not None else 4
        inter = int(self.hidden_size * ratio * 2 / 3)
        return 256 * ((inter + 256 - 1) // 256)

    # --------------------------------------------------------------- validation
    def _validate_base(self) -> None:
        if self.hidden_size % self.num_heads != 0:
            raise ValueError("`hidden_size` must be divisible by `num_heads`.")
        if self.num_heads % self.kv_heads != 0:
            raise ValueError("`num_heads` must be divisible by `num_kv_heads`.")
        if self.fuse_cross_entropy and self.fuse_linear_cross_entropy:
            raise ValueError(
                "`fuse_cross_entropy` and `fuse_linear_cross_entropy` cannot be True at the same time.")
        if self.memory_shared_kv_cache and self.memory_reuse_kv_cache:
            raise ValueError("`memory_shared_kv_cache` and `memory_reuse_kv_cache` cannot both be True.")
        if self.memory_perlayer_k_share_v and self.memory_perlayer_k_reuse_v:
            raise ValueError(
                "`memory_perlayer_k_share_v` and `memory_perlayer_k_reuse_v` cannot both be True.")
        perlayer = self.memory_perlayer_k_share_v or self.memory_perlayer_k_reuse_v
        if perlayer and (self.memory_reuse_kv_cache or self.memory_shared_kv_cache):
            raise ValueError("`memory_perlayer_k_*` modes are incompatible with the kv-cache sharing flags.")
        for name in ("memory_k_compose_mode", "memory_v_compose_mode"):
            mode = getattr(self, name)
            if mode is not None and mode not in _COMPOSE_MODES:
                raise ValueError(f"`{name}` must be one of {sorted(_COMPOSE_MODES)}, got {mode!r}.")
        if (self.memory_k_compose_mode is not None or self.memory_v_compose_mode is not None) and (
            self.memory_shared_kv_cache or self.memory_reuse_kv_cache or perlayer
        ):
            raise ValueError("`memory_*_compose_mode` cannot be mixed with legacy explicit memory compose flags.")
        if "ttt-proj" in (self.memory_k_compose_mode, self.memory_v_compose_mode) and (
            self.memory_kv_proj != "ttt_kv_proj"
        ):
            raise ValueError('`ttt-proj` memory compose modes require `memory_kv_proj="ttt_kv_proj"`.')
        if self.memory_kv_mode == "reuse_kv" and self.memory_k_compose_mode == "ttt-proj":
            raise ValueError('`memory_k_compose_mode="ttt-proj"` is incompatible with `memory_kv_mode="reuse_kv"`.')
        if self.residual_style not in {"parallel", "sequential"}:
            raise ValueError(f"Invalid residual_style: {self.residual_style!r}")
        if self.memory_qk_norm_type not in {"l2", "rms"} or self.memory_norm_type not in {"l2", "rms"}:
            raise ValueError("memory norm types must be 'l2' or 'rms'.")
        if self.use_memory_block:
            if self.hidden_size % self.fw_heads != 0:
                raise ValueError("`hidden_size` must be divisible by `fw_num_heads`.")
            if self.chunk_size < 1:
                raise ValueError("`chunk_size` must be positive.")

    def _validate(self) -> None:  # subclass hook
        pass

    # ------------------------------------------------------------ serialisation
    def to_dict(self) -> Dict[str, Any]:
        out = {"model_type": self.model_type}
        for key in {**self._BASE_DEFAULTS, **self._all_extra_defaults()}:
            out[key] = getattr(self, key)
        out.update(self.extra)
        return out

    def to_json_string(self) -> str:
        return json.dumps(self.to_dict(), indent=2, sort_keys=True) + "\n"

    def save_pretrained(self, path: str) -> None:
        os.makedirs(path, exist_ok=True)
        with open(os.path.join(path, "config.json"), "w") as f:
            f.write(self.to_json_string())

    @classmethod
    def from_dict(cls, data: Dict[str, Any], **overrides: Any) -> "LMConfig":
        data = {**data, **overrides}
        return cls(**data)

    def replace(self, **overrides: Any) -> "LMConfig":
        return type(self).from_dict(self.to_dict(), **overrides)

    def __repr__(self) -> str:
        return f"{type(self).__name__}({self.to_dict()})"


class UTTTMoEConfig(LMConfig):
    """uTTT-MoE: one routed pool of SwiGLU fast-weight experts shared by all layers."""

    model_type = "uttt_moe"
    _EXTRA_DEFAULTS = dict(
        memory_num_experts=1,
        memory_num_active_experts=1,
        memory_router_alpha=1.0,
        memory_router_use_sigmoid=False,
        memory_router_from_v=False,
        memory_router_share_mode="share_all",
        memory_router_type="softmax",
        memory_router_combine_mode="selected_prob",
        memory_router_scale=0.0,
        memory_router_norm_eps=1e-6,
        memory_pool_mode="shared",
        memory_lb_loss_alpha=0.0,
        memory_lb_scope="layer",
        memory_lb_mode="loss",
        memory_loss_free_update_rate=1e-4,
        memory_loss_free_bias_max=2.0,
        memory_loss_free_warmup_steps=0,
        memory_loss_free_update_interval=1,
        memory_update_backward_mode="stop_state",
        memory_detach_m_coeff=False,
        memory_update_aggregate_write=False,
        memory_aggregate_momentum_mode="none",
        memory_aggregate_lr_scale=1.0,
        memory_cross_layer_cut_vjp_group=1,
        memory_write_layers="all",
        # expert-parallel degree of the pool in this framework (1 = replicated state)
        memory_expert_parallel=1,
    )
    _POOL_MODES = {"shared"}

    def _validate(self) -> None:
        if self.memory_update_backward_mode == "first_order":
            self.memory_update_backward_mode = "stop_state"
        if self.memory_num_experts < 1:
            raise ValueError("`memory_num_experts` must be >= 1.")
        if self.memory_num_active_experts < 1:
            raise ValueError("`memory_num_active_experts` must be >= 1.")
        if self.memory_num_active_experts > self.memory_num_experts:
            raise ValueError("`memory_num_active_experts` cannot be greater than `memory_num_experts`.")
        if self.memory_pool_mode not in self._POOL_MODES:
            raise ValueError(f"`memory_pool_mode` must be one of {sorted(self._POOL_MODES)}.")
        if self.memory_router_use_sigmoid:
            raise NotImplementedError("Sigmoid routing is not implemented.")
        if self.memory_router_share_mode not in {"share_all", "per_layer"}:
            raise ValueError("`memory_router_share_mode` must be 'share_all' or 'per_layer'.")
        if self.memory_router_type not in {"softmax", "norm_softmax", "norm_relu"}:
            raise ValueError(
                f"`memory_router_type` must be 'softmax', 'norm_softmax', or 'norm_relu', got {self.memory_router_type!r}.")
        if self.memory_router_combine_mode not in {"selected_prob", "topk_renorm"}:
            raise ValueError("`memory_router_combine_mode` must be 'selected_prob' or 'topk_renorm'.")
        if self.memory_router_scale < 0:
            raise ValueError("`memory_router_scale` must be non-negative.")
        if self.memory_router_norm_eps <= 0:
            raise ValueError("`memory_router_norm_eps` must be positive.")
        if self.memory_lb_scope not in {"layer", "pool"}:
            raise ValueError("`memory_lb_scope` must be 'layer' or 'pool'.")
        if self.memory_lb_mode not in {"loss", "loss_free", "none"}:
            raise ValueError("`memory_lb_mode` must be 'loss', 'loss_free', or 'none'.")
        for name in ("memory_loss_free_update_rate", "memory_loss_free_bias_max", "memory_loss_free_warmup_steps"):
            if getattr(self, name) < 0:
                raise ValueError(f"`{name}` must be non-negative.")
        if self.memory_loss_free_update_interval < 1:
            raise ValueError("`memory_loss_free_update_interval` must be >= 1.")
        if self.memory_update_backward_mode not in {"full", "first_order_state", "stop_state", "cross_layer_cut"}:
            raise ValueError(
                "`memory_update_backward_mode` must be 'full', 'first_order_state', 'stop_state', or "
                f"'cross_layer_cut', got {self.memory_update_backward_mode!r}.")
        if self.memory_aggregate_momentum_mode not in {"none", "pool_mean"}:
            raise ValueError("`memory_aggregate_momentum_mode` must be 'none' or 'pool_mean'.")
        if self.memory_aggregate_lr_scale <= 0:
            raise ValueError("`memory_aggregate_lr_scale` must be positive.")
        group = self.memory_cross_layer_cut_vjp_group
        if isinstance(group, bool) or not isinstance(group, int) or group < 1:
            raise ValueError("`memory_cross_layer_cut_vjp_group` must be a positive integer.")
        layers = self.memory_write_layers
        if isinstance(layers, str):
            if layers not in {"all", "last"}:
                raise ValueError("`memory_write_layers` must be 'all', 'last', or a list of layer indices.")
        elif isinstance(layers, (list, tuple)):
            layers = list(layers)
            bad = any(isinstance(i, bool) or not isinstance(i, int) or i < 0 or i >= self.num_hidden_layers
                      for i in layers)
            if not layers or len(set(layers)) != len(layers) or bad:
                raise ValueError("`memory_write_layers` list must hold distinct 0-based layer indices.")
            self.memory_write_layers = sorted(layers)
        else:
            raise ValueError("`memory_write_layers` must be 'all', 'last', or a list of layer indices.")
        if self.memory_write_layers != "all":
            if not self.memory_update_aggregate_write:
                raise ValueError("`memory_write_layers` other than 'all' requires memory_update_aggregate_write=True.")
            if self.memory_update_backward_mode == "cross_layer_cut":
                raise ValueError("`memory_write_layers` other than 'all' is not supported with 'cross_layer_cut'.")
        if self.memory_update_backward_mode == "cross_layer_cut":
            if not self.memory_update_aggregate_write:
                raise ValueError("'cross_layer_cut' requires `memory_update_aggregate_write=True`.")
            if self.memory_aggregate_momentum_mode != "pool_mean":
                raise ValueError("'cross_layer_cut' requires `memory_aggregate_momentum_mode='pool_mean'`.")
            if not self.use_memory_block:
                raise ValueError("'cross_layer_cut' requires `use_memory_block=True`.")
            if self.memory_detach_m_coeff:
                raise ValueError("'cross_layer_cut' is implemented for `memory_detach_m_coeff=False` only.")
        if self.memory_update_aggregate_write:
            if self.memory_aggregate_momentum_mode == "pool_mean" and not self.use_momentum:
                raise ValueError("`memory_aggregate_momentum_mode='pool_mean'` requires `use_momentum=True`.")
            if self.memory_aggregate_momentum_mode == "none" and self.use_momentum:
                raise ValueError(
                    "`memory_aggregate_momentum_mode='none'` with `use_momentum=True` would silently drop momentum.")
        else:
            if self.memory_aggregate_momentum_mode != "none":
                raise ValueError("`memory_aggregate_momentum_mode` requires `memory_update_aggregate_write=True`.")
            if self.memory_aggregate_lr_scale != 1.0:
                raise ValueError("`memory_aggregate_lr_scale` requires `memory_update_aggregate_write=True`.")
        ep = self.memory_expert_parallel
        if not isinstance(ep, int) or ep < 1 or self.memory_num_experts % ep != 0:
            raise ValueError("`memory_expert_parallel` must divide `memory_num_experts`.")


class TTTMoEConfig(UTTTMoEConfig):
    """TTT-MoE: a routed pool per layer (layer-local ownership).

    ``ttt_moe_lb`` adds the loss-free bias to the router *logits* before the
    softmax (uttt_llm/flame/custom_models/ttt_moe_lb/modeling_recurrent_lact.py:248-249);
    ``ttt_moe_no_lb`` trains with the auxiliary loss only.
    """

    model_type = "ttt_moe_lb"
    _POOL_MODES = {"shared", "per_layer", "layer_local"}
    _EXTRA_DEFAULTS = dict(memory_pool_mode="per_layer", memory_bias_in_logits=True)


class TTTMoENoLBConfig(TTTMoEConfig):
    model_type = "ttt_moe_no_lb"
    _EXTRA_DEFAULTS = dict(memory_bias_in_logits=False, memory_lb_mode="loss")


class UTTTDenseConfig(LMConfig):
    """uTTT-Dense: one dense SwiGLU fast-weight operator ``[H, r*D, D]`` shared by all layers."""

    model_type = "uttt_dense"
    _EXTRA_DEFAULTS = dict(
        uttt_dense_r=1,
        uttt_agg_reduce="mean",
        uttt_agg_lr_scale=1.0,
        uttt_master_renorm=False,
        uttt_update_mode="aggregate",
        uttt_update_checkpoint=True,
        memory_update_backward_mode="full",
    )

    def __init__(self, **kwargs: Any):
        if "memory_aggregate_lr_scale" in kwargs:
            raise ValueError("use `uttt_agg_lr_scale`; the `memory_aggregate_lr_scale` alias is not accepted.")
        r = kwargs.get("uttt_dense_r", 1)
        if isinstance(r, bool) or not isinstance(r, (int, float)) or float(r) != int(r) or int(r) < 1:
            raise ValueError(f"`uttt_dense_r` must be a positive integer, got {r!r}.")
        r = int(r)
        if "fw_inter_multi" in kwargs and float(kwargs["fw_inter_multi"]) != float(r):
            raise ValueError("`fw_inter_multi` must exactly match `uttt_dense_r`.")
        kwargs["uttt_dense_r"] = r
        kwargs["fw_inter_multi"] = r
        super().__init__(**kwargs)

    def _validate(self) -> None:
        if self.uttt_agg_reduce not in {"mean", "sum"}:
            raise ValueError("`uttt_agg_reduce` must be 'mean' or 'sum'.")
        if self.uttt_update_mode != "aggregate":
            raise ValueError("`uttt_update_mode` supports only 'aggregate'.")
        if self.uttt_agg_lr_scale <= 0:
            raise ValueError("`uttt_agg_lr_scale` must be positive.")
        if self.use_memory_block and self.w0_w2_low_rank > 0 and self.w0_w2_low_rank > self.fw_head_dim // 2:
            raise ValueError("`w0_w2_low_rank` must be <= fw head dim / 2.")
        if self.memory_update_backward_mode not in {"full", "first_order_state", "stop_state"}:
            raise ValueError("invalid `memory_update_backward_mode` for uTTT-Dense.")


class TTTDenseConfig(LMConfig):
    """TTT-Dense: a private dense fast-weight MLP per layer (LaCT-style)."""

    model_type = "ttt_dense"
    _EXTRA_DEFAULTS = dict(memory_update_backward_mode="full")


class LaCTConfig(LMConfig):
    """Published LaCT baseline (``lact_swiglu``): layer-private, large-chunk TTT."""

    model_type = "lact_swiglu"
    _EXTRA_DEFAULTS = dict(
        num_attn_heads=None, num_lact_heads=4, inter_multi=1, lact_chunk_size=2048,
        use_muon=True, lr_dim=1, qkv_silu=True, no_v_silu=False, lr_parameterization="mamba",
        learnable_ttt_scale=True, use_momentum=True, ttt_loss_type="dot_product", ttt_prenorm=True,
        ttt_nope=False, w0_w2_low_rank=-1, use_fused_kernel=False, fp32_states=False,
        memory_update_backward_mode="full",
    )

    def _validate_base(self) -> None:
        if self.num_attn_heads is not None:
            self.num_heads = self.num_attn_heads
        self.use_memory_block = True
        self.fw_num_heads = self.num_lact_heads
        self.fw_inter_multi = self.inter_multi
        self.chunk_size = self.lact_chunk_size
        self.use_moun = bool(self.use_muon)
        self.memory_kv_mode = "reuse_kv"
        self.memory_kv_feature = "x_attn_in"
        self.memory_qkv_silu = bool(self.qkv_silu)
        self.memory_qk_norm = True
        self.memory_qk_rescale = True
        self.per_head_lr = True
        self.enable_attention_memory_output_proj = True
        self.same_rope = not self.ttt_nope
        super()._validate_base()


class TransformerConfig(LMConfig):
    """Transformer / Transformer-SWA baseline (no memory block)."""

    model_type = "transformer"
    _EXTRA_DEFAULTS = dict(enable_attention_output_proj=True)

    def _validate(self) -> None:
        self.use_memory_block = False


class SWAMixerConfig(LMConfig):
    """Bounded-state token-mixer baselines that share the sliding-window attention branch
    (uttt_llm/flame/custom_models/fla_window_mix_utils.py:68-133)."""

    model_type = "deltanet_swa"
    _EXTRA_DEFAULTS = dict(
        mixer="deltanet", expand_k=1.0, expand_v=1.0, use_gate=False, use_short_conv=True, conv_size=4,
        use_beta=True, qk_activation="silu", qk_norm_mixer="l2", state_size=64, mixer_head_dim=64,
        num_memories=4, topk_memories=2, mixer_num_heads=None, swa_mix="sum",
    )

    def _validate(self) -> None:
        self.use_memory_block = False


def _mixer_config(name: str, mixer: str) -> Type[SWAMixerConfig]:
    return type(f"{mixer.title().replace('_', '')}SWAConfig", (SWAMixerConfig,),
                {"model_type": name, "_EXTRA_DEFAULTS": {"mixer": mixer}})


GatedDeltaNetSWAConfig = _mixer_config("gated_deltanet_swa", "gated_deltanet")
KDASWAConfig = _mixer_config("kda_swa", "kda")
Mamba2SWAConfig = _mixer_config("mamba2_swa", "mamba2")
MoMSWAConfig = _mixer_config("mom_swa", "mom")


CONFIG_REGISTRY: Dict[str, Type[LMConfig]] = {
    cls.model_type: cls
    for cls in (
        UTTTMoEConfig, TTTMoEConfig, TTTMoENoLBConfig, UTTTDenseConfig, TTTDenseConfig, LaCTConfig,
        TransformerConfig, SWAMixerConfig, GatedDeltaNetSWAConfig, KDASWAConfig, Mamba2SWAConfig, MoMSWAConfig,
    )
}


def config_from_dict(data: Dict[str, Any], **overrides: Any) -> LMConfig:
    model_type = data.get("model_type")
    if model_type not in CONFIG_REGISTRY:
        raise KeyError(f"unknown model_type {model_type!r}; known: {sorted(CONFIG_REGISTRY)}")
    return CONFIG_REGISTRY[model_type].from_dict(data, **overrides)


def load_config(path: str, **overrides: Any) -> LMConfig:
    """Load ``config.json`` from a file or a directory that contains one."""
    if os.path.isdir(path):
        path = os.path.join(path, "config.json")
    with open(path) as f:
        return config_from_dict(json.load(f), **overrides)


# ---------------------------------------------------------------------------
# Named shapes used by the benchmarks and tests.
# ---------------------------------------------------------------------------
_COMMON_UTTT = dict(
    hidden_ratio=4, hidden_act="swish", norm_eps=1e-6, rope_theta=1000000, use_memory_block=True,
    base_lr=0.001, per_head_lr=True, fw_init_gain=0.5, memory_kv_mode="reuse_kv",
    memory_kv_feature="x_attn_in", memory_qkv_silu=True, memory_qk_norm=True, memory_qk_norm_type="l2",
    memory_norm_type="l2", memory_qk_rescale=True, learnable_ttt_scale=True, ttt_prenorm=True, same_rope=True,
    use_momentum=True, use_moun=True, residual_style="parallel", enable_attention_output_proj=False,
    enable_memory_output_proj=False, enable_attention_memory_output_proj=True, vocab_size=32000,
    max_position_embeddings=32768,
)


def named_config(name: str, **overrides: Any) -> LMConfig:
    """Shapes named by the benchmark definition (not the shipped JSON files).

    ``760M-uttt-moe``: 24 layers, d 1536, 16 heads, a pool of 32 experts of hidden
    1536 (4 fast-weight heads of D=384, inner multiplier 4), top-2, window/chunk 2048.
    ``124M-uttt-moe``: 12 layers, d 768, 12 heads, 16 experts of hidden 768, top-2, aux loss.
    ``124M-uttt-dense``: 12 layers, d 768, one dense operator of hidden 1536 (1 head, r=2).
    ``tiny-uttt-moe``: CPU plumbing shape (2 layers, d 64, 4 experts of hidden 128, top-1).
    """
    moe_common = dict(
        memory_router_share_mode="per_layer", memory_pool_mode="shared", memory_update_aggregate_write=True,
        memory_aggregate_momentum_mode="pool_mean", memory_update_backward_mode="full",
        memory_router_type="softmax", memory_router_combine_mode="selected_prob",
    )
    if name == "760M-uttt-moe":
        cfg = dict(_COMMON_UTTT, **moe_common, model_type="uttt_moe", hidden_size=1536, num_hidden_layers=24,
                   num_heads=16, fw_num_heads=4, fw_inter_multi=4, memory_num_experts=32,
                   memory_num_active_experts=2, window_size=2048, chunk_size=2048, w0_w2_low_rank=32,
                   memory_lb_mode="loss_free", memory_lb_scope="pool", memory_loss_free_update_rate=1e-3)
    elif name == "124M-uttt-moe":
        cfg = dict(_COMMON_UTTT, **moe_common, model_type="uttt_moe", hidden_size=768, num_hidden_layers=12,
                   num_heads=12, fw_num_heads=4, fw_inter_multi=4, memory_num_experts=16,
                   memory_num_active_experts=2, window_size=2048, chunk_size=2048, w0_w2_low_rank=32,
                   memory_lb_mode="loss", memory_lb_scope="pool", memory_lb_loss_alpha=0.01)
    elif name == "124M-uttt-dense":
        cfg = dict(_COMMON_UTTT, model_type="uttt_dense", hidden_size=768, num_hidden_layers=12, num_heads=12,
                   fw_num_heads=1, fw_inter_multi=2, uttt_dense_r=2, window_size=2048, chunk_size=2048,
                   w0_w2_low_rank=0)
    elif name == "tiny-uttt-moe":
        cfg = dict(_COMMON_UTTT, **moe_common, model_type="uttt_moe", hidden_size=64, num_hidden_layers=2,
                   num_heads=4, fw_num_heads=1, fw_inter_multi=2, memory_num_experts=4,
                   memory_num_active_experts=1, window_size=128, chunk_size=64, w0_w2_low_rank=0,
                   vocab_size=1024, max_position_embeddings=256, memory_lb_mode="loss", memory_lb_scope="pool",
                   memory_lb_loss_alpha=0.01)
    else:
        raise KeyError(f"unknown named config {name!r}")
    cfg.update(overrides)
    return config_from_dict(cfg)

"""Ops of the framework: hand-written sm_100a kernels on CUDA tensors, plain PyTorch on CPU."""
from . import reference
from ._ext import available as ext_available, load as load_ext
from .functional import (GroupPlan, TILE_ROWS, bmm, bmm_nt, build_group_plan, route_softmax_topk, route_topk, pool_step, patch_decode, grad_sink, reset_grad_sinks, fanout_linear, split_linear, linear, stacked_linear, set_fused_weight_grad, set_dense_gemm, set_strict, library_fallbacks, KernelCoverageError, fw_qk_prep, fw_write_grad, fw_write_grad_accumulate, fw_write_pointwise, gg_nn, gg_swiglu, write_stash_for, fw_write_accumulate_skips, WriteStash,
                         gg_nt, gg_tn, l2_norm, launch_count, layer_norm, linear_cross_entropy, newton_schulz,
                         permute_rows, plucker_embed, rms_norm, rms_norm_gated, add_rms_norm, embedding, rope, swa_attention, swiglu, unpermute_rows)

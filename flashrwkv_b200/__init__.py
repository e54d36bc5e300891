"""flashrwkv_b200 -- B200 (sm_100a) implementation of the RWKV-7 WKV7 time-mix operators.

The operator names, signatures and error behaviour follow the FlashRWKV2
reference (`flashrwkv2.tmix.*`, contracts in its docs/kernel_api.md); the
kernels are hand-written CUDA for sm_100a reached through the C ABI of
include/frwkv_b200.h.  There is no CPU fallback.
"""
from .rl_infctx.wkv7 import rl_infctx_chunk_fp32io16, rl_infctx_chunk_fp32io16_factor_recompute
from .tmix.wkv7 import (
    infer_chunk_bf16_forward_varlen,
    infer_recurrent_add_vec_forward_varlen,
    infer_recurrent_fp16_advance_i32,
    infer_recurrent_fp16_advance_i32_varlen,
    infer_recurrent_fp16_forward_varlen,
    infer_recurrent_fp32io16_forward_varlen,
    prepare_recurrent_metadata,
    pretrain_recurrent_bf16,
    statetune_recurrent_fp32io16,
)

from .tmix.a_gate import pretrain_tmix_a_gate_bf16
from .tmix.kk_a_gate import infer_tmix_kk_a_gate_forward_varlen
from .tmix.kk_pre import pretrain_tmix_kk_pre_bf16
from .tmix.linear import *  # noqa: F401,F403
from .tmix.linear import __all__ as _linear_all
from .tmix.lnx_rkvres_xg import infer_tmix_lnx_rkvres_xg_forward_varlen, pretrain_tmix_lnx_rkvres_xg_bf16
from .tmix.mix6 import (
    infer_tmix_mix6_add_layer_norm_forward_varlen,
    infer_tmix_mix6_forward_varlen,
    infer_tmix_shift_project_forward_varlen,
    pretrain_tmix_mix6_bf16,
    statetune_tmix_mix6_bf16,
)
from .tmix.normalization import *  # noqa: F401,F403
from .tmix.normalization import __all__ as _norm_all
from .tmix.vres_gate import infer_tmix_vres_gate_forward_varlen, pretrain_tmix_vres_gate_bf16
from .tmix.layer import TMixLayerWeights, infer_tmix_decode_layer_forward_varlen
from ._ext import check_device_error_flags, device_error_flags

__all__ = [
    "infer_tmix_kk_a_gate_forward_varlen",
    "infer_tmix_lnx_rkvres_xg_forward_varlen",
    "infer_tmix_mix6_forward_varlen",
    "infer_tmix_mix6_add_layer_norm_forward_varlen",
    *_norm_all,
    "infer_tmix_shift_project_forward_varlen",
    "infer_tmix_decode_layer_forward_varlen",
    "TMixLayerWeights",
    "device_error_flags",
    "check_device_error_flags",
    "infer_tmix_vres_gate_forward_varlen",
    *_linear_all,
    "infer_chunk_bf16_forward_varlen",
    "infer_recurrent_add_vec_forward_varlen",
    "infer_recurrent_fp16_advance_i32",
    "infer_recurrent_fp16_advance_i32_varlen",
    "infer_recurrent_fp16_forward_varlen",
    "infer_recurrent_fp32io16_forward_varlen",
    "prepare_recurrent_metadata",
    "pretrain_recurrent_bf16",
    "pretrain_tmix_a_gate_bf16",
    "pretrain_tmix_kk_pre_bf16",
    "pretrain_tmix_lnx_rkvres_xg_bf16",
    "pretrain_tmix_mix6_bf16",
    "pretrain_tmix_vres_gate_bf16",
    "statetune_recurrent_fp32io16",
    "statetune_tmix_mix6_bf16",
    "rl_infctx_chunk_fp32io16",
    "rl_infctx_chunk_fp32io16_factor_recompute",
]
__version__ = "0.1.0"

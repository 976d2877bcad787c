"""ctypes prototypes of the non-GEMM entry points of libopake_kernels.so (see csrc/kernels/opk_api.h)."""
from ctypes import POINTER, Structure, c_float, c_int32, c_int64, c_uint32, c_uint64, c_void_p

P, I, L, F = c_void_p, c_int32, c_int64, c_float


class DpStepArgs(Structure):
    _fields_ = [
        ("grad_src", POINTER(c_void_p)), ("n_src", c_int32),
        ("shard_begin", c_int64), ("shard_len", c_int64),
        ("inv_batch", c_float), ("sigma", c_float),
        ("seed", c_uint64), ("stream_id", c_uint32), ("step", c_uint32),
        ("m", c_void_p), ("v", c_void_p), ("master", c_void_p),
        ("param_dst", POINTER(c_void_p)), ("n_dst", c_int32), ("param_src", c_void_p),
        ("lr", c_float), ("beta1", c_float), ("beta2", c_float), ("eps", c_float), ("weight_decay", c_float),
        ("bc1", c_float), ("bc2", c_float), ("phi_hat", c_float), ("zero_grad", c_int32),
        ("blt_state", c_void_p), ("blt_nbuf", c_int32), ("blt_decay", c_void_p), ("blt_scale", c_void_p),
        ("sgd_mode", c_int32),
        ("toep_state", c_void_p), ("toep_nlag", c_int32), ("toep_coef", c_void_p), ("toep_pos", c_int32),
    ]


class EpGroup(Structure):
    _fields_ = [("world", c_int32), ("rank", c_int32), ("n_experts", c_int32), ("r_cap", c_int32), ("ctrl", c_void_p * 8),
                ("epoch_base", c_void_p)]


class EpPeers(Structure):
    _fields_ = [("p", c_void_p * 8)]


_G, _PE = POINTER(EpGroup), POINTER(EpPeers)

PROTOTYPES: dict = {
    "opk_ep_ctrl_ints": (I, [I, I]),
    "opk_ep_rows_capacity": (I, [I, I, I]),
    "opk_ep_count": (I, [_G, P, I, P, I, P]),
    "opk_ep_dispatch": (I, [_G, _PE, P, L, I, P, P, P, P, I, I, I, I, I, I, P, P]),
    "opk_ep_prepare": (I, [_G, I, I, P, P, P, P, P, P, P]),
    "opk_ep_zero_pad": (I, [P, P, P, I, I, P]),
    "opk_ep_scale_rows": (I, [P, P, P, I, I, P, P]),
    "opk_ep_signal": (I, [_G, I, I, P]),
    "opk_ep_advance": (I, [P, I, I, P]),
    "opk_ep_allreduce_f64": (I, [_G, _PE, P, I, I, P, P, P]),
    "opk_ep_wait": (I, [_G, I, I, P, P]),
    "opk_ep_combine": (I, [_G, _PE, P, P, I, P, I, I, P, I, I, P, P]),
    "opk_ep_combine_bwd": (I, [_PE, P, P, I, I, I, P, P]),
    "opk_rmsnorm_fwd": (I, [P, P, P, P, I, I, F, F, P]),
    "opk_rmsnorm_fwd_ld": (I, [P, L, P, P, L, P, I, I, F, F, P]),
    "opk_rmsnorm_bwd_ld": (I, [P, L, P, L, P, P, P, P, L, P, P, I, I, I, F, P]),
    "opk_add_rmsnorm_fwd": (I, [P, P, P, P, P, P, I, I, F, F, P]),
    "opk_rmsnorm_bwd": (I, [P, P, P, P, P, P, P, P, I, I, I, F, P]),
    "opk_layernorm_fwd": (I, [P, P, P, P, P, P, I, I, F, P]),
    "opk_layernorm_bwd": (I, [P, P, P, P, P, P, P, P, P, I, I, P]),
    "opk_rope": (I, [P, P, P, I, I, I, L, F, P]),
    "opk_swiglu_fwd": (I, [P, P, I, I, P]),
    "opk_swiglu_bwd": (I, [P, P, P, I, I, P]),
    "opk_geglu_fwd": (I, [P, P, I, I, I, P]),
    "opk_geglu_bwd": (I, [P, P, P, I, I, I, P]),
    "opk_gelu_fwd": (I, [P, P, L, P]),
    "opk_gelu_bwd": (I, [P, P, P, L, P]),
    "opk_embedding_fwd": (I, [P, P, P, P, I, I, I, P]),
    "opk_embedding_bwd_compact": (I, [P, P, P, P, P, P, I, I, I, P]),
    "opk_embedding_accumulate": (I, [P, P, P, P, P, I, I, P]),
    "opk_lce_finalize": (I, [P, P, P, P, P, P, I, I, P]),
    "opk_loss_coef": (I, [P, P, P, P, P, P, I, P]),
    "opk_rmsnorm_dw_per_example": (I, [P, P, P, P, I, I, I, P]),
    "opk_cross_entropy_fwd": (I, [P, I, P, P, P, I, I, L, F, F, P]),
    "opk_cross_entropy_bwd": (I, [P, I, P, P, P, P, I, I, L, F, F, P]),
    "opk_sumsq": (I, [P, I, I, L, P, P]),
    "opk_moe_route": (I, [P, L, I, I, I, I, P, P, P, P]),
    "opk_moe_route_bwd": (I, [P, P, P, I, I, I, I, P, L, P]),
    "opk_moe_rows_capacity": (I, [I, I]),
    "opk_moe_plan": (I, [P, I, I, I, P, P, P, P, P, P]),
    "opk_moe_gather": (I, [P, L, P, I, P, I, I, P, P]),
    "opk_moe_combine": (I, [P, P, P, I, P, I, I, P, P]),
    "opk_moe_combine_bwd": (I, [P, P, P, I, I, I, P, P]),
    "opk_wait_selftest": (I, [P, L, P, P]),
    "opk_clip_sum_tile": (I, []),
    "opk_clip_sum_desc_bytes": (I, []),
    "opk_clip_sumsq_partial": (I, [P, I, I, P, P]),
    "opk_clip_apply_sum": (I, [P, I, I, P, P, P, P]),
    "opk_scatter_rows_cast_sumsq": (I, [P, P, P, I, I, P, P]),
    "opk_colsum": (I, [P, P, I, I, L, P]),
    "opk_embedding_add_rows": (I, [P, P, P, P, I, I, P]),
    "opk_cast_f32_bf16": (I, [P, P, L, P]),
    "opk_clip_scale": (I, [P, F, I, F, I, L, P, P, P, I, P]),
    "opk_clip_accumulate": (I, [P, P, P, L, P]),
    "opk_clip_accumulate2": (I, [P, P, P, L, I, P]),
    "opk_clip_accumulate_group": (I, [POINTER(c_void_p), POINTER(c_void_p), I, P, L, I, P]),
    "opk_clip_accumulate_group_push": (I, [POINTER(c_void_p), POINTER(c_void_p), I, POINTER(c_void_p), POINTER(c_int64), I, I, L, P]),
    "opk_copy_bytes": (I, [P, P, L, P]),
    "opk_embedding_accumulate_shared": (I, [P, P, P, P, P, I, I, P]),
    "opk_philox_normal": (I, [P, L, c_uint64, c_uint32, c_uint32, c_uint64, F, I, P]),
    "opk_dp_step": (I, [POINTER(DpStepArgs), P]),
}

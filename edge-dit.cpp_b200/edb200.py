"""ctypes binding of libedb200.so (the C ABI declared in include/edb200_ops.h).

This module only loads the shared library and declares argument types; all
compute happens in the CUDA kernels behind the C entry points.  It fails loudly
(ImportError / RuntimeError) when the library is missing or a call returns an
error status -- there is no fallback path.
"""
from __future__ import annotations

import ctypes as C
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libedb200.so")

OK = 0
TYPE_F32, TYPE_F16, TYPE_Q8_0, TYPE_Q4_K, TYPE_I8, TYPE_BF16 = 0, 1, 8, 12, 24, 30
ACT_NONE, ACT_GELU_TANH, ACT_SILU = 0, 1, 2
SPLIT_K_NEVER, SPLIT_K_UNORDERED = 0, 1

c_i64 = C.c_int64
c_vp = C.c_void_p


class Epilogue(C.Structure):
    _fields_ = [
        ("bias", c_vp), ("act", C.c_int), ("out", c_vp), ("out_dtype", C.c_int), ("ldo", c_i64),
        ("residual", c_vp), ("ld_res", c_i64), ("gate", c_vp),
        ("split_n", c_i64), ("out2", c_vp), ("out2_dtype", C.c_int), ("ldo2", c_i64), ("act2", C.c_int),
        ("split_k", C.c_int), ("pack", c_vp),
    ]


class QkPack(C.Structure):
    """edb200_qk_pack_t: head-major destination of a QKV projection's leading q | k | v features."""
    _fields_ = [
        ("n_heads", C.c_int), ("d_head", C.c_int), ("only", C.c_int), ("q_weight", c_vp), ("k_weight", c_vp),
        ("eps", C.c_float),
        ("pe", c_vp), ("tok_off", c_i64), ("l_total", c_i64), ("q_out", c_vp), ("k_out", c_vp), ("v_out", c_vp),
        ("peers", c_vp),
    ]


class QwenConfig(C.Structure):
    """edb200_qwen_config_t"""
    _fields_ = [
        ("num_layers", C.c_int), ("num_heads", C.c_int), ("head_dim", C.c_int), ("mlp_hidden", C.c_int),
        ("in_channels", C.c_int), ("out_channels", C.c_int), ("joint_attention_dim", C.c_int), ("patch_size", C.c_int),
        ("axes_dim", C.c_int * 3), ("theta", C.c_int), ("wtype", C.c_int), ("attention", C.c_int),
        ("sage_smooth_q", C.c_int),
    ]


class SD3Config(C.Structure):
    """edb200_sd3_config_t"""
    _fields_ = [
        ("hidden_size", C.c_int), ("num_heads", C.c_int), ("depth", C.c_int), ("mlp_hidden", C.c_int),
        ("in_channels", C.c_int), ("out_channels", C.c_int), ("patch_size", C.c_int), ("adm_in_channels", C.c_int),
        ("context_size", C.c_int), ("pos_embed_max_size", C.c_int), ("wtype", C.c_int), ("attention", C.c_int),
        ("sage_smooth_q", C.c_int), ("sage_skip_first", C.c_int), ("sage_skip_last", C.c_int),
    ]


class WanConfig(C.Structure):
    """edb200_wan_config_t"""
    _fields_ = [
        ("dim", C.c_int), ("num_heads", C.c_int), ("ffn_dim", C.c_int), ("num_layers", C.c_int),
        ("in_dim", C.c_int), ("out_dim", C.c_int), ("text_dim", C.c_int), ("freq_dim", C.c_int),
        ("patch_size", C.c_int * 3), ("axes_dim", C.c_int * 3), ("theta", C.c_int),
        ("wtype", C.c_int), ("attention", C.c_int), ("sage_smooth_q", C.c_int),
        ("sage_skip_first", C.c_int), ("sage_skip_last", C.c_int),
    ]


class FluxConfig(C.Structure):
    _fields_ = [
        ("hidden_size", C.c_int), ("num_heads", C.c_int), ("depth", C.c_int), ("depth_single_blocks", C.c_int),
        ("mlp_hidden", C.c_int), ("in_channels", C.c_int), ("context_in_dim", C.c_int), ("vec_in_dim", C.c_int),
        ("patch_size", C.c_int), ("axes_dim", C.c_int * 3), ("theta", C.c_int), ("guidance_embed", C.c_int),
        ("wtype", C.c_int), ("attention", C.c_int), ("sage_smooth_q", C.c_int),
    ]


ATTN_F16, ATTN_SAGE_INT8 = 0, 1
ANCHOR_MODEL_IN, ANCHOR_MODEL_OUT = -1, -2


class EdbError(RuntimeError):
    def __init__(self, status: int, msg: str):
        super().__init__(f"edb200 status {status}: {msg}")
        self.status = status


_SIGS = {
    "edb200_last_error": (C.c_char_p, []),
    "edb200_version": (C.c_char_p, []),
    "edb200_launch_count": (c_i64, []),
    "edb200_probe_mma_rate": (C.c_int, [C.c_int, C.c_int, C.POINTER(C.c_double), c_vp]),
    "edb200_profile_begin": (C.c_int, []),
    "edb200_profile_end": (C.c_int, [C.POINTER(C.c_double), C.POINTER(C.c_double), C.POINTER(C.c_double),
                                     C.POINTER(c_i64)]),
    "edb200_dequantize_rows": (C.c_int, [C.c_int, c_vp, c_vp, c_i64, c_i64, c_vp]),
    "edb200_quantize_rows_q8_0": (C.c_int, [c_vp, c_vp, c_i64, c_i64, c_vp]),
    "edb200_fill_normal": (C.c_int, [c_vp, c_i64, C.c_uint64, C.c_float, C.c_float, c_vp]),
    "edb200_qweight_create": (C.c_int, [C.c_int, c_vp, c_i64, c_i64, c_vp, C.POINTER(c_vp)]),
    "edb200_qweight_destroy": (None, [c_vp]),
    "edb200_qweight_dequantize": (C.c_int, [c_vp, c_vp, c_vp]),
    "edb200_qweight_bytes": (c_i64, [c_vp]),
    "edb200_mul_mat_q": (C.c_int, [c_vp, c_vp, C.c_int, c_i64, c_i64, C.POINTER(Epilogue), c_vp]),
    "edb200_mul_mat_q_pair": (C.c_int, [c_vp, c_vp, c_i64, c_i64, C.POINTER(Epilogue),
                                        c_vp, c_vp, c_i64, c_i64, C.POINTER(Epilogue), C.c_int, c_vp]),
    "edb200_gemv_q": (C.c_int, [c_vp, c_vp, c_i64, c_i64, C.c_int, c_vp, c_vp, c_i64, c_vp]),
    "edb200_gemv_batch_create": (C.c_int, [C.POINTER(c_vp), C.POINTER(c_vp), C.POINTER(c_vp), C.c_int, c_vp, C.POINTER(c_vp)]),
    "edb200_gemv_batch_destroy": (None, [c_vp]),
    "edb200_gemv_batch_run": (C.c_int, [c_vp, c_vp, C.c_int, c_vp, c_vp]),
    "edb200_linear_f32": (C.c_int, [c_vp, c_vp, c_vp, c_i64, c_i64, c_i64, c_i64, C.c_int, C.c_int, c_vp, c_i64,
                                    c_vp]),
    "edb200_layernorm_modulate": (C.c_int, [c_vp, c_i64, c_vp, c_vp, c_vp, c_vp, c_i64, c_i64, C.c_float, c_vp,
                                            C.c_int, c_i64, c_vp]),
    "edb200_fused_modulate": (C.c_int, [c_vp, c_vp, c_vp, c_vp, c_i64, c_i64, c_vp]),
    "edb200_fused_residual_gate": (C.c_int, [c_vp, c_vp, c_vp, c_vp, c_i64, c_i64, c_vp]),
    "edb200_euler_update": (C.c_int, [c_vp, c_vp, C.c_float, C.c_float, c_i64, c_vp]),
    "edb200_euler_update_sched": (C.c_int, [c_vp, c_vp, c_vp, c_vp, c_i64, c_vp]),
    "edb200_flow_update": (C.c_int, [c_vp, c_vp, C.c_float, C.c_float, c_i64, c_vp]),
    "edb200_flow_update_sched": (C.c_int, [c_vp, c_vp, c_vp, c_vp, c_i64, c_vp]),
    "edb200_sub_f32": (C.c_int, [c_vp, c_vp, c_vp, c_i64, c_vp]),
    "edb200_flux_set_anchor_capture": (C.c_int, [c_vp, C.c_int, c_vp]),
    "edb200_flux_set_stop_after": (C.c_int, [c_vp, C.c_int]),
    "edb200_flux_set_stream_override": (C.c_int, [c_vp, c_vp]),
    "edb200_sd3_set_anchor_capture": (C.c_int, [c_vp, C.c_int, c_vp]),
    "edb200_sd3_set_stop_after": (C.c_int, [c_vp, C.c_int]),
    "edb200_sd3_set_stream_override": (C.c_int, [c_vp, c_vp]),
    "edb200_sd3_set_region_inject": (C.c_int, [c_vp, C.c_int, C.c_int, c_vp]),
    "edb200_wan_set_anchor_capture": (C.c_int, [c_vp, C.c_int, c_vp]),
    "edb200_wan_set_stop_after": (C.c_int, [c_vp, C.c_int]),
    "edb200_wan_set_stream_override": (C.c_int, [c_vp, c_vp]),
    "edb200_wan_set_region_inject": (C.c_int, [c_vp, C.c_int, C.c_int, c_vp]),
    "edb200_qwen_set_anchor_capture": (C.c_int, [c_vp, C.c_int, c_vp]),
    "edb200_qwen_set_stop_after": (C.c_int, [c_vp, C.c_int]),
    "edb200_qwen_set_stream_override": (C.c_int, [c_vp, c_vp]),
    "edb200_sd3_step_sched": (C.c_int, [c_vp, c_vp, c_vp, c_vp, C.c_float, c_vp, c_vp, c_vp, c_vp]),
    "edb200_qwen_step_sched": (C.c_int, [c_vp, c_vp, c_vp, c_vp, C.c_float, c_vp, c_vp, c_vp]),
    "edb200_wan_step_sched": (C.c_int, [c_vp, c_vp, c_vp, c_vp, C.c_float, c_vp, c_vp, c_vp]),
    "edb200_qk_norm_rope_pack": (C.c_int, [c_vp, C.c_int, c_i64, c_i64, c_i64, c_i64, c_i64, C.c_int, C.c_int,
                                           c_vp, c_vp, C.c_float, c_vp, c_i64, c_i64, c_vp, c_vp, c_vp, C.c_int,
                                           c_vp]),
    "edb200_cast": (C.c_int, [c_vp, C.c_int, c_vp, C.c_int, c_i64, c_vp]),
    "edb200_attention_f16": (C.c_int, [c_vp, c_vp, c_vp, C.c_int, c_i64, c_i64, C.c_int, C.c_float, c_vp, C.c_int,
                                       c_i64, c_vp]),
    "edb200_sage_scratch_bytes": (c_i64, [C.c_int, c_i64, C.c_int]),
    "edb200_sage_scratch_layout": (C.c_int, [C.c_int, c_i64, C.c_int, C.POINTER(c_i64), C.POINTER(C.c_int)]),
    "edb200_sage_quantize_qk": (C.c_int, [c_vp, c_vp, C.c_int, c_i64, C.c_int, C.c_int, c_vp, c_i64, c_vp]),
    "edb200_attention_sage_int8": (C.c_int, [c_vp, c_vp, c_vp, c_vp, C.c_int, c_vp, C.c_int, c_vp, C.c_int, C.c_int,
                                             c_i64, C.c_int, C.c_float, c_vp, C.c_int, c_i64, c_vp]),
    "edb200_sage_attention": (C.c_int, [c_vp, c_vp, c_vp, C.c_int, c_i64, C.c_int, C.c_float, C.c_int, c_vp, c_i64,
                                        c_vp, C.c_int, c_i64, c_vp]),
    "edb200_sage_key_means_static": (C.c_int, [c_vp, C.c_int, c_i64, C.c_int, c_vp, c_vp]),
    "edb200_sp_shard": (C.c_int, [c_i64, c_i64, C.c_int, C.c_int, C.POINTER(c_i64), C.POINTER(c_i64), C.POINTER(c_i64),
                                  C.POINTER(c_i64)]),
    "edb200_poll_status": (C.c_int, [c_vp]),
    "edb200_comm_create_loopback": (C.c_int, [C.c_int, C.c_int, C.POINTER(c_vp)]),
    "edb200_comm_set_timeout_ms": (C.c_int, [c_vp, c_i64]),
    "edb200_comm_all_ok": (C.c_int, [c_vp, C.c_int, C.c_int]),
    "edb200_cfg_parallel_combine_rescaled": (C.c_int, [c_vp, c_vp, C.c_float, C.c_int, C.c_int, C.c_int, C.c_int, c_vp,
                                                       c_vp, c_vp]),
    "edb200_attention_f16_strided": (C.c_int, [c_vp, c_vp, c_vp, C.c_int, c_i64, c_i64, c_i64, c_i64, C.c_int, C.c_float,
                                               c_vp, C.c_int, c_i64, c_vp, c_vp]),
    "edb200_sage_quantize_qk_strided": (C.c_int, [c_vp, c_vp, C.c_int, c_i64, c_i64, C.c_int, C.c_int, c_vp, c_i64, c_vp]),
    "edb200_attention_sage_int8_strided": (C.c_int, [c_vp, c_vp, c_vp, c_i64, c_vp, C.c_int, c_vp, C.c_int, c_vp, C.c_int,
                                                     C.c_int, c_i64, C.c_int, C.c_float, c_vp, C.c_int, c_i64, c_vp,
                                                     c_vp]),
    "edb200_sage_attention_strided": (C.c_int, [c_vp, c_vp, c_vp, C.c_int, c_i64, c_i64, C.c_int, C.c_float, C.c_int,
                                                c_vp, c_i64, c_vp, C.c_int, c_i64, c_vp, c_vp]),
    "edb200_sd3_set_comm": (C.c_int, [c_vp, c_vp]),
    "edb200_flux_get_tensor_f32": (C.c_int, [c_vp, C.c_char_p, c_vp, c_i64, C.c_int, c_vp]),
    "edb200_sd3_get_tensor_f32": (C.c_int, [c_vp, C.c_char_p, c_vp, c_i64, C.c_int, c_vp]),
    "edb200_qwen_get_tensor_f32": (C.c_int, [c_vp, C.c_char_p, c_vp, c_i64, C.c_int, c_vp]),
    "edb200_wan_get_tensor_f32": (C.c_int, [c_vp, C.c_char_p, c_vp, c_i64, C.c_int, c_vp]),
    "edb200_sp_heads_plan": (C.c_int, [C.c_int, C.c_int, C.c_int, c_i64, c_i64, C.POINTER(C.c_int), C.POINTER(c_i64),
                                       C.POINTER(c_i64), C.POINTER(c_i64), C.c_int]),
    "edb200_comm_unique_id": (C.c_int, [c_vp]),
    "edb200_comm_create": (C.c_int, [c_vp, C.c_int, C.c_int, C.POINTER(c_vp)]),
    "edb200_comm_destroy": (None, [c_vp]),
    "edb200_comm_rank": (C.c_int, [c_vp]),
    "edb200_comm_world": (C.c_int, [c_vp]),
    "edb200_sp_all_to_all_heads": (C.c_int, [c_vp, C.POINTER(c_vp), C.POINTER(c_vp), C.c_int, C.c_int, c_i64, c_i64,
                                             c_vp]),
    "edb200_sp_all_to_all_tokens": (C.c_int, [c_vp, c_vp, c_vp, c_vp, c_i64, c_i64, c_i64, c_vp]),
    "edb200_sp_all_gather_rows": (C.c_int, [c_vp, c_vp, c_vp, C.POINTER(c_i64), C.POINTER(c_i64), c_i64, c_vp]),
    "edb200_sp_all_gather_rows_peer": (C.c_int, [c_vp, c_vp, c_vp, C.POINTER(c_i64), C.POINTER(c_i64), c_i64, c_vp]),
    "edb200_comm_map_peers": (C.c_int, [c_vp, c_vp, c_i64, c_i64, c_vp]),
    "edb200_comm_unmap_peers": (C.c_int, [c_vp]),
    "edb200_comm_peers_mapped": (C.c_int, [c_vp]),
    "edb200_comm_peer_ptr": (c_vp, [c_vp, C.c_int, c_vp]),
    "edb200_sp_barrier": (C.c_int, [c_vp, c_vp]),
    "edb200_qk_norm_rope_pack_sp": (C.c_int, [c_vp, C.c_int, c_i64, c_i64, c_i64, c_i64, c_i64, C.c_int, C.c_int, c_vp,
                                              c_vp, C.c_float, c_vp, c_i64, c_i64, c_vp, C.c_int, c_vp]),
    "edb200_attention_f16_sp": (C.c_int, [c_vp, c_vp, c_vp, C.c_int, c_i64, c_i64, C.c_int, C.c_float, c_vp, C.c_int,
                                          c_i64, c_vp, c_vp]),
    "edb200_attention_sage_int8_sp": (C.c_int, [c_vp, c_vp, c_vp, c_vp, C.c_int, c_vp, C.c_int, c_vp, C.c_int, C.c_int,
                                                c_i64, C.c_int, C.c_float, c_vp, C.c_int, c_i64, c_vp, c_vp]),
    "edb200_sage_attention_sp": (C.c_int, [c_vp, c_vp, c_vp, C.c_int, c_i64, C.c_int, C.c_float, C.c_int, c_vp, c_i64,
                                           c_vp, C.c_int, c_i64, c_vp, c_vp]),
    "edb200_cfg_parallel_combine": (C.c_int, [c_vp, c_vp, C.c_float, c_vp, c_vp, c_i64, c_vp]),
    "edb200_graph_begin": (C.c_int, [c_vp]),
    "edb200_graph_end": (C.c_int, [c_vp, C.POINTER(c_vp)]),
    "edb200_graph_launch": (C.c_int, [c_vp, c_vp]),
    "edb200_graph_destroy": (None, [c_vp]),
    "edb200_flux_set_comm": (C.c_int, [c_vp, c_vp]),
    "edb200_row_rstd": (C.c_int, [c_vp, C.c_int, c_i64, c_i64, c_i64, C.c_float, c_vp, c_vp]),
    "edb200_qk_rownorm_rope_pack": (C.c_int, [c_vp, C.c_int, c_i64, c_i64, c_i64, c_i64, c_i64, C.c_int, C.c_int, c_vp,
                                              c_vp, c_vp, c_vp, c_vp, c_i64, c_i64, c_vp, c_vp, c_vp, C.c_int, c_vp,
                                              c_vp]),
    "edb200_qwen_create": (C.c_int, [C.POINTER(QwenConfig), C.POINTER(c_vp)]),
    "edb200_qwen_destroy": (None, [c_vp]),
    "edb200_qwen_tensor_count": (C.c_int, [c_vp]),
    "edb200_qwen_tensor_info": (C.c_int, [c_vp, C.c_int, C.c_char_p, C.c_int, C.POINTER(C.c_int), C.POINTER(c_i64),
                                          C.POINTER(c_i64), C.POINTER(c_i64)]),
    "edb200_qwen_set_tensor": (C.c_int, [c_vp, C.c_char_p, C.c_int, c_vp, c_i64, C.c_int, c_vp]),
    "edb200_qwen_init_random": (C.c_int, [c_vp, C.c_uint64, C.c_float, c_vp]),
    "edb200_qwen_weight_bytes": (c_i64, [c_vp]),
    "edb200_qwen_prepare": (C.c_int, [c_vp, C.c_int, C.c_int, C.c_int, c_vp]),
    "edb200_qwen_set_tap": (C.c_int, [c_vp, c_vp]),
    "edb200_qwen_set_comm": (C.c_int, [c_vp, c_vp]),
    "edb200_qwen_step": (C.c_int, [c_vp, c_vp, C.c_float, c_vp, c_vp, c_vp]),
    "edb200_qwen_compute_host": (C.c_int, [c_vp, c_vp, C.c_int, C.c_int, C.c_float, c_vp, C.c_int, c_vp, c_vp]),
    "edb200_sd3_create": (C.c_int, [C.POINTER(SD3Config), C.POINTER(c_vp)]),
    "edb200_sd3_destroy": (None, [c_vp]),
    "edb200_sd3_tensor_count": (C.c_int, [c_vp]),
    "edb200_sd3_tensor_info": (C.c_int, [c_vp, C.c_int, C.c_char_p, C.c_int, C.POINTER(C.c_int), C.POINTER(c_i64),
                                         C.POINTER(c_i64), C.POINTER(c_i64)]),
    "edb200_sd3_set_tensor": (C.c_int, [c_vp, C.c_char_p, C.c_int, c_vp, c_i64, C.c_int, c_vp]),
    "edb200_sd3_init_random": (C.c_int, [c_vp, C.c_uint64, C.c_float, c_vp]),
    "edb200_sd3_weight_bytes": (c_i64, [c_vp]),
    "edb200_sd3_prepare": (C.c_int, [c_vp, C.c_int, C.c_int, C.c_int, c_vp]),
    "edb200_sd3_set_tap": (C.c_int, [c_vp, c_vp]),
    "edb200_sd3_step": (C.c_int, [c_vp, c_vp, C.c_float, c_vp, c_vp, c_vp, c_vp]),
    "edb200_sd3_compute_host": (C.c_int, [c_vp, c_vp, C.c_int, C.c_int, C.c_float, c_vp, C.c_int, c_vp, c_vp, c_vp]),
    "edb200_cfg_combine": (C.c_int, [c_vp, c_vp, C.c_float, c_vp, c_i64, c_vp]),
    "edb200_cfg_combine_rescaled": (C.c_int, [c_vp, c_vp, C.c_float, C.c_int, C.c_int, C.c_int, C.c_int, c_vp, c_vp]),
    "edb200_wan_create": (C.c_int, [C.POINTER(WanConfig), C.POINTER(c_vp)]),
    "edb200_wan_destroy": (None, [c_vp]),
    "edb200_wan_tensor_count": (C.c_int, [c_vp]),
    "edb200_wan_tensor_info": (C.c_int, [c_vp, C.c_int, C.c_char_p, C.c_int, C.POINTER(C.c_int), C.POINTER(c_i64),
                                         C.POINTER(c_i64), C.POINTER(c_i64)]),
    "edb200_wan_set_tensor": (C.c_int, [c_vp, C.c_char_p, C.c_int, c_vp, c_i64, C.c_int, c_vp]),
    "edb200_wan_init_random": (C.c_int, [c_vp, C.c_uint64, C.c_float, c_vp]),
    "edb200_wan_weight_bytes": (c_i64, [c_vp]),
    "edb200_wan_workspace_bytes": (c_i64, [c_vp]),
    "edb200_wan_prepare": (C.c_int, [c_vp, C.c_int, C.c_int, C.c_int, C.c_int, c_vp]),
    "edb200_wan_set_tap": (C.c_int, [c_vp, c_vp]),
    "edb200_wan_set_comm": (C.c_int, [c_vp, c_vp]),
    "edb200_wan_step": (C.c_int, [c_vp, c_vp, C.c_float, c_vp, c_vp, c_vp]),
    "edb200_wan_compute_host": (C.c_int, [c_vp, c_vp, C.c_int, C.c_int, C.c_int, C.c_float, c_vp, C.c_int, c_vp, c_vp]),
    "edb200_flux_create": (C.c_int, [C.POINTER(FluxConfig), C.POINTER(c_vp)]),
    "edb200_flux_destroy": (None, [c_vp]),
    "edb200_flux_tensor_count": (C.c_int, [c_vp]),
    "edb200_flux_tensor_info": (C.c_int, [c_vp, C.c_int, C.c_char_p, C.c_int, C.POINTER(C.c_int), C.POINTER(c_i64),
                                          C.POINTER(c_i64), C.POINTER(c_i64)]),
    "edb200_flux_set_tensor": (C.c_int, [c_vp, C.c_char_p, C.c_int, c_vp, c_i64, C.c_int, c_vp]),
    "edb200_flux_init_random": (C.c_int, [c_vp, C.c_uint64, C.c_float, c_vp]),
    "edb200_flux_weight_bytes": (c_i64, [c_vp]),
    "edb200_flux_workspace_bytes": (c_i64, [c_vp]),
    "edb200_flux_prepare": (C.c_int, [c_vp, C.c_int, C.c_int, C.c_int, c_vp]),
    "edb200_flux_set_tap": (C.c_int, [c_vp, c_vp]),
    "edb200_gguf_open": (C.c_int, [C.c_char_p, C.POINTER(c_vp)]),
    "edb200_gguf_close": (None, [c_vp]),
    "edb200_gguf_tensor_count": (C.c_int, [c_vp]),
    "edb200_gguf_tensor_info": (C.c_int, [c_vp, C.c_int, C.c_char_p, C.c_int, C.POINTER(C.c_int), C.POINTER(C.c_int),
                                          C.POINTER(c_i64), C.POINTER(c_i64)]),
    "edb200_gguf_tensor_data": (c_vp, [c_vp, C.c_int]),
    "edb200_safetensors_open": (C.c_int, [C.c_char_p, C.POINTER(c_vp)]),
    "edb200_safetensors_close": (None, [c_vp]),
    "edb200_safetensors_tensor_count": (C.c_int, [c_vp]),
    "edb200_safetensors_tensor_info": (C.c_int, [c_vp, C.c_int, C.c_char_p, C.c_int, C.c_char_p, C.c_int,
                                                 C.POINTER(C.c_int), C.POINTER(c_i64), C.POINTER(c_i64)]),
    "edb200_safetensors_tensor_data": (c_vp, [c_vp, C.c_int]),
    "edb200_safetensors_index_files": (C.c_int, [C.c_char_p, C.c_char_p, C.c_int, C.POINTER(C.c_int)]),
    "edb200_canonical_tensor_name": (C.c_int, [C.c_int, C.c_char_p, C.c_char_p, C.c_int64, C.POINTER(C.c_int)]),
    "edb200_mul_mat_q_fuses_qk_pack": (C.c_int, []),
    "edb200_flux_load_safetensors": (C.c_int, [c_vp, C.c_char_p, C.c_char_p, C.POINTER(C.c_int), c_vp]),
    "edb200_sd3_load_safetensors": (C.c_int, [c_vp, C.c_char_p, C.c_char_p, C.POINTER(C.c_int), c_vp]),
    "edb200_qwen_load_safetensors": (C.c_int, [c_vp, C.c_char_p, C.c_char_p, C.POINTER(C.c_int), c_vp]),
    "edb200_wan_load_safetensors": (C.c_int, [c_vp, C.c_char_p, C.c_char_p, C.POINTER(C.c_int), c_vp]),
    "edb200_flux_load_gguf": (C.c_int, [c_vp, C.c_char_p, C.c_char_p, C.POINTER(C.c_int), c_vp]),
    "edb200_sd3_load_gguf": (C.c_int, [c_vp, C.c_char_p, C.c_char_p, C.POINTER(C.c_int), c_vp]),
    "edb200_qwen_load_gguf": (C.c_int, [c_vp, C.c_char_p, C.c_char_p, C.POINTER(C.c_int), c_vp]),
    "edb200_wan_load_gguf": (C.c_int, [c_vp, C.c_char_p, C.c_char_p, C.POINTER(C.c_int), c_vp]),
    "edb200_flux_step": (C.c_int, [c_vp, c_vp, C.c_float, c_vp, c_vp, C.c_float, c_vp, c_vp]),
    "edb200_flux_step_sched": (C.c_int, [c_vp, c_vp, c_vp, c_vp, c_vp, c_vp, C.c_float, c_vp, c_vp]),
    "edb200_flux_compute_host": (C.c_int, [c_vp, c_vp, C.c_int, C.c_int, C.c_float, c_vp, C.c_int, c_vp, C.c_float,
                                           c_vp, c_vp]),
}

_lib = None


def declared_symbols():
    """Names this binding expects; tests cross-check them against the header."""
    return sorted(_SIGS)


def lib():
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise ImportError(f"{LIB_PATH} not built; run python edge-dit.cpp_b200/build.py")
        l = C.CDLL(LIB_PATH)
        for name, (res, args) in _SIGS.items():
            fn = getattr(l, name)
            fn.restype = res
            fn.argtypes = args
        _lib = l
    return _lib


def check(status: int):
    if status != OK:
        raise EdbError(status, lib().edb200_last_error().decode())


def ptr(t):
    """Device pointer of a torch tensor (or None)."""
    return None if t is None else c_vp(t.data_ptr())


def torch_dtype_id(t) -> int:
    import torch
    return {torch.float32: TYPE_F32, torch.float16: TYPE_F16, torch.bfloat16: TYPE_BF16}[t.dtype]


def current_stream():
    import torch
    return c_vp(torch.cuda.current_stream().cuda_stream)


class QWeight:
    """Owns an edb200_qweight_t built from raw ggml blocks (uint8 torch tensor on the device)."""

    def __init__(self, ggml_type: int, blocks, n_out: int, k: int):
        h = c_vp()
        check(lib().edb200_qweight_create(ggml_type, ptr(blocks), n_out, k, current_stream(), C.byref(h)))
        self.handle = h
        self.ggml_type, self.n_out, self.k = ggml_type, n_out, k

    def __del__(self):
        if getattr(self, "handle", None) and _lib is not None:
            _lib.edb200_qweight_destroy(self.handle)
            self.handle = None


def make_epilogue(out, bias=None, act=ACT_NONE, residual=None, gate=None, split_n=0, out2=None, act2=ACT_NONE,
                  ldo=None, ldo2=None, split_k=0):
    ep = Epilogue()
    ep.bias = ptr(bias)
    ep.act = act
    ep.out = ptr(out)
    ep.out_dtype = torch_dtype_id(out)
    ep.ldo = out.stride(0) if ldo is None else ldo
    ep.residual = ptr(residual)
    ep.ld_res = residual.stride(0) if residual is not None else 0
    ep.gate = ptr(gate)
    ep.split_n = split_n
    ep.out2 = ptr(out2)
    ep.out2_dtype = torch_dtype_id(out2) if out2 is not None else 0
    ep.ldo2 = (out2.stride(0) if ldo2 is None else ldo2) if out2 is not None else 0
    ep.act2 = act2
    ep.split_k = split_k
    return ep


def mul_mat_q(w: QWeight, x, ep: Epilogue):
    check(lib().edb200_mul_mat_q(w.handle, ptr(x), torch_dtype_id(x), x.shape[0], x.stride(0), C.byref(ep),
                                 current_stream()))


class GGUF:
    """Read-only view of a GGUF file through the library's reader (no GPU needed)."""

    def __init__(self, path):
        h = c_vp()
        check(lib().edb200_gguf_open(str(path).encode(), C.byref(h)))
        self.handle = h

    def __len__(self):
        return lib().edb200_gguf_tensor_count(self.handle)

    def tensor(self, i):
        """(name, ggml_type, dims in ggml order, bytes) of tensor i; bytes is None for a type that is not read."""
        name = C.create_string_buffer(512)
        t, nd, nb = C.c_int(), C.c_int(), c_i64()
        dims = (c_i64 * 4)()
        check(lib().edb200_gguf_tensor_info(self.handle, i, name, 512, C.byref(t), C.byref(nd), dims, C.byref(nb)))
        data = None
        if nb.value >= 0:
            data = C.string_at(lib().edb200_gguf_tensor_data(self.handle, i), nb.value)
        return name.value.decode(), t.value, tuple(dims[d] for d in range(nd.value)), data

    def close(self):
        if getattr(self, "handle", None) and _lib is not None:
            _lib.edb200_gguf_close(self.handle)
            self.handle = None

    __del__ = close


class SafeTensors:
    """Read-only view of a safetensors file through the library's reader (no GPU needed)."""

    def __init__(self, path):
        h = c_vp()
        check(lib().edb200_safetensors_open(str(path).encode(), C.byref(h)))
        self.handle = h

    def __len__(self):
        return lib().edb200_safetensors_tensor_count(self.handle)

    def tensor(self, i):
        """(name, dtype string, row-major shape, bytes) of tensor i."""
        name, dtype = C.create_string_buffer(512), C.create_string_buffer(16)
        nd, nb = C.c_int(), c_i64()
        dims = (c_i64 * 8)()
        check(lib().edb200_safetensors_tensor_info(self.handle, i, name, 512, dtype, 16, C.byref(nd), dims, C.byref(nb)))
        data = C.string_at(lib().edb200_safetensors_tensor_data(self.handle, i), nb.value)
        return name.value.decode(), dtype.value.decode(), tuple(dims[d] for d in range(nd.value)), data

    def close(self):
        if getattr(self, "handle", None) and _lib is not None:
            _lib.edb200_safetensors_close(self.handle)
            self.handle = None

    __del__ = close


FAMILY_FLUX, FAMILY_SD3, FAMILY_QWEN, FAMILY_WAN = 0, 1, 2, 3


def canonical_tensor_name(family, name):
    """(name in the executors' layout, part index) for a checkpoint tensor name, as the loaders see it
    (convert_diffusion_model_name, reference src/utils/name_conversion.cpp:802-822)."""
    buf = C.create_string_buffer(1024)
    part = C.c_int(0)
    check(lib().edb200_canonical_tensor_name(int(family), str(name).encode(), buf, len(buf), C.byref(part)))
    return buf.value.decode(), part.value


def safetensors_index_files(index_path):
    """Shard files named by a *.safetensors.index.json, in order of first appearance."""
    buf = C.create_string_buffer(1 << 16)
    n = C.c_int()
    check(lib().edb200_safetensors_index_files(str(index_path).encode(), buf, len(buf), C.byref(n)))
    files = buf.value.decode().splitlines()
    assert len(files) == n.value
    return files


def _load_gguf(fn, handle, path, strip_prefix):
    n = C.c_int()
    check(fn(handle, str(path).encode(), strip_prefix.encode() if strip_prefix else None, C.byref(n), current_stream()))
    return n.value


class _ParamAccess:
    """Parameter table access shared by the model classes (`_FAMILY` names the C entry points)."""

    def tensor_table(self):
        """[(name, ggml_type, n_out, k, raw bytes)] of every parameter."""
        l = lib()
        count = getattr(l, f"edb200_{self._FAMILY}_tensor_count")
        info = getattr(l, f"edb200_{self._FAMILY}_tensor_info")
        buf = C.create_string_buffer(256)
        t, no, k, nb = C.c_int(), c_i64(), c_i64(), c_i64()
        out = []
        for i in range(count(self.handle)):
            check(info(self.handle, i, buf, 256, C.byref(t), C.byref(no), C.byref(k), C.byref(nb)))
            out.append((buf.value.decode(), t.value, no.value, k.value, nb.value))
        return out

    def get_tensor(self, name):
        """The tensor as the device holds it, read back as numpy f32 [n_out, k] (vectors: [k]);
        quantised weights come back dequantised."""
        import numpy as np
        if not hasattr(self, "_shapes"):
            self._shapes = {n: (no, k) for n, _, no, k, _ in self.tensor_table()}
        no, k = self._shapes[name]
        out = np.empty((no, k), dtype=np.float32)
        fn = getattr(lib(), f"edb200_{self._FAMILY}_get_tensor_f32")
        check(fn(self.handle, name.encode(), out.ctypes.data_as(c_vp), out.size, 0, current_stream()))
        return out[0] if no == 1 else out


def euler_update(x, model_out, sigma, sigma_next):
    """In place on the device: x <- x + ((x - denoised)/sigma)*(sigma_next - sigma), denoised = x - sigma*model_out."""
    check(lib().edb200_euler_update(ptr(x), ptr(model_out), sigma, sigma_next, x.numel(), current_stream()))


def sp_shard(n_tokens, n_txt, rank, world):
    """(t_loc, n_txt_local, img_first, t_rows) of `rank`'s token slice: its slot of the padded
    sequence has t_loc rows, of which it owns the first t_rows."""
    a, b, c, d = c_i64(), c_i64(), c_i64(), c_i64()
    check(lib().edb200_sp_shard(n_tokens, n_txt, rank, world, C.byref(a), C.byref(b), C.byref(c), C.byref(d)))
    return a.value, b.value, c.value, d.value


def poll_status():
    """Synchronises the current stream and raises EdbError(status 4) if a device-side wait gave up."""
    check(lib().edb200_poll_status(current_stream()))


def sp_heads_plan(rank, world, heads, t_loc, row_bytes):
    """Messages of the heads exchange as (peer, send_off, recv_off, bytes) tuples."""
    n = lib().edb200_sp_heads_plan(rank, world, heads, t_loc, row_bytes, None, None, None, None, 0)
    if n < 0:
        raise EdbError(1, "sp_heads_plan: bad argument")
    peer, so, ro, nb = (C.c_int * n)(), (c_i64 * n)(), (c_i64 * n)(), (c_i64 * n)()
    lib().edb200_sp_heads_plan(rank, world, heads, t_loc, row_bytes, peer, so, ro, nb, n)
    return [(peer[i], so[i], ro[i], nb[i]) for i in range(n)]


class Comm:
    """NCCL communicator of the library over ranks of an initialised torch.distributed group (one
    process per GPU); torch.distributed only carries the 128-byte id.

    ranks = None: all ranks.  ranks = [global ranks]: a communicator over that subset, this process
    being one of them (its rank inside is its position in the list); EVERY process of the world must
    then call Comm(...) at the same point, each with the subset it belongs to, because the ids
    travel in one collective over the whole world.  This is how a CFG-parallel x sequence-parallel
    world is built: one communicator per guidance branch and one per pair of branch partners."""

    def __init__(self, ranks=None):
        import torch
        import torch.distributed as dist
        g_rank, g_world = dist.get_rank(), dist.get_world_size()
        ranks = list(range(g_world)) if ranks is None else [int(r) for r in ranks]
        if g_rank not in ranks:
            raise ValueError(f"rank {g_rank} is not in {ranks}")
        rank, world = ranks.index(g_rank), len(ranks)
        buf = C.create_string_buffer(128)
        if rank == 0:
            check(lib().edb200_comm_unique_id(buf))
        ids = [None] * g_world
        dist.all_gather_object(ids, bytes(buf.raw) if rank == 0 else None)
        h = c_vp()
        check(lib().edb200_comm_create(ids[ranks[0]], rank, world, C.byref(h)))
        self.handle, self.rank, self.world, self.ranks = h, rank, world, ranks
        torch.cuda.synchronize()

    def close(self):
        if getattr(self, "handle", None) and _lib is not None:
            _lib.edb200_comm_destroy(self.handle)
            self.handle = None


class FluxModel(_ParamAccess):
    _FAMILY = "flux"

    """Thin owner of an edb200_flux_t: the host-side mirror of the reference's
    FluxModel adapter (src/dit_models/diffusion_model.hpp) over the C ABI."""

    def __init__(self, hidden_size=3072, num_heads=24, depth=19, depth_single_blocks=38, mlp_hidden=None,
                 in_channels=64, context_in_dim=4096, vec_in_dim=768, patch_size=2, axes_dim=(16, 56, 56),
                 theta=10000, guidance_embed=True, wtype=TYPE_Q8_0, attention=ATTN_SAGE_INT8, sage_smooth_q=True):
        cfg = FluxConfig()
        cfg.hidden_size, cfg.num_heads, cfg.depth, cfg.depth_single_blocks = hidden_size, num_heads, depth, depth_single_blocks
        cfg.mlp_hidden = mlp_hidden if mlp_hidden is not None else 4 * hidden_size
        cfg.in_channels, cfg.context_in_dim, cfg.vec_in_dim, cfg.patch_size = in_channels, context_in_dim, vec_in_dim, patch_size
        cfg.axes_dim = (C.c_int * 3)(*axes_dim)
        cfg.theta, cfg.guidance_embed, cfg.wtype = theta, int(guidance_embed), wtype
        cfg.attention, cfg.sage_smooth_q = attention, int(sage_smooth_q)
        self.cfg = cfg
        h = c_vp()
        check(lib().edb200_flux_create(C.byref(cfg), C.byref(h)))
        self.handle = h

    def __del__(self):
        if getattr(self, "handle", None) and _lib is not None:
            _lib.edb200_flux_destroy(self.handle)
            self.handle = None

    def tensors(self):
        out = []
        n = lib().edb200_flux_tensor_count(self.handle)
        buf = C.create_string_buffer(256)
        t, no, k, nb = C.c_int(), c_i64(), c_i64(), c_i64()
        for i in range(n):
            check(lib().edb200_flux_tensor_info(self.handle, i, buf, 256, C.byref(t), C.byref(no), C.byref(k), C.byref(nb)))
            out.append((buf.value.decode(), t.value, no.value, k.value, nb.value))
        return out

    def load_numpy(self, weights: dict):
        """weights: {name: (ggml_type, ndarray)} as produced by oracle.flux_oracle.flux_make_weights."""
        import numpy as np
        for name, (t, arr) in weights.items():
            a = np.ascontiguousarray(arr)
            check(lib().edb200_flux_set_tensor(self.handle, name.encode(), t, a.ctypes.data_as(c_vp), a.nbytes, 0,
                                               current_stream()))

    def set_comm(self, comm):
        """Sequence-parallel execution over `comm` (None = single GPU); call before prepare."""
        self._comm = comm  # keep the communicator alive as long as the model uses it
        check(lib().edb200_flux_set_comm(self.handle, comm.handle if comm is not None else None))

    def init_random(self, seed=0, std=0.02):
        check(lib().edb200_flux_init_random(self.handle, seed, std, current_stream()))

    def load_gguf(self, path, strip_prefix="model.diffusion_model."):
        """Loads the tensors of a GGUF file this model has parameters for; returns how many were taken."""
        return _load_gguf(lib().edb200_flux_load_gguf, self.handle, path, strip_prefix)

    def load_safetensors(self, path, strip_prefix="model.diffusion_model."):
        """Loads (and, for quantised parameters, encodes on the device) the tensors of a safetensors file."""
        return _load_gguf(lib().edb200_flux_load_safetensors, self.handle, path, strip_prefix)

    def prepare(self, latent_h, latent_w, n_txt):
        check(lib().edb200_flux_prepare(self.handle, latent_h, latent_w, n_txt, current_stream()))

    def step(self, latent, timestep, context, y, guidance, out):
        check(lib().edb200_flux_step(self.handle, ptr(latent), timestep, ptr(context), ptr(y), guidance, ptr(out),
                                     current_stream()))

    def denoise(self, latent, sigmas, context, y, guidance, velocity=None):
        """The sampler loop with the latent resident on the device: for each consecutive pair of
        `sigmas` one step at timestep sigma and the reference's Euler update in place
        (src/dit_models/pipelines/flux_pipeline.cpp:1111-1116, :1290-1297).  Nothing returns to
        the host between steps.  `velocity` is scratch of the latent's shape."""
        import torch
        v = torch.empty_like(latent) if velocity is None else velocity
        for sigma, sigma_next in zip(sigmas[:-1], sigmas[1:]):
            self.step(latent, float(sigma), context, y, guidance, v)
            euler_update(latent, v, float(sigma), float(sigma_next))
        return latent

    def denoise_graph(self, latent, sigmas, context, y, guidance, velocity=None):
        """`denoise` with one recorded (step + update) replayed for every step: the schedule lives in
        device memory and a device counter walks through it, so the recording holds no sigma.
        Must run on a non-default stream (stream capture)."""
        import torch
        v = torch.empty_like(latent) if velocity is None else velocity
        sched = torch.tensor([float(x) for x in sigmas], dtype=torch.float32, device=latent.device)
        step = torch.zeros(1, dtype=torch.int32, device=latent.device)
        n = latent.numel()

        def one():
            check(lib().edb200_flux_step_sched(self.handle, ptr(latent), ptr(sched), ptr(step), ptr(context), ptr(y),
                                               guidance, ptr(v), current_stream()))
            check(lib().edb200_euler_update_sched(ptr(latent), ptr(v), ptr(sched), ptr(step), n, current_stream()))

        saved = latent.clone()
        one()                      # warm: first-call attribute settings happen outside the recording
        latent.copy_(saved)
        step.zero_()
        graph = Graph(one)         # recording executes nothing
        for _ in range(len(sigmas) - 1):
            graph.launch()
        torch.cuda.current_stream().synchronize()
        return latent

    def compute_host(self, latent, timestep, context, y, guidance):
        """numpy f32 in, numpy f32 out; host<->device copies happen inside the call."""
        import numpy as np
        latent = np.ascontiguousarray(latent, dtype=np.float32)
        context = np.ascontiguousarray(context, dtype=np.float32)
        y = np.ascontiguousarray(y, dtype=np.float32)
        out = np.empty_like(latent)
        check(lib().edb200_flux_compute_host(self.handle, latent.ctypes.data_as(c_vp), latent.shape[1], latent.shape[2],
                                             timestep, context.ctypes.data_as(c_vp), context.shape[0],
                                             y.ctypes.data_as(c_vp), guidance, out.ctypes.data_as(c_vp),
                                             current_stream()))
        return out


class QwenModel(_ParamAccess):
    _FAMILY = "qwen"

    """Thin owner of an edb200_qwen_t (host-side mirror of the reference's QwenImageModel adapter,
    src/dit_models/diffusion_model.hpp) over the C ABI; one call is one batch-1 pass."""

    def __init__(self, num_layers=60, num_heads=24, head_dim=128, mlp_hidden=None, in_channels=64, out_channels=16,
                 joint_attention_dim=3584, patch_size=2, axes_dim=(16, 56, 56), theta=10000, wtype=TYPE_Q4_K,
                 attention=ATTN_SAGE_INT8, sage_smooth_q=True):
        cfg = QwenConfig()
        cfg.num_layers, cfg.num_heads, cfg.head_dim = num_layers, num_heads, head_dim
        cfg.mlp_hidden = mlp_hidden if mlp_hidden is not None else 4 * num_heads * head_dim
        cfg.in_channels, cfg.out_channels, cfg.joint_attention_dim, cfg.patch_size = in_channels, out_channels, joint_attention_dim, patch_size
        cfg.axes_dim = (C.c_int * 3)(*axes_dim)
        cfg.theta, cfg.wtype, cfg.attention, cfg.sage_smooth_q = theta, wtype, attention, int(sage_smooth_q)
        self.cfg = cfg
        h = c_vp()
        check(lib().edb200_qwen_create(C.byref(cfg), C.byref(h)))
        self.handle = h

    def __del__(self):
        if getattr(self, "handle", None) and _lib is not None:
            _lib.edb200_qwen_destroy(self.handle)
            self.handle = None

    def tensor_names(self):
        buf = C.create_string_buffer(256)
        out = []
        for i in range(lib().edb200_qwen_tensor_count(self.handle)):
            check(lib().edb200_qwen_tensor_info(self.handle, i, buf, 256, None, None, None, None))
            out.append(buf.value.decode())
        return out

    def load_numpy(self, weights: dict):
        import numpy as np
        for name, (t, arr) in weights.items():
            a = np.ascontiguousarray(arr)
            check(lib().edb200_qwen_set_tensor(self.handle, name.encode(), t, a.ctypes.data_as(c_vp), a.nbytes, 0,
                                               current_stream()))

    def init_random(self, seed=0, std=0.02):
        check(lib().edb200_qwen_init_random(self.handle, seed, std, current_stream()))

    def load_gguf(self, path, strip_prefix="model.diffusion_model."):
        """Loads the tensors of a GGUF file this model has parameters for; returns how many were taken."""
        return _load_gguf(lib().edb200_qwen_load_gguf, self.handle, path, strip_prefix)

    def load_safetensors(self, path, strip_prefix="model.diffusion_model."):
        """Loads (and, for quantised parameters, encodes on the device) the tensors of a safetensors file."""
        return _load_gguf(lib().edb200_qwen_load_safetensors, self.handle, path, strip_prefix)

    def set_comm(self, comm):
        self._comm = comm
        check(lib().edb200_qwen_set_comm(self.handle, comm.handle if comm is not None else None))

    def set_tap(self, tap):
        self._tap = tap
        check(lib().edb200_qwen_set_tap(self.handle, ptr(tap)))

    def prepare(self, lat_h, lat_w, n_txt):
        check(lib().edb200_qwen_prepare(self.handle, lat_h, lat_w, n_txt, current_stream()))

    def step(self, latent, timestep, context, out):
        check(lib().edb200_qwen_step(self.handle, ptr(latent), timestep, ptr(context), ptr(out), current_stream()))

    def compute_host(self, latent, timestep, context):
        import numpy as np
        latent = np.ascontiguousarray(latent, dtype=np.float32)
        context = np.ascontiguousarray(context, dtype=np.float32)
        out = np.empty((self.cfg.out_channels,) + latent.shape[1:], dtype=np.float32)
        check(lib().edb200_qwen_compute_host(self.handle, latent.ctypes.data_as(c_vp), latent.shape[1], latent.shape[2],
                                             timestep, context.ctypes.data_as(c_vp), context.shape[0],
                                             out.ctypes.data_as(c_vp), current_stream()))
        return out


class SD3Model(_ParamAccess):
    _FAMILY = "sd3"

    """Thin owner of an edb200_sd3_t (host-side mirror of the reference's MMDiTModel adapter,
    src/dit_models/diffusion_model.hpp) over the C ABI; one call is one batch-1 pass."""

    def __init__(self, hidden_size=1536, num_heads=24, depth=24, mlp_hidden=None, in_channels=16, out_channels=16,
                 patch_size=2, adm_in_channels=2048, context_size=4096, pos_embed_max_size=192, wtype=TYPE_Q8_0,
                 attention=ATTN_F16, sage_smooth_q=False, sage_skip_first=2, sage_skip_last=2):
        cfg = SD3Config()
        cfg.hidden_size, cfg.num_heads, cfg.depth = hidden_size, num_heads, depth
        cfg.mlp_hidden = mlp_hidden if mlp_hidden is not None else 4 * hidden_size
        cfg.in_channels, cfg.out_channels, cfg.patch_size = in_channels, out_channels, patch_size
        cfg.adm_in_channels, cfg.context_size, cfg.pos_embed_max_size = adm_in_channels, context_size, pos_embed_max_size
        cfg.wtype, cfg.attention = wtype, attention
        cfg.sage_smooth_q, cfg.sage_skip_first, cfg.sage_skip_last = int(sage_smooth_q), sage_skip_first, sage_skip_last
        self.cfg = cfg
        h = c_vp()
        check(lib().edb200_sd3_create(C.byref(cfg), C.byref(h)))
        self.handle = h

    def __del__(self):
        if getattr(self, "handle", None) and _lib is not None:
            _lib.edb200_sd3_destroy(self.handle)
            self.handle = None

    def tensor_names(self):
        buf = C.create_string_buffer(256)
        out = []
        for i in range(lib().edb200_sd3_tensor_count(self.handle)):
            check(lib().edb200_sd3_tensor_info(self.handle, i, buf, 256, None, None, None, None))
            out.append(buf.value.decode())
        return out

    def load_numpy(self, weights: dict):
        import numpy as np
        for name, (t, arr) in weights.items():
            a = np.ascontiguousarray(arr)
            check(lib().edb200_sd3_set_tensor(self.handle, name.encode(), t, a.ctypes.data_as(c_vp), a.nbytes, 0,
                                              current_stream()))

    def init_random(self, seed=0, std=0.02):
        check(lib().edb200_sd3_init_random(self.handle, seed, std, current_stream()))

    def load_gguf(self, path, strip_prefix="model.diffusion_model."):
        """Loads the tensors of a GGUF file this model has parameters for; returns how many were taken."""
        return _load_gguf(lib().edb200_sd3_load_gguf, self.handle, path, strip_prefix)

    def load_safetensors(self, path, strip_prefix="model.diffusion_model."):
        """Loads (and, for quantised parameters, encodes on the device) the tensors of a safetensors file."""
        return _load_gguf(lib().edb200_sd3_load_safetensors, self.handle, path, strip_prefix)

    def set_comm(self, comm):
        self._comm = comm
        check(lib().edb200_sd3_set_comm(self.handle, comm.handle if comm is not None else None))

    def set_tap(self, tap):
        self._tap = tap
        check(lib().edb200_sd3_set_tap(self.handle, ptr(tap)))

    def prepare(self, lat_h, lat_w, n_ctx):
        check(lib().edb200_sd3_prepare(self.handle, lat_h, lat_w, n_ctx, current_stream()))

    def step(self, latent, timestep, context, y, out):
        check(lib().edb200_sd3_step(self.handle, ptr(latent), timestep, ptr(context), ptr(y), ptr(out), current_stream()))

    def compute_host(self, latent, timestep, context, y):
        import numpy as np
        latent = np.ascontiguousarray(latent, dtype=np.float32)
        context = np.ascontiguousarray(context, dtype=np.float32)
        y = np.ascontiguousarray(y, dtype=np.float32)
        out = np.empty((self.cfg.out_channels,) + latent.shape[1:], dtype=np.float32)
        check(lib().edb200_sd3_compute_host(self.handle, latent.ctypes.data_as(c_vp), latent.shape[1], latent.shape[2],
                                            timestep, context.ctypes.data_as(c_vp), context.shape[0],
                                            y.ctypes.data_as(c_vp), out.ctypes.data_as(c_vp), current_stream()))
        return out


class WanModel(_ParamAccess):
    _FAMILY = "wan"

    """Thin owner of an edb200_wan_t (host-side mirror of the reference's WanModel adapter,
    src/dit_models/diffusion_model.hpp) over the C ABI."""

    def __init__(self, dim=5120, num_heads=40, ffn_dim=13824, num_layers=40, in_dim=16, out_dim=16, text_dim=4096,
                 freq_dim=256, patch_size=(1, 2, 2), axes_dim=(44, 42, 42), theta=10000, wtype=TYPE_Q8_0,
                 attention=ATTN_SAGE_INT8, sage_smooth_q=True, sage_skip_first=2, sage_skip_last=2):
        cfg = WanConfig()
        cfg.dim, cfg.num_heads, cfg.ffn_dim, cfg.num_layers = dim, num_heads, ffn_dim, num_layers
        cfg.in_dim, cfg.out_dim, cfg.text_dim, cfg.freq_dim = in_dim, out_dim, text_dim, freq_dim
        cfg.patch_size = (C.c_int * 3)(*patch_size)
        cfg.axes_dim = (C.c_int * 3)(*axes_dim)
        cfg.theta, cfg.wtype, cfg.attention, cfg.sage_smooth_q = theta, wtype, attention, int(sage_smooth_q)
        cfg.sage_skip_first, cfg.sage_skip_last = sage_skip_first, sage_skip_last
        self.cfg = cfg
        h = c_vp()
        check(lib().edb200_wan_create(C.byref(cfg), C.byref(h)))
        self.handle = h

    def __del__(self):
        if getattr(self, "handle", None) and _lib is not None:
            _lib.edb200_wan_destroy(self.handle)
            self.handle = None

    def load_numpy(self, weights: dict):
        """weights: {name: (ggml_type, ndarray)} as produced by oracle.wan_oracle.wan_make_weights."""
        import numpy as np
        for name, (t, arr) in weights.items():
            a = np.ascontiguousarray(arr)
            check(lib().edb200_wan_set_tensor(self.handle, name.encode(), t, a.ctypes.data_as(c_vp), a.nbytes, 0,
                                              current_stream()))

    def init_random(self, seed=0, std=0.02):
        check(lib().edb200_wan_init_random(self.handle, seed, std, current_stream()))

    def load_gguf(self, path, strip_prefix="model.diffusion_model."):
        """Loads the tensors of a GGUF file this model has parameters for; returns how many were taken."""
        return _load_gguf(lib().edb200_wan_load_gguf, self.handle, path, strip_prefix)

    def load_safetensors(self, path, strip_prefix="model.diffusion_model."):
        """Loads (and, for quantised parameters, encodes on the device) the tensors of a safetensors file."""
        return _load_gguf(lib().edb200_wan_load_safetensors, self.handle, path, strip_prefix)

    def set_comm(self, comm):
        self._comm = comm
        check(lib().edb200_wan_set_comm(self.handle, comm.handle if comm is not None else None))

    def set_tap(self, tap):
        self._tap = tap
        check(lib().edb200_wan_set_tap(self.handle, ptr(tap)))

    def prepare(self, frames, lat_h, lat_w, n_ctx):
        check(lib().edb200_wan_prepare(self.handle, frames, lat_h, lat_w, n_ctx, current_stream()))

    def step(self, latent, timestep, context, out):
        check(lib().edb200_wan_step(self.handle, ptr(latent), timestep, ptr(context), ptr(out), current_stream()))

    def compute_host(self, latent, timestep, context):
        import numpy as np
        latent = np.ascontiguousarray(latent, dtype=np.float32)
        context = np.ascontiguousarray(context, dtype=np.float32)
        out = np.empty((self.cfg.out_dim,) + latent.shape[1:], dtype=np.float32)
        check(lib().edb200_wan_compute_host(self.handle, latent.ctypes.data_as(c_vp), latent.shape[1], latent.shape[2],
                                            latent.shape[3], timestep, context.ctypes.data_as(c_vp), context.shape[0],
                                            out.ctypes.data_as(c_vp), current_stream()))
        return out


class Graph:
    """Records what `fn()` enqueues on the current (non-default) stream and replays it."""

    def __init__(self, fn):
        check(lib().edb200_graph_begin(current_stream()))
        try:
            fn()
        finally:
            h = c_vp()
            st = lib().edb200_graph_end(current_stream(), C.byref(h))
        check(st)
        self.handle = h

    def launch(self):
        check(lib().edb200_graph_launch(self.handle, current_stream()))

    def __del__(self):
        if getattr(self, "handle", None) and _lib is not None:
            _lib.edb200_graph_destroy(self.handle)
            self.handle = None


PROF_CLASSES = ("gemm", "attention", "gemv", "elementwise", "other")


def profile_begin():
    check(lib().edb200_profile_begin())


def profile_end():
    ms, fl, by = (C.c_double * 5)(), (C.c_double * 5)(), (C.c_double * 5)()
    n = (c_i64 * 5)()
    check(lib().edb200_profile_end(ms, fl, by, n))
    return {name: {"ms": ms[i], "flops": fl[i], "bytes": by[i], "launches": n[i]}
            for i, name in enumerate(PROF_CLASSES)}

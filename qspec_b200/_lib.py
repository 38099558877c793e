"""ctypes binding of the C-ABI library (include/qspec_b200.h).

There is NO fallback: if the shared library is missing or a call fails, this raises.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import c_char_p, c_float, c_int, c_size_t, c_uint64, c_void_p

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.environ.get("QSPEC_LIB") or os.path.join(_HERE, "_C", "libqspec_b200.so")

QSPEC_OK = 0
DTYPE_F16 = 0
DTYPE_BF16 = 1

# name -> (restype, argtypes); mirrors include/qspec_b200.h one to one
SIGNATURES = {
    "qspec_abi_version": (c_int, []),
    "qspec_last_error": (c_char_p, []),
    "qspec_launch_count": (c_uint64, []),
    "qspec_sm_count": (c_int, []),
    "qspec_debug_set_gemm_trace": (None, [c_void_p]),
    "qspec_norm_quant_i4": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_float, c_void_p]),
    "qspec_norm_f16": (c_int, [c_void_p, c_void_p, c_int, c_int, c_float, c_int, c_void_p]),
    "qspec_add_norm_quant_i4": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_float, c_void_p]),
    "qspec_add_norm_f16": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_int, c_float, c_int, c_void_p]),
    "qspec_gemm_split_factor": (c_int, [c_int, c_int, c_int, c_int]),
    "qspec_gemm_w4a4_split": (c_int, [c_void_p, c_void_p, c_void_p, c_size_t, c_int, c_int, c_int, c_void_p, c_size_t,
                                      c_void_p]),
    "qspec_gemm_w4a16_split": (c_int, [c_void_p, c_void_p, c_void_p, c_size_t, c_int, c_int, c_int, c_int, c_void_p,
                                       c_size_t, c_void_p]),
    "qspec_split_add_norm_quant_i4": (c_int, [c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p,
                                              c_void_p, c_void_p, c_int, c_int, c_float, c_void_p]),
    "qspec_split_add_norm_f16": (c_int, [c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p,
                                         c_int, c_int, c_float, c_int, c_void_p]),
    "qspec_tp_add_norm_quant_i4": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p,
                                           c_void_p, c_int, c_int, c_float, c_void_p]),
    "qspec_tp_add_norm_f16": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p, c_int, c_int,
                                      c_float, c_int, c_void_p]),
    "qspec_tp_rs_add_norm_quant_i4": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int,
                                              c_void_p, c_void_p, c_void_p, c_int, c_int, c_float, c_void_p]),
    "qspec_tp_rs_add_norm_f16": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int,
                                         c_void_p, c_int, c_int, c_float, c_int, c_void_p]),
    "qspec_split_add_norm_quant_i4_c8": (c_int, [c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p,
                                              c_void_p, c_void_p, c_int, c_int, c_float, c_void_p]),
    "qspec_tp_add_norm_quant_i4_c8": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p,
                                           c_void_p, c_int, c_int, c_float, c_void_p]),
    "qspec_hadamard_heads_c8": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int,
                                     c_float, c_float, c_void_p]),
    "qspec_hadamard_k28_c8": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int,
                                   c_float, c_float, c_void_p]),
    "qspec_gemm_w4a8_split": (c_int, [c_void_p, c_void_p, c_void_p, c_size_t, c_int, c_int, c_int, c_void_p, c_size_t,
                                      c_void_p]),
    "qspec_debug_gemm_plan": (c_int, [c_int, c_int, c_int, c_int, c_int, c_void_p]),
    "qspec_tp_argmax_combine": (c_int, [c_void_p, c_void_p, ctypes.c_longlong, c_int, c_void_p, c_void_p, c_void_p, c_int, c_int,
                                        c_int, c_int, c_void_p, c_void_p]),
    "qspec_sym_quant_i4": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_int, c_float, c_void_p]),
    "qspec_norm_quant_i8": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_float, c_void_p]),
    "qspec_sym_quant_i8": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_int, c_float, c_void_p]),
    "qspec_gemm_w4a8_workspace_bytes": (c_size_t, [c_int, c_int, c_int]),
    "qspec_gemm_w4a8": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int,
                                c_int, c_int, c_int, c_void_p, c_size_t, c_void_p]),
    "qspec_gemm_w4a8_acc_i32": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p,
                                        c_size_t, c_void_p]),
    "qspec_fht": (c_int, [c_void_p, c_void_p, c_int, c_int, c_float, c_int, c_void_p]),
    "qspec_hadamard_heads": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int,
                                     c_float, c_float, c_void_p]),
    "qspec_hadamard_k28": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int,
                                   c_float, c_float, c_void_p]),
    "qspec_gemm_w4a4_workspace_bytes": (c_size_t, [c_int, c_int, c_int]),
    "qspec_gemm_w4a4": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int,
                                c_int, c_int, c_int, c_void_p, c_size_t, c_void_p]),
    "qspec_gemm_w4a4_acc_i32": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p,
                                        c_size_t, c_void_p]),
    "qspec_gemm_w4a16_workspace_bytes": (c_size_t, [c_int, c_int, c_int]),
    "qspec_gemm_w4a16": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int,
                                 c_int, c_int, c_void_p, c_size_t, c_void_p]),
    "qspec_add": (c_int, [c_void_p, c_void_p, c_void_p, c_size_t, c_int, c_void_p]),
    "qspec_silu_mul": (c_int, [c_void_p, c_void_p, c_int, c_int, c_int, c_void_p]),
    "qspec_rope_kvcache": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int,
                                   c_int, c_int, c_int, c_void_p]),
    "qspec_decode_attention": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int,
                                       c_int, c_int, c_int, c_int, c_float, c_void_p]),
    "qspec_seq_attention_supported": (c_int, [c_int, c_int, c_int, c_int, c_int]),
    "qspec_seq_attention": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int,
                                    c_int, c_int, c_float, c_void_p]),
    "qspec_argmax_rows_workspace_bytes": (ctypes.c_size_t, [c_int]),
    "qspec_argmax_rows_static_max_rows": (c_int, []),
    "qspec_argmax_rows_static": (c_int, [c_void_p, c_int, c_int, ctypes.c_longlong, c_void_p, c_void_p, c_void_p]),
    "qspec_argmax_rows": (c_int, [c_void_p, c_int, c_int, ctypes.c_longlong, c_void_p, c_void_p, c_void_p, ctypes.c_size_t,
                                  c_void_p]),
    "qspec_hadamard_k108": (c_int, [c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_float, c_float,
                                    c_void_p]),
    "qspec_hadamard_heads40": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_float, c_float,
                                       c_void_p]),
    "qspec_rope_qkhad_kvcache": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int,
                                         c_int, c_int, c_float, c_void_p]),
    "qspec_attn_block_supported": (c_int, [c_int, c_int, c_int, c_int, c_int]),
    "qspec_attn_block": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                 c_void_p, c_int, c_int, c_int, c_int, c_int, c_float, c_float, c_float, c_void_p]),
}

# libqspec_b200_seq.so (include/qspec_b200_seq.h): the sequence-mixer kernels
c_ll = ctypes.c_longlong
SEQ_LIB_PATH = os.environ.get("QSPEC_SEQ_LIB") or os.path.join(_HERE, "_C", "libqspec_b200_seq.so")
DTYPE_F32 = 2
SEQ_SIGNATURES = {
    "qspec_last_error": (c_char_p, []),
    "qspec_launch_count": (c_uint64, []),
    "qspec_seq_embed": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p]),
    "qspec_seq_norm_conv": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_ll, c_ll, c_void_p, c_void_p, c_void_p, c_void_p,
                                    c_int, c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_float, c_void_p, c_int, c_void_p]),
    "qspec_seq_qk_norm": (c_int, [c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_float, c_int, c_void_p]),
    "qspec_seq_chunk_attention": (c_int, [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int,
                                          c_int, c_int, c_int, c_float, c_float, c_int, c_int, c_void_p]),
    "qspec_seq_cache_append": (c_int, [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int,
                                       c_int, c_void_p]),
    "qspec_seq_relu2": (c_int, [c_void_p, c_ll, c_int, c_void_p]),
    "qspec_moe_route": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p]),
    "qspec_moe_expert_tokens": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int,
                                        c_float, c_int, c_void_p]),
    "qspec_seq_argmax_rows": (c_int, [c_void_p, c_int, c_int, c_ll, c_void_p, c_int, c_void_p]),
    "qspec_seq_chunk_attention_mma_supported": (c_int, [c_int, c_int, c_int, c_int]),
    "qspec_seq_chunk_attention_mma": (c_int, [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int,
                                              c_int, c_int, c_int, c_float, c_float, c_void_p]),
    "qspec_moe_expert_grouped_supported": (c_int, [c_int, c_int]),
    "qspec_moe_grouped_workspace_bytes": (c_size_t, [c_int, c_int, c_int, c_int]),
    "qspec_moe_expert_grouped": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int,
                                         c_float, c_void_p, c_size_t, c_void_p]),
    "qspec_moe_route_chosen": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p]),
    "qspec_moe_expert_tokens_act": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int,
                                            c_float, c_int, c_int, c_void_p]),
    "qspec_moe_expert_grouped_act": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int,
                                             c_float, c_int, c_void_p, c_size_t, c_void_p]),
    "qspec_seq_token_shift": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p]),
    "qspec_seq_add_norm": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_ll, c_ll, c_void_p, c_void_p, c_void_p, c_int, c_void_p,
                                   c_int, c_int, c_float, c_int, c_int, c_void_p]),
    "qspec_seq_latent_prep": (c_int, [c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p,
                                      c_int, c_void_p, c_int, c_float, c_int, c_void_p]),
    "qspec_seq_rotary": (c_int, [c_void_p, c_ll, c_int, c_int, c_void_p, c_ll, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_int,
                                 c_int, c_void_p]),
    "qspec_seq_qkv_prep": (c_int, [c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int,
                                   c_void_p, c_int, c_float, c_int, c_void_p]),
    "qspec_seq_window_attention": (c_int, [c_void_p, c_int, c_void_p]),
    "qspec_seq_window_attention_mma": (c_int, [c_void_p, c_void_p, c_ll, c_int, c_int, c_int, c_void_p]),
    "qspec_seq_window_attention_mma_supported": (c_int, [c_int, c_int, c_int, c_int, c_int, c_int]),
    "qspec_seq_hgrn2": (c_int, [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int,
                                c_int, c_int, c_int, c_int, c_float, c_int, c_void_p]),
    "qspec_seq_side_gate": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p]),
    "qspec_seq_residual_norm": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_ll, c_ll, c_void_p, c_void_p, c_void_p, c_int, c_float,
                                        c_void_p, c_float, c_void_p, c_int, c_int, c_float, c_int, c_int, c_void_p]),
    "qspec_seq_latent_prep_pairing": (c_int, [c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p,
                                              c_void_p, c_int, c_void_p, c_int, c_float, c_int, c_void_p]),
    "qspec_seq_rotary_pairing": (c_int, [c_void_p, c_ll, c_int, c_int, c_void_p, c_ll, c_int, c_int, c_int, c_int, c_int, c_void_p,
                                         c_void_p, c_int, c_int, c_void_p]),
    "qspec_seq_act": (c_int, [c_void_p, c_ll, c_int, c_int, c_void_p]),
    "qspec_seq_silu_mul": (c_int, [c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_void_p]),
    "qspec_seq_lightning": (c_int, [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int,
                                    c_int, c_int, c_int, c_float, c_int, c_void_p]),
    "qspec_seq_prompt_attention_mma": (c_int, [c_void_p, c_void_p, c_ll, c_int, c_int, c_int, c_int, c_void_p]),
    "qspec_seq_prompt_attention_mma_supported": (c_int, [c_int, c_int, c_int]),
    "qspec_moe_route_grouped": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int,
                                        c_int, c_int, c_int, c_int, c_float, c_int, c_int, c_void_p]),
    "qspec_seq_residual_norm_scaled": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_ll, c_ll, c_void_p, c_void_p, c_void_p, c_int,
                                               c_float, c_void_p, c_void_p, c_float, c_void_p, c_int, c_int, c_float, c_int, c_int,
                                               c_void_p]),
    "qspec_seq_conv_act": (c_int, [c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p, c_int, c_void_p, c_int, c_int,
                                   c_void_p, c_int, c_int, c_void_p]),
    "qspec_seq_delta_rule": (c_int, [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p,
                                     c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_float,
                                     c_float, c_int, c_void_p]),
    "qspec_seq_selective_scan": (c_int, [c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p, c_int, c_void_p, c_int, c_void_p,
                                         c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int,
                                         c_void_p]),
    "qspec_seq_gqa_prep": (c_int, [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p,
                                   c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_int,
                                   c_void_p]),
    "qspec_seq_talking_attention": (c_int, [c_void_p, c_int, c_int, c_void_p]),
    "qspec_seq_glu_clamp": (c_int, [c_void_p, c_int, c_void_p, c_int, c_int, c_float, c_float, c_int, c_void_p]),
    "qspec_seq_scale_f32": (c_int, [c_void_p, c_ll, c_float, c_void_p]),
}


class WindowAttnArgs(ctypes.Structure):
    """qspec_window_attn_args of include/qspec_b200_seq.h."""
    _fields_ = [("qa", c_void_p), ("qa_tok_stride", c_ll), ("qa_head_stride", c_ll), ("DA", c_int),
                ("qb", c_void_p), ("qb_tok_stride", c_ll), ("qb_head_stride", c_ll), ("DB", c_int),
                ("k", c_void_p), ("k_slot_stride", c_ll), ("k_row_stride", c_int), ("k_head_stride", c_int),
                ("v", c_void_p), ("v_slot_stride", c_ll), ("v_row_stride", c_int), ("v_head_stride", c_int), ("DV", c_int),
                ("sink", c_void_p), ("gate", c_void_p), ("gate_ld", c_int),
                ("out", c_void_p), ("meta", c_void_p), ("ntok", c_int), ("H", c_int), ("G", c_int), ("window", c_int),
                ("cap", c_int), ("scale", c_float), ("gate_per_head", c_int)]



class TalkingAttnArgs(ctypes.Structure):
    """qspec_talking_attn_args of include/qspec_b200_seq.h."""
    _fields_ = [("q", c_void_p),
                ("k", c_void_p), ("k_slot_stride", c_ll), ("k_row_stride", c_int), ("k_head_stride", c_int),
                ("v", c_void_p), ("v_slot_stride", c_ll), ("v_row_stride", c_int), ("v_head_stride", c_int),
                ("talk", c_void_p), ("sink", c_void_p),
                ("out", c_void_p), ("meta", c_void_p), ("ntok", c_int), ("H", c_int), ("G", c_int), ("D", c_int), ("DV", c_int),
                ("window", c_int), ("cap", c_int), ("scale", c_float)]


_lib = None
_seq_lib = None


class QSpecNativeError(RuntimeError):
    """A C-ABI call returned a non-zero status (the reference raises RuntimeError via TORCH_CHECK)."""


def load() -> ctypes.CDLL:
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `python -m qspec_b200.build` "
            "(qspec_b200 has no CPU or PyTorch fallback for its kernels)")
    lib = ctypes.CDLL(LIB_PATH)
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)          # AttributeError if the header and the library drifted
        fn.restype = res
        fn.argtypes = args
    _lib = lib
    return lib


def load_seq() -> ctypes.CDLL:
    """The sequence-mixer library; like `load`, no fallback."""
    global _seq_lib
    if _seq_lib is not None:
        return _seq_lib
    if not os.environ.get("QSPEC_SEQ_LIB"):
        # a library older than its sources is rebuilt (20 s) rather than loaded: kernels and bindings must not drift apart
        from . import build
        try:
            build.build_seq_library()
        except Exception as e:  # no compiler or a read-only tree: an existing library is still the best there is
            if os.path.exists(SEQ_LIB_PATH):
                import warnings
                warnings.warn(f"{SEQ_LIB_PATH} may be older than its sources and could not be rebuilt: {e}")
    if not os.path.exists(SEQ_LIB_PATH):
        raise ImportError(
            f"{SEQ_LIB_PATH} is missing: build it with `python -m qspec_b200.build --seq` "
            "(qspec_b200 has no CPU or PyTorch fallback for its kernels)")
    lib = ctypes.CDLL(SEQ_LIB_PATH)
    for name, (res, args) in SEQ_SIGNATURES.items():
        fn = getattr(lib, name)
        fn.restype = res
        fn.argtypes = args
    _seq_lib = lib
    return lib


def check(status: int, what: str, lib=None) -> None:
    """Status 1/2 (bad argument / unsupported shape) -> ValueError, anything else -> QSpecNativeError."""
    if status == QSPEC_OK:
        return
    msg = (lib or load()).qspec_last_error()
    text = msg.decode() if msg else "?"
    if status in (1, 2):
        raise ValueError(f"{what}: {text} (status {status})")
    raise QSpecNativeError(f"{what}: {text} (status {status})")

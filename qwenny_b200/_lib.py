"""ctypes binding of libqwenny_b200.so (the C ABI declared in include/qwenny_b200.h).

There is no fallback: if the library has not been built (python -m qwenny_b200.build) loading raises, and every
entry point that computes needs a CUDA device.
"""
from __future__ import annotations

import ctypes as C
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libqwenny_b200.so")

P, I, LL, F = C.c_void_p, C.c_int, C.c_longlong, C.c_float

# name -> argument types (all return int unless listed in _RESTYPE)
SIGNATURES = {
    "qb_create": [I, C.POINTER(P)],
    "qb_destroy": [P],
    "qb_device_error": [P],
    "qb_sm_count": [P],
    "qb_version": [],
    "qb_set_pdl": [P, I],
    "qb_marlin_gemm": [P, P, P, P, P, P, I, I, I, I, I, P, P, I],
    "qb_marlin_early": [P, I],
    "qb_marlin_gemm_z": [P, P, P, P, P, P, I, I, I, I, I, P, P, I],
    "qb_marlin_gemm_noalloc": [P, P, P, P, P, I, I, I, I, I, P, P, I],
    "qb_static_scratch_bytes": [],
    "qb_static_device_error": [],
    "qb_gemm_f16_plain": [P, P, P, P, P, I, I, I, I, P, I],
    "qb_gemm_dec": [P, P, P, P, I, P, P, I, I, I, I, I, P, I, P],
    "qb_pack_i8": [P, I, I, P, I, P, P],
    "qb_mtp_in": [P, P, P, P, P, P, P, P, P, F, I],
    "qb_draft_pick": [P, P, P, P, I, P, P, I, I],
    "qb_lora_add": [P, P, P, I, I, P, I, P, P, P, I, P, I, I],
    "qb_lora_silu": [P, P, P, I, I, P, I, P, P, P, I, P, I, P, I],
    "qb_sample_rows": [P, P, P, I, I, I, I, P, P, P, P, P, P, P, P, P, P, P, P, P],
    "qb_host_sample_row": [P, I, P, P, P, I, P, P, P, I, P, P],
    "qb_draft_sample": [P, P, P, I, I, P, I, I, P, P, P, P, P, P, P, P, P, P],
    "qb_model_set_mtp": [P, P],
    "qb_model_draft": [P, P, P, I, P, P, I, I, P],
    "qb_model_kv_bytes": [P, I, I],
    "qb_model_save_kv": [P, P, I, I, I, P, C.c_size_t],
    "qb_model_load_kv": [P, P, I, I, I, P, C.c_size_t],
    "qb_model_state_bytes": [P],
    "qb_model_save_state": [P, P, I, P, C.c_size_t, P],
    "qb_model_load_state": [P, P, I, P, C.c_size_t, I],
    "qb_model_set_adapter": [P, I, P],
    "qb_model_set_slot_scale": [P, P, I, F],
    "qb_model_set_outputs": [P, P, I, P],
    "qb_model_sample": [P, P, P, I, P, P],
    "qb_model_draft_sampled": [P, P, P, I, P, P, I, I, P, P, P],
    "qb_model_draft_q": [P, P, I, I, P, P, P, P],
    "qb_embed": [P, P, P, P, P, P, I, I],
    "qb_embed_q8": [P, P, P, P, P, P, P, I, I],
    "qb_rmsnorm": [P, P, P, P, P, F, I],
    "qb_add_rmsnorm": [P, P, P, P, I, I, P, P, F],
    "qb_to_xin": [P, P, P, P, I],
    "qb_sum_parts": [P, P, P, I, I, I, P],
    "qb_mark_seen": [P, P, P, P, P, P, P, I, I],
    "qb_marlin_gather": [P, P, P, P, P, I, I],
    "qb_attn_prep": [P, P, P, I, I, P, P, P, F, P, P, P, P, P, P, P, P, I],
    "qb_attn_decode": [P, P, P, P, P, P, P, P, P, P, P, P, I, I, I, I, I, P, P, P, P],
    "qb_attn_dec_splits": [I],
    "qb_attn_dec_splits_sm": [I, I],
    "qb_attn_prefill": [P, P, P, P, P, P, P, P, P, P, I, I, I, P, P, P, P],
    "qb_attn_tile_splits": [I, I],
    "qb_delta_conv": [P, P, P, I, I, P, I, P, P, P, P, LL, P, P, P],
    "qb_delta_rule": [P, P, P, I, I, P, P, LL, P, P, P, P, P, P, I],
    "qb_delta_norm": [P, P, P, I, I, P, P, P, P, P, P, P, I],
    "qb_delta_mixer": [P, P, P, I, I, P, I, P, P, P, P, P, LL, P, P, P, P, P, P, P, I],
    "qb_model_use_fused": [P, I],
    "qb_model_create": [P, I, I, I, I, I, C.POINTER(P)],
    "qb_model_destroy": [P],
    "qb_model_set_layer": [P, I, P],
    "qb_model_set_head": [P, P, P, P, P],
    "qb_model_step": [P, P, P, I, P, I],
    "qb_model_upload": [P, P, P, I, P, I],
    "qb_model_step_marks": [P, P, P, I, P, I, P, P],
    "qb_model_upload_marks": [P, P, P, I, P, I, P, P],
    "qb_step_arrays": [P, I, P, I, P, P, I, I, I, P, P, P],
    "qb_step_ints": [],
    "qb_draft_vocab_create": [I, P, P, I, I, C.POINTER(P)],
    "qb_draft_vocab_load": [I, P, P, I, P, I, C.POINTER(P)],
    "qb_draft_vocab_destroy": [P],
    "qb_draft_vocab_rows": [P],
    "qb_draft_vocab_get": [P, P, P, I],
    "qb_draft_vocab_row_of": [P, C.c_uint32],
    "qb_draft_vocab_waiting": [P, C.c_uint32],
    "qb_draft_vocab_pending": [P],
    "qb_draft_vocab_dirty": [P],
    "qb_draft_vocab_saved": [P],
    "qb_draft_vocab_may_change": [P, P, I],
    "qb_draft_vocab_learn": [P, P, I, P, P, P],
    "qb_draft_ids_pt": [P, C.c_size_t, I, P, I, P],
    "qb_model_learn": [P, P, P, P, I, P, P, P, I, I, I, I, P],
    "qb_model_run": [P, P],
    "qb_model_use_graphs": [P, I],
    "qb_model_argmax": [P, P, P, I],
    "qb_model_logits": [P],
    "qb_model_hidden": [P],
    "qb_model_xn": [P],
    "qb_model_seen": [P],
    "qb_model_use_fork": [P, I],
    "qb_model_launches": [P],
    "qb_model_step_kernels": [P],
    "qb_pool_create": [I, C.POINTER(P)],
    "qb_pool_destroy": [P],
    "qb_pool_page": [P],
    "qb_pool_set_budget": [P, C.c_size_t],
    "qb_pool_fill": [P],
    "qb_pool_release": [P, C.c_size_t, P],
    "qb_pool_usage": [P, P, P],
    "qb_pool_available": [P],
    "qb_region_reserve": [P, C.c_size_t, C.POINTER(P)],
    "qb_region_ptr": [P],
    "qb_region_size": [P],
    "qb_region_is_mapped": [P, C.c_size_t, C.c_size_t],
    "qb_region_map": [P, P, C.c_size_t, C.c_size_t, P],
    "qb_region_unmap": [P, P, C.c_size_t, C.c_size_t],
    "qb_region_read": [P, P, C.c_size_t, P, C.c_size_t],
    "qb_region_write": [P, P, C.c_size_t, P, C.c_size_t],
    "qb_region_free": [P, P],
    "qb_row_order": [I, I, P],
    "qb_pack_marlin": [P, P, I, I, I, P, I, P, P],
    "qb_pack_marlin_z": [P, P, P, I, I, I, P, I, P, P],
    "qb_pack_f16": [P, I, I, P, I, P],
    "qb_split_for": [I, I, I, I],
    "qb_marlin_block": [P, P, P, I, I, I, I, P, P, P],
    "qb_marlin_put_block": [P, P, P, P, P, P, I, I, I, I, I, I],
    "qb_model_learn_block": [P, P, I, P, P, P, P],
    "qb_model_set_pool": [P, P],
    "qb_model_graph_stats": [P, P, P, P],
}
# measurement-only entry points (declared in csrc/measure.h, not part of the public header)
MEASURE_SIGNATURES = {
    "qb_marlin_tune": [P, I, I, I, I],
    "qb_marlin_trace": [P, P],
    "qb_marlin_probe": [P, I],
    "qb_attr_cache_selftest": [],
    "qb_graph_cache_selftest": [],
    "qb_model_fail_captures": [P, I],
    "qb_wait_probe": [P, P, C.c_uint],
}
_RESTYPE = {"qb_version": C.c_char_p, "qb_destroy": None, "qb_model_destroy": None, "qb_draft_vocab_destroy": None, "qb_model_logits": P,
            "qb_model_hidden": P, "qb_model_xn": P, "qb_model_seen": P, "qb_model_launches": LL, "qb_model_kv_bytes": C.c_size_t,
            "qb_model_state_bytes": C.c_size_t, "qb_pool_destroy": None, "qb_pool_page": C.c_size_t,
            "qb_pool_available": C.c_size_t, "qb_region_ptr": P, "qb_region_size": C.c_size_t}


class QbLayer(C.Structure):
    """qb_layer of include/qwenny_b200.h."""
    _fields_ = [
        ("kind", I),
        ("in_proj_w", P), ("in_proj_s", P), ("in_ba", P), ("out_w", P), ("out_s", P),
        ("input_norm", P), ("post_norm", P), ("gate_up_w", P), ("gate_up_s", P), ("down_w", P), ("down_s", P),
        ("conv_w", P), ("a_log", P), ("dt_bias", P), ("norm_w", P), ("mem", P), ("sst", LL), ("meta", P),
        ("q_norm", P), ("k_norm", P), ("inv_freq", P), ("kc", P), ("vc", P), ("ks", P), ("vs", P), ("cap", I),
    ]


class QbMtp(C.Structure):
    """qb_mtp of include/qwenny_b200.h."""
    _fields_ = [
        ("layer", QbLayer), ("fc_w", P), ("fc_s", P), ("pre_e", P), ("pre_h", P), ("norm", P), ("head_w", P),
        ("head_s", P), ("head_rows", I), ("head_valid", I), ("head_ids", P), ("head_zero_points", I),
    ]


class QbLoraProd(C.Structure):
    """qb_lora_prod of include/qwenny_b200.h."""
    _fields_ = [("a", P), ("a_tiles", I), ("b", P), ("tab", P), ("b2", P), ("tab2", P)]


class QbLoraLayer(C.Structure):
    """qb_lora_layer of include/qwenny_b200.h."""
    _fields_ = [("rank", I), ("inp", QbLoraProd), ("out", QbLoraProd), ("gate_up", QbLoraProd), ("down", QbLoraProd)]


class QbTok(C.Structure):
    _fields_ = [("id", C.c_uint32), ("slot", C.c_uint32), ("pos", C.c_uint32)]

_lib = None


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                f"{LIB_PATH} is missing: build it with `python -m qwenny_b200.build` (there is no CPU fallback)")
        _lib = C.CDLL(LIB_PATH)
        for name, args in list(SIGNATURES.items()) + list(MEASURE_SIGNATURES.items()):
            fn = getattr(_lib, name)
            fn.argtypes = args
            fn.restype = _RESTYPE.get(name, I)
    return _lib


class QbError(RuntimeError):
    pass


def check(rc: int, what: str) -> None:
    if rc != 0:
        raise QbError(f"{what} failed with code {rc}")

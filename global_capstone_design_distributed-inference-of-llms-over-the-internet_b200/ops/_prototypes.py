"""ctypes prototypes for the non-GEMM entry points of libb200petals.so."""
from __future__ import annotations

import ctypes as C

vp, i32, i64, f32 = C.c_void_p, C.c_int32, C.c_int64, C.c_float


from .native import LLChainArgs as _LLChainArgs  # noqa: E402


class AttnDecodeArgs(C.Structure):
    """Mirror of ``b200_attn_decode_args``."""

    _fields_ = [
        ("qkv", vp), ("out", vp), ("kv_ptrs", vp), ("pos", vp), ("inv_freq", vp), ("scratch", vp),
        ("counters", vp),
        ("T", i32), ("n_heads", i32), ("n_kv_heads", i32), ("head_dim", i32), ("s_max", i32),
        ("splits", i32), ("ldqkv", i32), ("ldo", i32),
        ("scale", f32), ("dtype", i32), ("pdl", i32), ("ll_scratch", vp), ("chain", _LLChainArgs),
    ]


class SampleRow(C.Structure):
    """Mirror of ``b200::SampleRow`` (csrc/sampling.cu)."""

    _fields_ = [("temperature", f32), ("top_p", f32), ("penalty", f32), ("top_k", i32), ("n_recent", i32),
                ("recent", i32 * 50)]


class HopArgs(C.Structure):
    """Mirror of ``b200_hop_args``."""

    _fields_ = [("x", vp), ("extra", vp), ("ring", vp), ("counter", vp),
                ("T", i32), ("hidden", i32), ("ldx", i32), ("n_extra", i32),
                ("depth", i32), ("t_max", i32), ("pairs_per_token", i32), ("timeout_ms", i32), ("pdl", i32)]


class AddNormArgs(C.Structure):
    """Mirror of ``b200_add_norm_args``."""

    _fields_ = [("x", vp), ("add_a", vp), ("add_b", vp), ("pair_y", vp), ("pair_w", vp), ("gain", vp), ("out", vp),
                ("T", i32), ("width", i32), ("ldx", i32), ("lda", i32), ("ldb", i32), ("ldp", i32), ("top", i32),
                ("ldo", i32), ("out_dtype", i32), ("eps", f32), ("gain_offset", f32), ("pdl", i32), ("add_scale", f32)]


class SimtGemmArgs(C.Structure):
    """Mirror of ``b200_simt_gemm_args``."""

    _fields_ = [("x", vp), ("w", vp), ("w2", vp), ("out", vp), ("row_src", vp), ("row_dst", vp), ("group_off", vp),
                ("row_scale", vp),
                ("T", i32), ("N", i32), ("K", i32), ("ldx", i32), ("ldw", i32), ("ldo", i32),
                ("x_dtype", i32), ("w_dtype", i32), ("out_dtype", i32), ("batch", i32), ("groups", i32),
                ("x_bs", i64), ("w_bs", i64), ("o_bs", i64), ("w_gs", i64), ("pdl", i32), ("reserved", i32)]


class LatentArgs(C.Structure):
    """Mirror of ``b200_latent_args``."""

    _fields_ = [("proj", vp), ("ldp", i32), ("q_off", i32), ("kv_off", i32), ("c_gain", vp), ("inv_freq", vp),
                ("cache", vp), ("kv_ptrs", vp), ("pos", vp), ("kv_ptr_stride", i32), ("pos0", i32),
                ("T", i32), ("heads", i32), ("dim", i32), ("rot", i32), ("rot_dims", i32), ("kv_rank", i32),
                ("row_elems", i32), ("cache_dtype", i32), ("eps", f32),
                ("q_abs", vp), ("out", vp), ("ldqa", i32), ("ldout", i32), ("window", i32), ("scale", f32),
                ("pdl", i32), ("reserved", i32)]


class SinkAttnArgs(C.Structure):
    """Mirror of ``b200_sink_attn_args``."""

    _fields_ = [("proj", vp), ("ldp", i32), ("q_off", i32), ("k_off", i32), ("v_off", i32), ("g_off", i32),
                ("bias", vp), ("q_gain", vp), ("k_gain", vp), ("temp", vp), ("vmix", vp), ("v_first", vp),
                ("ldvf", i32), ("vmix_mode", i32), ("k_cache", vp), ("v_cache", vp), ("kv_ptrs", vp), ("pos", vp),
                ("kv_ptr_stride", i32), ("pos0", i32),
                ("T", i32), ("heads", i32), ("kv_heads", i32), ("dim", i32), ("vdim", i32), ("row_elems", i32),
                ("cache_dtype", i32), ("eps", f32), ("scale", f32), ("sink", f32), ("out", vp), ("ldo", i32),
                ("out_dtype", i32), ("pdl", i32), ("ldq16", i32), ("q16", vp)]


class DeltaArgs(C.Structure):
    """Mirror of ``b200_delta_args``."""

    _fields_ = [("proj", vp), ("ldp", i32), ("c_off", i32), ("b_off", i32), ("a_off", i32), ("conv_w", vp), ("A_log", vp),
                ("dt_bias", vp), ("work", vp), ("ldw", i32), ("state", vp), ("state_ptrs", vp), ("state_ptr_stride", i32),
                ("reserved0", i32), ("state_off", i64), ("pos", vp), ("pos0", i32), ("n_seq", i32), ("seq_len", i32),
                ("heads", i32), ("kv_heads", i32), ("dim", i32), ("vdim", i32), ("taps", i32), ("unit_eps", f32),
                ("o", vp), ("ldo", i32), ("pdl", i32)]


PROTOTYPES = [
    ("b200_embed_pos_f32", [vp, vp, vp, i32, vp, i32, vp, i32, i32, i32, i32, i32, i32, vp], C.c_int),
    ("b200_xielu", [vp, i32, vp, f32, f32, vp, i32, i32, i32, i32, i32, vp], C.c_int),
    ("b200_sink_attn_append", [C.POINTER(SinkAttnArgs), vp], C.c_int),
    ("b200_sink_attn", [C.POINTER(SinkAttnArgs), i32, vp, vp], C.c_int),
    ("b200_sink_attn_prefill", [C.POINTER(SinkAttnArgs), vp], C.c_int),
    ("b200_sink_attn_scratch_bytes", [i32, i32, i32, i32], i64),
    ("b200_delta_prep", [C.POINTER(DeltaArgs), vp], C.c_int),
    ("b200_delta_rule", [C.POINTER(DeltaArgs), vp], C.c_int),
    ("b200_head_gate", [vp, i32, i32, vp, i32, i32, i32, i32, i32, vp], C.c_int),
    ("b200_attn_prefill_tc_rows", [vp, vp, vp, vp, i32, i32, i32, i32, i32, i32, i32, i32, f32, i32, i64, i64, i32, vp], C.c_int),
    ("b200_gated_head_norm", [vp, i32, vp, i32, vp, vp, i32, i32, i32, i32, i32, f32, i32, vp], C.c_int),
    ("b200_embed_f32", [vp, vp, i32, vp, i32, i32, i32, i32, i32, vp], C.c_int),
    ("b200_add_rms_norm", [C.POINTER(AddNormArgs), vp], C.c_int),
    ("b200_glu_clamp", [vp, vp, i32, vp, i32, i32, i32, i32, f32, f32, f32, i32, vp], C.c_int),
    ("b200_gemm_simt", [C.POINTER(SimtGemmArgs), vp], C.c_int),
    ("b200_latent_rope_append", [C.POINTER(LatentArgs), vp], C.c_int),
    ("b200_latent_attn", [C.POINTER(LatentArgs), vp], C.c_int),
    ("b200_latent_attn_split", [C.POINTER(LatentArgs), i32, vp, vp], C.c_int),
    ("b200_latent_attn_scratch_bytes", [i32, i32, i32, i32], i64),
    ("b200_latent_attn_prefill", [vp, i32, i32, vp, i32, i32, vp, i32, i32, vp, i32, i32, i32, i32, i32, i32, i32, i32, i32,
                                  f32, i32, i32, vp], C.c_int),
    ("b200_moe_route", [vp, i32, i32, i32, i32, i32, i32, i32, vp, vp, i32, vp], C.c_int),
    ("b200_moe_plan", [vp, i32, i32, i32, vp, vp, vp, i32, vp], C.c_int),
    ("b200_moe_scale", [vp, i32, i32, vp, vp, i32, i32, i32, i32, i32, vp], C.c_int),
    ("b200_hop_ring_bytes", [i32, i32, i32], i64),
    ("b200_hop_send", [C.POINTER(HopArgs), vp], C.c_int),
    ("b200_hop_recv", [C.POINTER(HopArgs), vp], C.c_int),
    ("b200_hop_init", [], C.c_int),
    ("b200_ll_publish", [vp, i32, vp, i32, i32, i32, vp, i32, i32, vp], C.c_int),
    ("b200_trace_set", [vp, i32], C.c_int),
    ("b200_argmax_partial", [vp, i32, i32, i32, vp, vp, vp, vp, i32, i32, vp, vp, i32, vp], C.c_int),
    ("b200_sample_row_bytes", [], i32),
    ("b200_sample", [vp, i32, i32, i32, vp, vp, vp, vp, i32, vp], C.c_int),
    ("b200_sample_state_bytes", [], i32),
    ("b200_sample_stateful", [vp, i32, i32, i32, vp, vp, vp, vp, vp, i32, vp], C.c_int),
    ("b200_gemm_static_scratch", [vp, vp], C.c_int),
    ("b200_attn_decode", [C.POINTER(AttnDecodeArgs), vp], C.c_int),
    ("b200_attn_decode_scratch_bytes", [i32, i32, i32, i32], i64),
    ("b200_rope_append", [vp, vp, vp, vp, i32, i32, i32, i32, i32, i32, i32, i32, i32, vp], C.c_int),
    ("b200_attn_prefill", [vp, vp, vp, vp, i32, i32, i32, i32, i32, i32, i32, i32, f32, i32, i32, vp], C.c_int),
    ("b200_attn_prefill_tc", [vp, vp, vp, vp, i32, i32, i32, i32, i32, i32, i32, i32, f32, i32, i32, vp], C.c_int),
    ("b200_embed", [vp, vp, i32, vp, vp, vp, i32, i32, i32, i32, i32, i32, vp], C.c_int),
    ("b200_norm", [vp, vp, vp, vp, i32, i32, i32, i32, f32, i32, i32, i32, vp], C.c_int),
    ("b200_rms_rstd", [vp, vp, i32, i32, i32, f32, i32, i32, vp], C.c_int),
    ("b200_argmax", [vp, i32, i32, i32, vp, vp, vp, vp, i32, i32, vp], C.c_int),
]


def register(L) -> None:
    for name, args, res in PROTOTYPES:
        fn = getattr(L, name, None)
        if fn is None:  # older build without this entry point
            continue
        fn.argtypes = args
        fn.restype = res

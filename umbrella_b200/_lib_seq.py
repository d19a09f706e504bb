"""ctypes binding of libumbrella_b200_seq.so (the C ABI declared in include/umbrella_b200_seq.h): the batched step
of the sequence-state decoders and its building blocks.

The library is compiled in-tree on first use when it is missing or older than its sources (``build.build_seq``: eight
small translation units, seconds) -- a fresh checkout serves these models without a separate build step.  There is
no PyTorch / CPU fallback behind these calls: without nvcc and without the library, loading is an error.
"""
from __future__ import annotations

import ctypes as C
import os

from ._lib import c_float, c_int, c_int64, c_size_t, c_void_p

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libumbrella_b200_seq.so")

UMBS_BF16, UMBS_F32 = 0, 1
UMBS_MIX_RETENTION, UMBS_MIX_LATENT_ATTENTION, UMBS_MIX_CACHED_ATTENTION, UMBS_MIX_MLSTM, UMBS_MIX_TIME_MIX = 0, 1, 2, 3, 4
UMBS_FORM_PARALLEL, UMBS_FORM_PRENORM = 0, 1
UMBS_ACT_CLAMPED_GLU, UMBS_ACT_GELU_TANH, UMBS_ACT_SILU = 1, 2, 3
UMBS_NORM_RMS, UMBS_NORM_LAYER, UMBS_NORM_DYT = 0, 1, 2
UMBS_UNARY_TANH, UMBS_UNARY_XIELU = 1, 2
UMBS_ROUTE_SOFTMAX_TOP, UMBS_ROUTE_SIGMOID_GROUPS, UMBS_ROUTE_SOFTMAX_ALL = 0, 1, 2
UMBS_ATTN_SOFTMAX, UMBS_ATTN_SOFTMAX_SINK, UMBS_ATTN_SIGMOID = 0, 1, 2


class Batch(C.Structure):
    _fields_ = [("n_tokens", c_int), ("n_seqs", c_int), ("n_want", c_int), ("max_seq_len", c_int),
                ("tok_ids", c_void_p), ("tok_seq", c_void_p), ("tok_pos", c_void_p), ("seq_slot", c_void_p),
                ("seq_start", c_void_p), ("seq_len", c_void_p), ("seq_pos0", c_void_p), ("seq_parity", c_void_p),
                ("want_rows", c_void_p), ("max_pos0", c_int)]


class Mlp(C.Structure):
    _fields_ = [("experts", c_int), ("top", c_int), ("ff", c_int), ("limit", c_float), ("w_router", c_void_p),
                ("w_gu", c_void_p), ("w_down", c_void_p), ("shared_ff", c_int), ("shared_limit", c_float),
                ("ws_gu", c_void_p), ("ws_down", c_void_p), ("act", c_int), ("route_mode", c_int), ("groups", c_int),
                ("keep", c_int), ("bias_gu", c_void_p), ("bias_down", c_void_p), ("w_shared_gate", c_void_p),
                ("route_scale", c_float), ("plain", c_int), ("unary", c_int), ("unary_p0", c_float), ("unary_p1", c_float)]


class Delta(C.Structure):
    _fields_ = [("delta", c_void_p), ("pair_out", c_void_p), ("sel_w", c_void_p), ("pair_pos", c_void_p), ("top", c_int),
                ("shared", c_void_p), ("shared_gate", c_void_p), ("scale", c_void_p), ("mult", c_float),
                ("delta_mult", c_float), ("delta2", c_void_p), ("delta2_mult", c_float)]


class Layer(C.Structure):
    pass


Layer._fields_ = [("mixer", c_int), ("heads", c_int), ("dim", c_int), ("vdim", c_int),
                ("rot_dims", c_int), ("inv_freq", c_void_p), ("decay", c_void_p), ("ret_state", c_void_p),
                ("q_rank", c_int), ("kv_rank", c_int), ("window", c_int), ("ring_len", c_int), ("scale", c_float),
                ("q_norm", c_void_p), ("kv_norm", c_void_p), ("w_uq", c_void_p), ("w_ukT", c_void_p), ("w_uv", c_void_p),
                ("w_ukv", c_void_p), ("ring", c_void_p),
                ("w_in", c_void_p), ("w_o", c_void_p), ("norm_w", c_void_p), ("shift_w", c_void_p),
                ("shift_state", c_void_p), ("depth_w", c_void_p), ("has_mlp", c_int), ("mlp", Mlp),
                ("form", c_int), ("norm_offset", c_float), ("norm2_w", c_void_p),
                ("kv_heads", c_int), ("attn_mode", c_int), ("gate_kind", c_int), ("values_are_keys", c_int), ("pool", c_int),
                ("taps", c_int), ("rot_mag", c_float), ("gate_cap", c_float), ("bias_in", c_void_p), ("conv_w", c_void_p),
                ("head_bias", c_void_p), ("out_norm_w", c_void_p), ("kv_cache", c_void_p), ("kv_len", c_int),
                ("pool_cache", c_void_p), ("pool_len", c_int), ("conv_state", c_void_p), ("mlstm_state", c_void_p),
                ("norm_kind", c_int), ("norm_b", c_void_p), ("norm2_b", c_void_p), ("out_scale", c_void_p),
                ("out_scale2", c_void_p), ("residual_mult", c_float), ("rope_dim", c_int), ("sink", c_void_p),
                ("norm_alpha", c_float), ("norm2_alpha", c_float), ("softcap", c_float), ("dist_r1", c_void_p),
                ("dist_r2", c_void_p), ("talk", c_void_p), ("chunk", c_int), ("maps", c_int), ("diff_lambda", c_float),
                ("head_unit_norm", c_int), ("out_mult", c_float), ("q_norm_w", c_void_p), ("k_norm_w", c_void_p),
                ("kv_from", c_int), ("mix_mu", c_void_p), ("decay_rank", c_int), ("w_decay1", c_void_p),
                ("w_decay2", c_void_p), ("decay_bias", c_void_p), ("bonus", c_void_p), ("tm_state", c_void_p),
                ("second", C.POINTER(Layer)), ("mix_scale", c_float), ("second_scale", c_float)]


class Model(C.Structure):
    _fields_ = [("dtype", c_int), ("width", c_int), ("vocab", c_int), ("n_layers", c_int), ("norm_groups", c_int),
                ("slots", c_int), ("norm_eps", c_float), ("embed", c_void_p), ("final_norm", c_void_p), ("head", c_void_p),
                ("layers", C.POINTER(Layer)), ("norm_offset", c_float), ("logit_softcap", c_float),
                ("embed_scale", c_float), ("norm_kind", c_int), ("final_norm_b", c_void_p), ("final_norm_alpha", c_float),
                ("pos_freq", c_void_p)]


class AttnOpts(C.Structure):
    _fields_ = [("softcap", c_float), ("dist_r1", c_void_p), ("dist_r2", c_void_p), ("chunk", c_int), ("maps", c_int),
                ("value_heads", c_int), ("raw_out", c_void_p)]


_BP = C.POINTER(Batch)
# name -> (restype, argtypes); lists every symbol include/umbrella_b200_seq.h declares
SIGNATURES = {
    "umbs_version": (C.c_char_p, []),
    "umbs_launch_count": (C.c_ulonglong, []),
    "umbs_workspace_bytes": (c_size_t, [C.POINTER(Model), c_int, c_int]),
    "umbs_forward": (c_int, [C.POINTER(Model), _BP, c_void_p, c_void_p, c_void_p, c_size_t, c_void_p]),
    "umbs_gemm": (c_int, [c_int, c_void_p, c_int64, c_int, c_void_p, c_int64, c_int64, c_void_p, c_int64, c_int, c_int,
                          c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_int, c_float, c_void_p]),
    "umbs_gemm_ex": (c_int, [c_int, c_void_p, c_int64, c_int, c_void_p, c_int64, c_int64, c_void_p, c_int64, c_int, c_int,
                             c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_int, c_float, c_void_p, c_void_p, c_int64, c_int,
                             c_void_p]),
    "umbs_group_norm_shift": (c_int, [c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int, _BP, c_int, c_int, c_float,
                                      c_void_p, c_void_p, c_void_p]),
    "umbs_group_norm_rows": (c_int, [c_int, c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_float, c_void_p, c_void_p]),
    "umbs_retention": (c_int, [c_int, c_void_p, c_int64, _BP, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_float,
                               c_void_p, c_void_p, c_void_p, c_void_p, c_size_t, c_void_p, c_void_p]),
    "umbs_latent_norm": (c_int, [c_int, c_void_p, c_int, c_int, c_int, c_void_p, c_void_p, c_float, c_void_p, c_void_p,
                                 c_void_p]),
    "umbs_latent_attention": (c_int, [c_int, c_void_p, c_void_p, c_void_p, c_int, _BP, c_int, c_int, c_int, c_float,
                                      c_void_p, c_size_t, c_void_p, c_void_p]),
    "umbs_latent_attention_ex": (c_int, [c_int, c_void_p, c_void_p, c_void_p, c_int, _BP, c_int, c_int, c_int, c_int, c_float,
                                         c_int, c_void_p, c_void_p, c_size_t, c_void_p, c_void_p]),
    "umbs_latent_prep": (c_int, [c_int, c_void_p, c_int64, _BP, c_int, c_int, c_int, c_int, c_void_p, c_float, c_int, c_void_p,
                                 c_float, c_void_p, c_void_p, c_void_p, c_int64, c_void_p]),
    "umbs_window_attention_fits": (c_int, [c_int, c_int]),
    "umbs_window_attention": (c_int, [c_int, c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_int64, _BP, c_int, c_int,
                                      c_int, c_int, c_float, c_void_p, c_int64, c_void_p]),
    "umbs_window_attention_ex_fits": (c_int, [c_int, c_int, c_int]),
    "umbs_window_attention_ex": (c_int, [c_int, c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_int64, c_int, c_void_p,
                                         c_int64, _BP, c_int, c_int, c_int, c_int, c_float, c_int, c_void_p, c_void_p,
                                         c_int64, c_void_p, c_int64, c_void_p]),
    "umbs_ring_append": (c_int, [c_int, c_void_p, c_void_p, c_int, _BP, c_int, c_void_p]),
    "umbs_moe_route": (c_int, [c_int, c_void_p, c_int, c_int, c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p,
                               c_void_p, c_void_p, c_void_p]),
    "umbs_moe_route_ex": (c_int, [c_int, c_void_p, c_int, c_int, c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p,
                                  c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p]),
    "umbs_token_gate": (c_int, [c_int, c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p]),
    "umbs_depth_mix": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int,
                               c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p]),
    "umbs_add_rms_norm": (c_int, [c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_float, c_int, c_float, c_void_p,
                                  c_void_p, c_void_p]),
    "umbs_add_norm": (c_int, [c_int, c_void_p, C.POINTER(Delta), c_void_p, c_int, c_int, c_void_p, c_void_p, c_float, c_int,
                              c_float, c_void_p, c_void_p, c_void_p]),
    "umbs_softcap": (c_int, [c_void_p, c_int64, c_float, c_void_p]),
    "umbs_attention_prep": (c_int, [c_int, c_void_p, c_int64, c_void_p, _BP, c_int, c_int, c_int, c_int, c_int, c_int,
                                    c_void_p, c_void_p, c_int, c_int, c_void_p, c_float, c_void_p, c_void_p, c_void_p]),
    "umbs_kv_pool": (c_int, [c_int, c_void_p, c_void_p, c_int, c_void_p, c_int, _BP, c_int, c_int, c_void_p]),
    "umbs_cached_attention": (c_int, [c_int, c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, _BP, c_int, c_int,
                                      c_int, c_int, c_int, c_int, c_float, c_void_p, c_void_p, c_int64, c_int, c_void_p,
                                      c_size_t, c_void_p, c_void_p]),
    "umbs_mlstm": (c_int, [c_int, c_void_p, c_int64, c_void_p, _BP, c_int, c_int, c_int, c_float, c_float, c_void_p,
                           c_void_p, c_void_p, c_void_p, c_void_p, c_size_t, c_void_p, c_void_p]),
    "umbs_add_norm_ex": (c_int, [c_int, c_void_p, C.POINTER(Delta), c_void_p, c_int, c_int, c_void_p, c_void_p, c_float, c_float,
                                 c_int, c_float, c_void_p, c_void_p, c_void_p]),
    "umbs_attention_prep_ex": (c_int, [c_int, c_void_p, c_int64, c_void_p, _BP, c_int, c_int, c_int, c_int, c_int, c_int,
                                       c_void_p, c_void_p, c_int, c_int, c_void_p, c_float, c_int, c_void_p, c_void_p, c_float,
                                       c_void_p, c_void_p, c_void_p]),
    "umbs_cached_attention_ex": (c_int, [c_int, c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, _BP, c_int, c_int,
                                         c_int, c_int, c_int, c_int, c_float, c_void_p, c_void_p, c_int64, c_int,
                                         C.POINTER(AttnOpts), c_void_p, c_size_t, c_void_p, c_void_p]),
    "umbs_attention_finish": (c_int, [c_int, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p, c_float, c_int,
                                      c_float, c_float, c_void_p, c_int64, c_void_p, c_void_p]),
    "umbs_shift_mix": (c_int, [c_int, c_void_p, c_void_p, c_int, c_void_p, c_int, _BP, c_int, c_void_p, c_void_p]),
    "umbs_time_mix": (c_int, [c_int, c_void_p, c_int64, c_void_p, c_void_p, c_void_p, _BP, c_int, c_int, c_float, c_void_p,
                              c_void_p, c_void_p, c_void_p, c_void_p]),
    "umbs_gemm_unary": (c_int, [c_int, c_void_p, c_int64, c_int, c_void_p, c_int64, c_int64, c_void_p, c_int64, c_int, c_int,
                                c_int, c_int, c_int, c_int, c_void_p, c_int, c_float, c_float, c_void_p]),
    "umbs_moe_route_scaled": (c_int, [c_int, c_void_p, c_int, c_int, c_void_p, c_int, c_int, c_int, c_int, c_int, c_float,
                                      c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p]),
    "umbs_embedding_pos": (c_int, [c_int, c_void_p, c_void_p, c_void_p, c_float, c_void_p, c_void_p, c_int, c_int, c_void_p]),
    "umbs_embedding": (c_int, [c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p]),
    "umbs_embedding_scaled": (c_int, [c_int, c_void_p, c_void_p, c_float, c_void_p, c_int, c_int, c_void_p]),
}

_lib = None


def load() -> C.CDLL:
    """Load the library (once), compiling it first when it is missing or stale and nvcc is there."""
    global _lib
    if _lib is not None:
        return _lib
    from . import build
    try:
        build.build_seq()
    except RuntimeError:
        if not os.path.exists(LIB_PATH):
            raise
    lib = C.CDLL(LIB_PATH)
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)
        fn.restype = res
        fn.argtypes = args
    _lib = lib
    return lib


def check(rc: int, what: str = "") -> None:
    if rc != 0:
        from . import _lib as core
        msg = {-1: "invalid argument", -2: "shape or option not supported", -3: "workspace too small"}.get(rc)
        if msg is None:
            try:
                msg = core.load().umb_error_string(rc).decode()
            except Exception:
                msg = "CUDA error"
        raise RuntimeError(f"umbrella_b200_seq {what} failed: status {rc} ({msg})")

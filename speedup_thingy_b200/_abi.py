"""ctypes binding of ``include/rte_b200.h`` (the C ABI of ``lib/librte_b200.so``).

The library is the product's only compute path: if it is missing or a symbol is absent the import
of this module's ``load()`` raises -- there is no CPU or PyTorch fallback.
"""
from __future__ import annotations

import ctypes as C
from pathlib import Path

LIB_PATH = Path(__file__).resolve().parent / "lib" / "librte_b200.so"

c_i32, c_i64, c_f32, c_vp = C.c_int32, C.c_int64, C.c_float, C.c_void_p

EPI_BF16, EPI_F32, EPI_SWIGLU_FWD, EPI_SWIGLU_BWD = 0, 1, 2, 3
ROUTER_MAX_R, ROUTER_MAX_K, ROUTER_MAX_T = 32, 8, 128
ROUTER_DPOOLED_PARTS = 4
ADAMW_CHUNK = 4096


class GemmArgs(C.Structure):
    _fields_ = [
        ("M", c_i32), ("N", c_i32), ("K", c_i32),
        ("A", c_vp), ("lda", c_i32), ("a_mn_major", c_i32),
        ("B", c_vp), ("ldb", c_i32), ("b_mn_major", c_i32),
        ("epilogue", c_i32),
        ("C", c_vp), ("ldc", c_i32),
        ("R", c_vp), ("ldr", c_i32),
        ("C2", c_vp), ("ldc2", c_i32),
        ("b_pair_offset", c_i32),
        ("splits", c_i32),
        ("split_stride", c_i64),
        ("max_ctas", c_i32),
        ("status", c_vp),
        ("tile_group", c_vp),
        ("n_groups", c_i32),
        ("b_group_stride", c_i32),
        ("split_kblocks", c_vp),
        ("tile_n", c_i32),
        ("cta_pair", c_i32),
        ("split_counters", c_vp),
        ("split_out", c_vp),
        ("split_accumulate", c_i32),
    ]


class RouterWeights(C.Structure):
    _fields_ = [(n, c_vp) for n in ("r_w0", "r_b0", "r_w2", "r_b2", "d_w0", "d_b0", "d_w2", "d_b2", "pass_recipe_bias")]


class RouterOut(C.Structure):
    _fields_ = [(n, c_vp) for n in ("pooled", "r_hidden_pre", "d_hidden_pre", "recipe_logits", "recipe_probs",
                                    "depth_probs", "expected_depth", "router_entropy", "recipe_id",
                                    "recipe_id_by_pass", "depth_id", "depth")]


class RouterGrads(C.Structure):
    _fields_ = [(n, c_vp) for n in ("r_w0", "r_b0", "r_w2", "r_b2", "d_w0", "d_b0", "d_w2", "d_b2")]


class PhiParams(C.Structure):
    _fields_ = [(n, c_vp) for n in ("gain", "v", "u", "bias", "scale", "wt")] + [("n_keys", C.c_int32)]


class PhiGrads(C.Structure):
    _fields_ = [(n, c_vp) for n in ("gain", "v", "u", "bias")]


class AdamWTensor(C.Structure):
    _fields_ = [("p", c_vp), ("g", c_vp), ("m", c_vp), ("v", c_vp), ("bf16_shadow", c_vp),
                ("n", c_i64), ("lr_group", c_i32), ("step_slot", c_i32)]


COMM_MAX_RANKS, COMM_MAX_SLOTS, IPC_HANDLE_BYTES = 8, 64, 64


class PeerComm(C.Structure):
    _fields_ = [("buf", c_vp * COMM_MAX_RANKS), ("stage", c_vp * COMM_MAX_RANKS), ("flags", c_vp * COMM_MAX_RANKS),
                ("epoch", c_vp), ("done_count", c_vp),
                ("world", c_i32), ("rank", c_i32)]


class AuditSampleParams(C.Structure):
    _fields_ = [(n, C.c_float) for n in ("p_min", "p_max", "alpha", "beta", "gamma", "coverage_min", "coverage_beta",
                                         "inv_r_plus_k", "w0")] + \
               [(n, c_i32) for n in ("B", "R", "cap", "n_cap", "weight_mode")]


class AdamWExtras(C.Structure):
    _fields_ = [("skip", c_vp), ("metric_partial", c_vp), ("metric_group", c_vp), ("metric_out", c_vp),
                ("n_metric_groups", c_i32), ("absent_flag", c_vp), ("absent_mask", c_vp)]


P = C.POINTER

# name -> (restype, argtypes); mirrors include/rte_b200.h declaration by declaration
PROTOTYPES = {
    "rte_backend_name": (C.c_char_p, []),
    "rte_status_string": (C.c_char_p, [C.c_int]),
    "rte_device_sm_count": (C.c_int, []),
    "rte_gemm_bf16": (C.c_int, [P(GemmArgs), c_vp]),
    "rte_gemm_bf16_small": (C.c_int, [P(GemmArgs), c_vp]),
    "rte_gemm_tile_plan": (C.c_int, [P(GemmArgs), P(c_i32), P(c_i32), P(c_i32)]),
    "rte_reduce_splits": (C.c_int, [c_vp, c_i32, c_i64, c_i64, c_vp, c_i32, c_vp]),
    "rte_embed_fwd": (C.c_int, [c_vp, c_vp, c_vp, c_i32, c_i32, c_i32, c_vp, c_vp]),
    "rte_embed_bwd": (C.c_int, [c_vp, c_vp, c_vp, c_vp, c_i32, c_i32, c_i32, c_vp, c_vp]),
    "rte_rmsnorm_fwd": (C.c_int, [c_vp, c_vp, c_vp, c_vp, c_vp, c_vp, c_vp, c_i32, c_i32, c_f32, c_vp]),
    "rte_rmsnorm_bwd": (C.c_int, [c_vp] * 12 + [c_i32, c_i32, c_i32, P(c_i32), c_vp]),
    "rte_rmsnorm_bwd_splits": (C.c_int, [c_vp] * 6 + [c_i32, c_i64] + [c_vp] * 6 + [c_i32, c_i32, c_i32, P(c_i32), c_vp]),
    "rte_residual_rmsnorm_fwd_splits": (C.c_int, [c_vp, c_vp, c_i32, c_i64, c_vp, c_vp, c_vp, c_vp, c_i32, c_vp, c_vp, c_vp, c_vp,
                                                  c_vp, c_vp, c_vp, c_vp, c_vp, c_i32, c_i32, C.c_float, c_vp]),
    "rte_colsum_partials3": (C.c_int, [c_vp, c_vp, c_vp, c_i32, c_i32, c_i32, c_vp]),
    "rte_colsum_partials": (C.c_int, [c_vp, c_i32, c_i32, c_vp, c_i32, c_vp]),
    "rte_rope_table": (C.c_int, [c_vp, c_i32, c_i32, c_vp]),
    "rte_rope_apply": (C.c_int, [c_vp, c_vp, c_vp, c_vp, c_i64, c_i32, c_i32, c_i32, c_i32, c_vp]),
    "rte_attn_fwd": (C.c_int, [c_vp, c_i32, c_i32, c_vp, c_i32, c_vp, c_vp, c_i32, c_i32, c_i32, c_i32, c_vp]),
    "rte_attn_fwd_masked": (C.c_int, [c_vp, c_i32, c_i32, c_vp, c_vp, c_i32, c_vp, c_vp, c_vp, c_vp, c_i32, c_i32, c_i32, c_i32, c_vp]),
    "rte_attn_bwd": (C.c_int, [c_vp, c_i32, c_i32, c_vp, c_vp, c_i32, c_vp, c_vp, c_vp, c_i32, c_i32, c_i32, c_i32, c_vp]),
    "rte_attn_bwd_masked": (C.c_int, [c_vp, c_i32, c_i32, c_vp, c_vp, c_i32, c_vp, c_vp, c_vp, c_vp, c_vp, c_i32, c_i32, c_i32,
                                      c_i32, c_vp]),
    "rte_ce_fwd_bwd": (C.c_int, [c_vp, c_i32, c_vp, c_vp, c_i32, c_vp, c_vp, c_i32, c_i32, c_vp, c_vp]),
    "rte_segment_sum": (C.c_int, [c_vp, c_vp, c_i32, c_i32, c_vp]),
    "rte_router_fwd": (C.c_int, [c_vp, P(RouterWeights), c_vp, P(RouterOut)] + [c_i32] * 9 + [c_vp]),
    "rte_router_aux_add_dh0": (C.c_int, [c_vp, c_vp] + [c_i32] * 6 + [c_vp]),
    "rte_router_aux_bwd_data": (C.c_int, [P(RouterWeights), P(RouterOut), c_vp, c_f32, c_f32, c_vp, c_vp, c_vp, c_vp] + [c_i32] * 6 + [c_vp]),
    "rte_router_mean_prob": (C.c_int, [c_vp, c_vp, c_f32, c_i32, c_i32, c_vp]),
    "rte_router_aux_bwd_params": (C.c_int, [P(RouterOut), P(RouterGrads), c_vp] + [c_i32] * 5 + [c_vp]),
    "rte_router_aux_bwd": (C.c_int, [P(RouterWeights), P(RouterOut), c_vp, c_f32, c_f32, c_vp, P(RouterGrads), c_vp,
                                     c_vp] + [c_i32] * 6 + [c_vp]),
    "rte_topk_lowest_index": (C.c_int, [c_vp, c_i32, c_i32, c_i32, c_i32, c_vp, c_vp, c_vp]),
    "rte_macro_phi_prepare": (C.c_int, [c_vp, c_vp, c_vp, c_i32, c_i32, c_i32, c_vp]),
    "rte_macro_phi_fwd": (C.c_int, [c_vp, P(PhiParams), c_vp, c_vp, c_f32, c_vp, c_vp, c_vp, c_vp] + [c_i32] * 5 +
                          [c_f32, c_vp]),
    "rte_macro_phi_bwd": (C.c_int, [c_vp, c_vp, P(PhiParams), c_vp, c_vp, c_f32, c_vp, c_vp, c_vp, c_vp, P(PhiGrads),
                                    c_vp] + [c_i32] * 6 + [c_f32, c_vp]),
    "rte_macro_phi_fwd_hx": (C.c_int, [c_vp, c_vp, P(PhiParams), c_vp, c_vp, c_f32, c_vp, c_vp, c_vp, c_vp] + [c_i32] * 5 +
                             [c_f32, c_vp]),
    "rte_macro_phi_bwd_hx": (C.c_int, [c_vp, c_vp, c_vp, P(PhiParams), c_vp, c_vp, c_f32, c_vp, c_vp, c_vp, c_vp, c_vp,
                                       P(PhiGrads), c_vp] + [c_i32] * 6 + [c_vp]),
    "rte_sqdiff_grad": (C.c_int, [c_vp, c_vp, c_i64, c_f32, c_vp, c_vp, c_vp, c_i32, c_vp]),
    "rte_macro_phi_bwd_data": (C.c_int, [c_vp, c_vp, P(PhiParams), c_vp, c_vp, c_f32, c_vp, c_vp, c_vp, c_vp] + [c_i32] * 5 + [c_vp]),
    "rte_macro_phi_bwd_params": (C.c_int, [c_vp, c_vp, c_vp, c_vp, c_vp, c_vp, P(PhiGrads), c_vp] + [c_i32] * 6 + [c_vp]),
    "rte_cluster_route": (C.c_int, [c_vp, c_i32, c_vp, c_vp, c_vp, c_i32, c_i32, c_i32, c_vp]),
    "rte_cluster_pack": (C.c_int, [c_vp, c_i32, c_i32, c_i32, c_vp, c_vp, c_vp, c_vp, c_vp, c_vp, c_vp, c_vp]),
    "rte_gather_rows_convert": (C.c_int, [c_vp, c_i32, c_vp, c_vp, c_i32, c_i64, c_i32, c_vp]),
    "rte_csr_row_reduce_f32": (C.c_int, [c_vp, c_vp, c_vp, c_vp, c_i64, c_i32, c_i32, c_vp]),
    "rte_transpose_f32": (C.c_int, [c_vp, c_vp, c_i32, c_i32, c_i32, c_i32, c_vp]),
    "rte_svd_ffn_select": (C.c_int, [c_vp, c_vp, c_vp, c_vp, c_vp, c_vp, c_i32, c_i32, c_i32, c_i32, c_i32, c_i32, c_vp]),
    "rte_svd_ffn_swiglu_bwd": (C.c_int, [c_vp, c_vp, c_vp, c_vp, c_i64, c_i32, c_vp]),
    "rte_row_norm_f32": (C.c_int, [c_vp, c_vp, c_i32, c_i32, c_vp]),
    "rte_residual_rmsnorm_fwd": (C.c_int, [c_vp, c_vp, c_vp, c_vp, c_vp, c_i32, c_vp, c_vp, c_vp, c_vp, c_vp, c_vp, c_vp, c_vp,
                                           c_vp, c_i32, c_i32, C.c_float, c_vp]),
    "rte_swiglu_fwd": (C.c_int, [c_vp, c_vp, c_i64, c_i32, c_vp]),
    "rte_swiglu_bwd": (C.c_int, [c_vp, c_vp, c_vp, c_i64, c_i32, c_vp]),
    "rte_cast_f32_bf16": (C.c_int, [c_vp, c_vp, c_i64, c_vp]),
    "rte_add_f32": (C.c_int, [c_vp, c_vp, c_i64, c_vp]),
    "rte_fill_f32": (C.c_int, [c_vp, c_f32, c_i64, c_vp]),
    "rte_axpy_rows_f32": (C.c_int, [c_vp, c_vp, c_f32, c_i32, c_i32, c_i32, c_vp]),
    "rte_adamw_multi_tensor": (C.c_int, [c_vp, c_i32, c_i64, c_vp, c_vp, c_vp, c_vp, c_f32, c_f32, c_f32, c_f32,
                                         c_vp, c_vp]),
    "rte_adamw_multi_tensor_ex": (C.c_int, [c_vp, c_i32, c_i64, c_vp, c_vp, c_vp, c_vp, c_f32, c_f32, c_f32, c_f32,
                                            c_vp, P(AdamWExtras), c_vp]),
    "rte_nonfinite_guard": (C.c_int, [c_vp, c_i32, c_vp, c_i32, c_vp, c_i32, c_vp, c_vp, c_vp]),
    "rte_add_f32_guarded": (C.c_int, [c_vp, c_vp, c_i64, c_vp, c_vp]),
    "rte_grad_norm_multi_tensor": (C.c_int, [c_vp, c_i64, c_vp, c_vp, c_vp, c_vp, c_f32, c_vp, c_vp]),
    "rte_shortlist_build": (C.c_int, [c_vp, c_vp, c_vp, c_vp, c_vp] + [c_i32] * 7 + [c_vp, c_vp]),
    "rte_shortlist_ce": (C.c_int, [c_vp, c_vp, c_vp, c_vp, c_i32, c_vp, c_vp, c_vp, c_i32, c_i32, c_i32, c_i32, c_vp]),
    "rte_shortlist_ce_from_logits": (C.c_int, [c_vp, c_vp, c_vp, c_i32, c_vp, c_i32, c_i32, c_i32, c_vp]),
    "rte_random_tokens": (C.c_int, [c_vp, c_i64, c_i32, c_vp, c_vp]),
    "rte_scatter_cols_bf16": (C.c_int, [c_vp, c_vp, c_vp, c_i32, c_i32, c_i32, c_vp]),
    "rte_gather_rows": (C.c_int, [c_vp, c_vp, c_vp, c_i32, c_i64, c_vp]),
    "rte_scatter_add_rows_f32": (C.c_int, [c_vp, c_vp, c_vp, c_i32, c_i64, c_vp]),
    "rte_audit_route": (C.c_int, [c_vp, c_vp, c_vp, c_vp, c_vp, c_i32, c_i32, c_vp]),
    "rte_colmask_mul_bf16": (C.c_int, [c_vp, c_vp, c_vp, c_i32, c_vp, c_i32, c_i32, c_vp]),
    "rte_swiglu_masked_fwd": (C.c_int, [c_vp, c_vp, c_vp, c_i32, c_vp, c_i32, c_i32, c_vp]),
    "rte_swiglu_masked_bwd": (C.c_int, [c_vp, c_vp, c_vp, c_vp, c_i32, c_vp, c_i32, c_i32, c_vp]),
    "rte_scaled_residual_fwd": (C.c_int, [c_vp, c_vp, c_vp, c_vp, c_vp, c_vp, c_i32, c_i64, c_vp]),
    "rte_scaled_residual_bwd": (C.c_int, [c_vp] * 9 + [c_i32, P(c_i32), c_vp, c_vp, c_i32, c_i64, c_vp]),
    "rte_macro_distill": (C.c_int, [c_vp, c_vp, c_vp, c_f32, c_f32, c_f32, c_f32, c_vp, c_vp, c_i32, c_i32, c_i32, c_vp]),
    "rte_kl_distill": (C.c_int, [c_vp, c_vp, c_f32, c_f32, c_vp, c_i32, c_vp, c_i32, c_vp, c_i32, c_i32, c_vp]),
    "rte_kl_distill_grad": (C.c_int, [c_vp, c_vp, c_f32, c_f32, c_vp, c_vp, c_vp, c_i32, c_i32, c_vp]),
    "rte_audit_clip": (C.c_int, [c_vp, c_vp, c_vp, c_i32, C.c_float, c_vp, C.c_float, c_vp, c_vp, c_vp]),
    "rte_audit_sample_bernoulli": (C.c_int, [c_vp, c_vp, c_vp, c_vp, c_vp, c_vp, P(AuditSampleParams), c_vp, c_vp, c_vp, c_vp,
                                             c_vp, c_vp, c_vp, c_vp, c_vp, c_vp, c_vp]),
    "rte_scale_rows_f32": (C.c_int, [c_vp, c_vp, c_i32, c_i64, c_vp]),
    "rte_audit_alignment_sums": (C.c_int, [c_vp, c_vp, c_vp, c_i32, c_i64, c_vp, c_vp]),
    "rte_audit_recent_residual": (C.c_int, [c_vp, c_vp, c_vp, c_i32, c_i64, c_vp, c_vp, c_vp]),
    "rte_scale_rows_bf16": (C.c_int, [c_vp, c_i32, c_vp, c_i32, c_vp, c_i32, c_i32, c_vp]),
    "rte_add_rows_f32_to_bf16": (C.c_int, [c_vp, c_i32, c_vp, c_i32, c_vp, c_i32, c_i32, c_vp]),
    "rte_normalize_rows_f32": (C.c_int, [c_vp, c_vp, c_i32, c_i32, c_vp]),
    "rte_kmeans_update": (C.c_int, [c_vp, c_vp, c_vp, c_vp, c_vp, c_i32, c_i32, c_i32, c_vp]),
    "rte_cluster_aggregate": (C.c_int, [c_vp, c_vp, c_vp, c_i32, c_i32, c_i32, c_i32, c_vp]),
    "rte_cluster_pool_scores": (C.c_int, [c_vp, c_vp, c_vp, c_vp, c_i64, c_i32, c_i32, c_vp]),
    "rte_peer_allreduce_sum_f32": (C.c_int, [P(PeerComm), c_i64, c_i64, c_i32, c_i32, c_vp, c_vp]),
    "rte_peer_alloc": (C.c_int, [c_i64, P(c_vp), C.c_char_p]),
    "rte_peer_open": (C.c_int, [C.c_char_p, c_i32, P(c_vp)]),
    "rte_peer_close": (C.c_int, [c_vp]),
    "rte_peer_free": (C.c_int, [c_vp]),
    "rte_grad_norm_multi_tensor_static": (C.c_int, [c_vp, c_i64, c_vp, c_vp, c_vp, c_f32, c_vp, c_vp]),
}

_lib = None


class RteError(RuntimeError):
    pass


def load() -> C.CDLL:
    """dlopen the library and bind every declared symbol; raises if anything is missing."""
    global _lib
    if _lib is not None:
        return _lib
    if not LIB_PATH.exists():
        raise RteError(f"{LIB_PATH} is missing: build it with `python -m speedup_thingy_b200.build` "
                       "(CUDA + the sm_100a kernels are required; there is no fallback path)")
    lib = C.CDLL(str(LIB_PATH))
    for name, (restype, argtypes) in PROTOTYPES.items():
        try:
            fn = getattr(lib, name)
        except AttributeError as exc:
            raise RteError(f"librte_b200.so does not export {name}") from exc
        fn.restype = restype
        fn.argtypes = argtypes
    _lib = lib
    return lib


def check(code: int, what: str) -> None:
    if code != 0:
        msg = load().rte_status_string(code).decode()
        raise RteError(f"{what} failed: {msg} (code {code})")

"""ctypes bindings for libds41_kernels.so / libds41_core.so.

The kernels library is a plain C ABI: every call is asynchronous on the current
torch CUDA stream, allocation-free, and returns a cudaError_t.  `kernels()` builds
the library on first use when it is missing and raises loudly if it cannot be
loaded on a CUDA machine - there is no silent PyTorch fallback.
"""
from __future__ import annotations

import ctypes as C
import os
from pathlib import Path

import torch

_LIBDIR = Path(__file__).resolve().parent.parent / "_lib"
_kernels = None
_core = None


class GemmArgs(C.Structure):
    _fields_ = [
        ("A", C.c_void_p), ("B", C.c_void_p), ("out", C.c_void_p), ("split_workspace", C.c_void_p),
        ("sfa", C.c_void_p), ("sfb", C.c_void_p), ("batch_map", C.c_void_p), ("n_active", C.c_void_p),
        ("row_w", C.c_void_p), ("status", C.c_void_p),
        ("lda", C.c_longlong), ("ldb", C.c_longlong), ("ldo", C.c_longlong),
        ("a_batch_stride", C.c_longlong), ("b_batch_stride", C.c_longlong), ("out_batch_stride", C.c_longlong),
        ("sfa_batch_stride", C.c_longlong), ("sfb_batch_stride", C.c_longlong),
        ("M", C.c_int), ("N", C.c_int), ("K", C.c_int), ("batch", C.c_int), ("a_batches", C.c_int),
        ("kind", C.c_int), ("out_mode", C.c_int), ("k_splits", C.c_int), ("bn", C.c_int),
        ("b_batch_kind", C.c_int), ("up_row_offset", C.c_int), ("row_w_ld", C.c_int), ("act_limit", C.c_float),
        ("static_operand", C.c_int),
        ("ag_world", C.c_int), ("ag_rank", C.c_int), ("ag_rows", C.c_int),
        ("rs_world", C.c_int), ("rs_rank", C.c_int), ("rs_rows", C.c_int),
        ("a_peers", C.c_void_p * 8), ("ag_arrive", C.c_void_p * 8), ("ag_epoch", C.c_void_p), ("rs_out", C.c_void_p * 8),
        ("tile_group", C.c_void_p), ("tile_row0", C.c_void_p), ("tile_end", C.c_void_p), ("n_tiles_dev", C.c_void_p),
        ("scatter_meta", C.c_void_p), ("wait_flags", C.c_void_p), ("wait_epoch", C.c_void_p),
        ("scatter_out", C.c_void_p * 8), ("max_tiles", C.c_int), ("wait_world", C.c_int), ("a_format", C.c_int), ("col_limit", C.c_void_p), ("alpha", C.c_float), ("alpha_batch", C.c_void_p),
        ("sig_counter", C.c_void_p), ("sig_epoch", C.c_void_p), ("sig_flags", C.c_void_p), ("sig_world", C.c_int),
    ]


class HcStepArgs(C.Structure):
    _fields_ = [
        ("streams_in", C.c_void_p), ("streams_out", C.c_void_p), ("part_bases", C.c_void_p), ("post", C.c_void_p),
        ("comb", C.c_void_p), ("pre_in", C.c_void_p), ("fn", C.c_void_p), ("scale", C.c_void_p),
        ("base", C.c_void_p), ("norm_w", C.c_void_p), ("partial", C.c_void_p), ("xc", C.c_void_p),
        ("next_pre", C.c_void_p), ("post_out", C.c_void_p), ("comb_out", C.c_void_p), ("xn", C.c_void_p),
        ("tap_mean", C.c_void_p), ("xq", C.c_void_p), ("xq_sf", C.c_void_p), ("tickets", C.c_void_p),
        ("wait_flags", C.c_void_p), ("wait_epoch", C.c_void_p), ("status", C.c_void_p),
        ("split_stride", C.c_longlong), ("n_ranks", C.c_int), ("n_splits", C.c_int),
        ("rows", C.c_int), ("H", C.c_int), ("iters", C.c_int), ("hc_eps", C.c_float), ("norm_eps", C.c_float),
    ]


class AttendArgs(C.Structure):
    _fields_ = [
        ("q", C.c_void_p), ("ldq", C.c_longlong), ("q_off", C.c_int),
        ("rows", C.c_int), ("heads", C.c_int), ("D", C.c_int), ("window", C.c_int), ("ring", C.c_int),
        ("row_pos", C.c_void_p), ("row_slot", C.c_void_p), ("row_hi", C.c_void_p), ("row_lo", C.c_void_p),
        ("win", C.c_void_p), ("comp_pool", C.c_void_p), ("sel", C.c_void_p), ("n_sel", C.c_void_p), ("k", C.c_int),
        ("page_table", C.c_void_p), ("max_pages", C.c_int), ("page_rows", C.c_int),
        ("inv_freq", C.c_void_p), ("rope_dim", C.c_int), ("scale", C.c_float),
        ("n_splits", C.c_int), ("part_o", C.c_void_p), ("part_ml", C.c_void_p), ("sink", C.c_void_p),
        ("out", C.c_void_p), ("ldo", C.c_longlong), ("kv_row_bytes", C.c_int), ("comp_row_bytes", C.c_int),
        ("status", C.c_void_p),
    ]


class EpArgs(C.Structure):
    _fields_ = [
        ("world", C.c_int), ("rank", C.c_int), ("e_local", C.c_int), ("topk", C.c_int), ("tokens", C.c_int),
        ("H", C.c_int), ("cap", C.c_int), ("bn", C.c_int), ("bn2", C.c_int), ("max_tiles", C.c_int),
        ("x", C.c_void_p), ("ids", C.c_void_p), ("weights", C.c_void_p), ("epoch", C.c_void_p),
        ("cursor", C.c_void_p), ("ticket", C.c_void_p),
        ("counts", C.c_void_p * 8), ("send_base", C.c_void_p * 8), ("recv_x", C.c_void_p * 8),
        ("recv_meta", C.c_void_p * 8), ("recv_w", C.c_void_p * 8), ("flags", C.c_void_p * 8),
        ("tile_group", C.c_void_p), ("tile_row0", C.c_void_p), ("tile_end", C.c_void_p), ("n_tiles", C.c_void_p),
        ("total_rows", C.c_void_p), ("status", C.c_void_p),
        ("recv_q", C.c_void_p * 8), ("recv_sf", C.c_void_p * 8), ("wire_fp8", C.c_int),
    ]


class DraftRng(C.Structure):
    _fields_ = [("temperature", C.c_float), ("seed", C.c_ulonglong), ("subsequence", C.c_ulonglong),
                ("offset", C.c_ulonglong)]


class SampleRow(C.Structure):
    _fields_ = [
        ("temperature", C.c_float), ("top_k", C.c_int), ("top_p", C.c_float), ("min_p", C.c_float),
        ("seed", C.c_ulonglong), ("position", C.c_ulonglong), ("mask_row", C.c_int), ("reserved", C.c_int * 7),
    ]


def _load(name: str, builder: str):
    path = _LIBDIR / name
    if not path.exists() or os.environ.get("DS41_REBUILD"):
        from .. import build
        getattr(build, builder)()
    return C.CDLL(str(path), mode=C.RTLD_GLOBAL)


def kernels():
    global _kernels
    if _kernels is None:
        lib = _load("libds41_kernels.so", "build_kernels")
        for fn in dir_functions():
            getattr(lib, fn).restype = C.c_int
        _kernels = lib
    return _kernels


def core():
    global _core
    if _core is None:
        _core = _load("libds41_core.so", "build_core")
    return _core


def dir_functions():
    return [
        "ds41_gemm_tc", "ds41_embed_streams", "ds41_hc_post_mix", "ds41_hc_finish", "ds41_qkv_post",
        "ds41_compress", "ds41_index_score", "ds41_topk_select", "ds41_attend", "ds41_router_select",
        "ds41_moe_plan", "ds41_moe_combine", "ds41_signal", "ds41_signal_all", "ds41_moe_combine_signal", "ds41_reduce_planes", "ds41_reduce_groups", "ds41_argmax_rows",
        "ds41_argmax_merge", "ds41_spec_accept", "ds41_act_quant_mx", "ds41_decode_feedback", "ds41_hc_step", "ds41_taps_pack", "ds41_norm_rows", "ds41_markov_step", "ds41_dspark_confidence", "ds41_spec_feedback",
        "ds41_copy_ints", "ds41_rs_reduce", "ds41_ep_count", "ds41_ep_plan", "ds41_ep_dispatch", "ds41_ep_mark",
        "ds41_ep_wait", "ds41_ep_combine", "ds41_act_quant_mx_rows", "ds41_sample_rows", "ds41_engram_dequant", "ds41_engram_gate", "ds41_vis_rmsnorm", "ds41_vis_bias_act", "ds41_vis_silu_mul",
        "ds41_index_prepare", "ds41_candidate_select", "ds41_pp_signal", "ds41_pp_wait", "ds41_pp_pull", "ds41_attend_floor", "ds41_attend_kv", "ds41_index_score_cand", "ds41_topk_select_cand", "ds41_act_quant_nvfp4_rows", "ds41_vis_rope2d", "ds41_vis_softmax", "ds41_vis_merge", "ds41_vis_scatter",
        "ds41_attend_tc", "ds41_attend_merge", "ds41_engram_dequant_nvfp4", "ds41_wire_encode", "ds41_wire_decode",
    ]


class KernelError(RuntimeError):
    pass


def check(err: int, what: str):
    if err != 0:
        raise KernelError(f"{what}: cudaError {err}")


def ptr(t) -> C.c_void_p:
    if t is None:
        return C.c_void_p(0)
    if isinstance(t, int):
        return C.c_void_p(t)
    return C.c_void_p(t.data_ptr())


def stream() -> C.c_void_p:
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


STATUS_NAMES = {0: "ok", 1: "mbarrier wait timed out", 2: "flag wait timed out", 3: "bad argument",
                7: "expert-parallel receive buffer too small"}


def new_status(device) -> torch.Tensor:
    return torch.zeros(4, dtype=torch.int32, device=device)


def read_status(status: torch.Tensor):
    """Synchronising read of a kernel status word -> (code, where, block, detail)."""
    vals = status.tolist()
    return tuple(vals)


def raise_on_status(status: torch.Tensor, what: str = "kernel"):
    code, where, block, detail = read_status(status)
    if code != 0:
        raise KernelError(f"{what}: {STATUS_NAMES.get(code, code)} at site {where}, block {block}, detail {detail}")

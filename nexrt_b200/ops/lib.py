"""ctypes binding of ``libnexrt_b200.so`` (one library, ``extern "C"`` launchers, see csrc/api.h).

Same mechanism as the reference's block wrappers, which ``ctypes.CDLL`` each kernel ``.so`` and
declare ``argtypes`` by hand (``nex_n2_5_pro/head.py:69-80``); here the prototypes live in one
table.  On a machine with a GPU a missing or unloadable library is an error, never a silent
fallback to PyTorch.
"""

from __future__ import annotations

import ctypes
import os
from ctypes import POINTER, c_float, c_int, c_int64, c_size_t, c_uint, c_ulonglong, c_void_p
from typing import Optional

import torch

from ..build import build_library, library_path

vp, ci, cf, cu = c_void_p, c_int, c_float, c_uint


class LLChannelStruct(ctypes.Structure):
    """Field-for-field mirror of ``NexrtLLChannel`` in csrc/api.h."""

    _fields_ = [
        ("local", c_void_p),
        ("mc", c_void_p),
        ("peer", c_void_p * 8),
        ("seq", c_void_p),
        ("status", c_void_p),
        ("world", c_int),
        ("rank", c_int),
        ("slots", c_uint),
        ("reserved", c_uint),
        ("budget_ns", c_ulonglong),
    ]


CH = POINTER(LLChannelStruct)

_PROTOTYPES = {
    "nexrt_set_pdl": [ci],
    "nexrt_version": [],
    "nexrt_set_gemv_threads": [ci],
    "nexrt_set_event_ring": [vp],
    "nexrt_set_attn_event_ring": [vp],
    "nexrt_set_gemv_mode": [ci],
    "nexrt_set_trace": [vp],
    "nexrt_null_node": [ci, ci, ci, c_ulonglong, ci, vp, vp],
    "nexrt_trace_layout": [POINTER(ci), POINTER(ci), POINTER(ci)],
    "nexrt_embed_gather": [vp, vp, vp, vp, ci, ci, ci, vp],
    "nexrt_step_end": [vp, vp, cu, vp, vp, ci, vp],
    "nexrt_residual_add": [vp, vp, ci, vp],
    "nexrt_gdn_front": [vp] * 14 + [ci] * 6 + [cf, ci, ci, vp],
    "nexrt_gdn_core": [vp] * 6 + [ci] * 5 + [vp],
    "nexrt_attn_front": [vp] * 9 + [ci] * 7 + [cf, ci, vp],
    "nexrt_attn_decode_merges_cp": [ci],
    "nexrt_attn_decode": [vp] * 14 + [ci] * 8 + [cf, ci, ci, ci, ci, ci, ci, CH, cu, vp],
    "nexrt_oproj_allreduce": [vp] * 6 + [ci] * 4 + [cf, ci, CH, cu, CH, cu, ci, vp],
    "nexrt_moe_router": [vp] * 8 + [ci] * 5 + [cf, ci, vp, vp],
    "nexrt_moe_l1": [vp] * 6 + [ci] * 4 + [cf, ci, ci, vp],
    "nexrt_moe_router_partial": [vp] * 4 + [ci] * 5 + [cf, vp, vp],
    "nexrt_moe_l1_routed": [vp] * 5 + [ci] + [vp] * 6 + [c_ulonglong] + [ci] * 5 + [cf, vp],
    "nexrt_set_partial_out": [vp],
    "nexrt_moe_l2_allreduce": [vp] * 6 + [ci] * 4 + [CH, cu, ci, vp],
    "nexrt_lmhead_sample": [vp] * 9 + [ci] * 4 + [cf, ci, ci, CH, cu, ci, vp],
    "nexrt_sample_logits": [vp, vp, vp, ci, ci, vp],
    "nexrt_mtp_prep": [vp, vp, ci, ci, vp],
    "nexrt_mtp_preprocess": [vp] * 7 + [ci] * 4 + [cf, ci, ci, vp],
    "nexrt_row_select": [vp, vp, vp, ci, ci, vp],
    "nexrt_zero_rows": [vp, ci, vp],
    "nexrt_dflash_noise": [vp, vp, vp, vp, ci, ci, ci, ci, vp],
    "nexrt_dflash_commit": [vp, vp, ci, vp],
    "nexrt_feature_tap": [vp, vp, ci, ci, ci, ci, vp],
    "nexrt_dense_bf16": [vp] * 5 + [ci] * 6 + [cf, CH, cu, vp],
    "nexrt_kv_publish": [vp, ci, ci, ci, vp, vp, vp, vp, vp, ci, ci, ci, ci, ci, cf, ci, vp],
    "nexrt_tc_gemm_fp8": [vp, vp, c_int64, vp, vp, vp, ci, ci, ci, ci, ci, vp, vp],
    "nexrt_tc_gemm_bf16": [vp, c_int64, vp, c_int64, vp, ci, ci, ci, ci, ci, vp, vp],
    "nexrt_act_quant": [vp, ci, ci, vp, cf, vp, vp, ci, ci, ci, vp],
    "nexrt_tc_gemm_bf16_ex": [vp, c_int64, vp, c_int64, vp, ci, ci, ci, ci, ci, vp, vp],
    "nexrt_tc_gemm_fp8_ex": [vp, vp, c_int64, vp, vp, vp, ci, ci, ci, ci, ci, ci, ci, vp, ci, vp, vp],
    "nexrt_moe_mark_used": [vp, vp, ci, ci, vp],
    "nexrt_prefill_embed": [vp, vp, vp, vp, ci, ci, ci, vp],
    "nexrt_prefill_ctl": [vp, vp, ci, ci, vp],
    "nexrt_prefill_advance": [vp, ci, vp, cu, vp],
    "nexrt_planes_allreduce_residual": [vp, vp, c_int64, ci, CH, cu, vp],
    "nexrt_ll_allreduce_bench": [vp, vp, ci, ci, CH, cu, vp, vp],
    "nexrt_ll_seq_advance": [vp, cu, vp],
    "nexrt_ll_pingpong": [CH, ci, ci, cu, ci, ci, vp, vp],
    "nexrt_norm_rows": [vp, vp, vp, vp, vp, vp, ci, ci, cf, ci, vp],
    "nexrt_gdn_gate_quant": [vp, vp, vp, vp, vp, ci, ci, cf, ci, vp],
    "nexrt_moe_dense_act": [vp, vp, vp, vp, vp, ci, ci, ci, ci, ci, ci, vp],
    "nexrt_planes_residual": [vp, vp, vp, c_int64, ci, vp],
    "nexrt_gdn_chunk": [vp] * 14 + [ci] * 9 + [vp],
    "nexrt_rows_norm_split": [vp, vp, vp, vp, ci, ci, cf, vp],
    "nexrt_tc_rows_gemm": [vp, vp, vp, vp, vp, ci, ci, ci, ci, vp, vp],
    "nexrt_gdn_front_tail": [vp] * 12 + [ci] * 7 + [vp],
    "nexrt_tc_router_logits": [vp] * 6 + [ci] * 5 + [cf, vp, vp, vp],
    "nexrt_moe_router_topk": [vp, ci, ci, vp, vp, vp, ci, ci, ci, vp],
    "nexrt_lmhead_sample_from_logits": [vp] * 6 + [ci] * 6 + [CH, cu, ci, vp],
    "nexrt_oproj_stage_split": [vp] * 5 + [ci, ci, ci, cf, ci, CH, cu, vp],
    "nexrt_tc_oproj_allreduce": [vp] * 6 + [ci] * 4 + [CH, cu, vp, vp],
    "nexrt_attn_front_tail": [vp] * 6 + [ci] * 7 + [vp],
    "nexrt_tc_moe_l1": [vp] * 7 + [ci] * 6 + [cf, ci, vp, vp],
    "nexrt_tc_moe_l2_allreduce": [vp] * 8 + [ci] * 6 + [CH, cu, vp, vp],
    "nexrt_ipc_alloc": [c_size_t, POINTER(c_void_p)],
    "nexrt_ipc_get_handle": [vp, vp],
    "nexrt_ipc_open": [vp, POINTER(c_void_p)],
    "nexrt_ipc_close": [vp],
    "nexrt_ipc_free": [vp],
    "nexrt_host_mapped_alloc": [c_size_t, POINTER(c_void_p), POINTER(c_void_p)],
    "nexrt_host_mapped_free": [vp],
    "nexrt_host_wait_flag": [vp, ci, ctypes.c_double],
}

_lib: Optional[ctypes.CDLL] = None


def load(build: bool = True) -> ctypes.CDLL:
    """Load (building first if stale) the native library and install the prototypes."""
    global _lib
    if _lib is not None:
        return _lib
    path = build_library() if build else library_path()
    lib = ctypes.CDLL(str(path))
    for name, args in _PROTOTYPES.items():
        fn = getattr(lib, name)
        fn.argtypes = args
        fn.restype = ci
    lib.nexrt_attn_decode_smem.argtypes = [ci, ci, ci, ci]
    lib.nexrt_attn_decode_smem.restype = c_size_t
    lib.nexrt_moe_router_partial_split.argtypes = []
    lib.nexrt_moe_router_partial_split.restype = ci
    lib.nexrt_launch_count.argtypes = []
    lib.nexrt_launch_count.restype = c_ulonglong
    _install_optional(lib)
    if os.environ.get("NEXRT_GEMV_MODE") is not None:   # bit mask of the tensor-core / cluster kernel forms (csrc/api.h: nexrt_set_gemv_mode); 0 = CUDA-core kernels
        lib.nexrt_set_gemv_mode(int(os.environ["NEXRT_GEMV_MODE"]))
    if os.environ.get("NEXRT_PDL") is not None:
        lib.nexrt_set_pdl(int(os.environ["NEXRT_PDL"]))
    _lib = lib
    return lib


_OPTIONAL = {}


def register_optional(name: str, argtypes, restype=ci) -> None:
    """Prototype of an entry point that later translation units add."""
    _OPTIONAL[name] = (argtypes, restype)
    if _lib is not None:
        _install_optional(_lib)


def _install_optional(lib) -> None:
    for name, (args, res) in _OPTIONAL.items():
        if hasattr(lib, name):
            fn = getattr(lib, name)
            fn.argtypes = args
            fn.restype = res


class KernelError(RuntimeError):
    pass


def check(err: int, what: str) -> None:
    if err != 0:
        raise KernelError(f"{what} failed with cudaError {err}")


def ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


def stream_ptr() -> int:
    return torch.cuda.current_stream().cuda_stream

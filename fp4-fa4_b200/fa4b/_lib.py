"""ctypes binding of libfa4b.so (the C ABI declared in include/fa4b.h).

There is no fallback: if the shared library is missing or a call fails, the
caller gets an exception.  Build with ``make -C fp4-fa4_b200/csrc``.
"""

from __future__ import annotations

import ctypes as C
import pathlib

_LIB_PATH = pathlib.Path(__file__).resolve().parents[1] / "lib" / "libfa4b.so"

STATUS_EXC = {1: ValueError, 2: ValueError, 3: NotImplementedError, 4: RuntimeError, 5: TimeoutError, 6: ValueError}


class Fa4bError(RuntimeError):
    pass


class QuantNvfp4Args(C.Structure):
    _fields_ = [("x", C.c_void_p), ("rows", C.c_int64), ("cols", C.c_int64), ("ld", C.c_int64),
                ("amax", C.c_void_p), ("amax_is_input", C.c_int), ("global_scale", C.c_void_p),
                ("codes_row", C.c_void_p), ("scales_row", C.c_void_p),
                ("codes_col", C.c_void_p), ("scales_col", C.c_void_p), ("recipe", C.c_int)]


class ProjectNvfp4Args(C.Structure):
    _fields_ = [("a_codes", C.c_void_p), ("a_scales", C.c_void_p), ("a_global", C.c_void_p),
                ("w_codes", C.c_void_p), ("w_scales", C.c_void_p), ("w_global", C.c_void_p),
                ("M", C.c_int64), ("N", C.c_int64), ("K", C.c_int64), ("y", C.c_void_p), ("ldy", C.c_int64),
                ("status", C.c_void_p)]


class RopePairArgs(C.Structure):
    _fields_ = [("x", C.c_void_p), ("B", C.c_int64), ("S", C.c_int64), ("H", C.c_int64), ("D", C.c_int64),
                ("stride_b", C.c_int64), ("stride_s", C.c_int64), ("stride_h", C.c_int64),
                ("rope_cos", C.c_void_p), ("rope_sin", C.c_void_p), ("inverse", C.c_int)]


class PackQkvGradsArgs(C.Structure):
    _fields_ = [("dq", C.c_void_p), ("dk", C.c_void_p), ("dv", C.c_void_p), ("ld_q", C.c_int64), ("ld_k", C.c_int64), ("ld_v", C.c_int64),
                ("B", C.c_int64), ("S", C.c_int64), ("Hq", C.c_int64), ("Hkv", C.c_int64), ("D", C.c_int64),
                ("rope_cos", C.c_void_p), ("rope_sin", C.c_void_p), ("amax", C.c_void_p), ("amax_is_input", C.c_int),
                ("global_scale", C.c_void_p), ("codes_row", C.c_void_p), ("scales_row", C.c_void_p),
                ("codes_col", C.c_void_p), ("scales_col", C.c_void_p), ("recipe", C.c_int)]


class RmsnormQuantArgs(C.Structure):
    _fields_ = [("x", C.c_void_p), ("gamma", C.c_void_p), ("rows", C.c_int64), ("cols", C.c_int64), ("ld", C.c_int64),
                ("eps", C.c_float), ("inv_rms", C.c_void_p), ("y_out", C.c_void_p), ("amax", C.c_void_p),
                ("global_scale", C.c_void_p), ("codes_row", C.c_void_p), ("scales_row", C.c_void_p),
                ("codes_col", C.c_void_p), ("scales_col", C.c_void_p), ("recipe", C.c_int)]


class RmsnormBwdArgs(C.Structure):
    _fields_ = [("x", C.c_void_p), ("gamma", C.c_void_p), ("inv_rms", C.c_void_p), ("dy", C.c_void_p), ("rows", C.c_int64),
                ("cols", C.c_int64), ("ld", C.c_int64), ("ld_dy", C.c_int64), ("dx", C.c_void_p), ("dgamma", C.c_void_p),
                ("partials", C.c_void_p)]


class QuantMxfp4Args(C.Structure):
    _fields_ = [("x", C.c_void_p), ("rows", C.c_int64), ("cols", C.c_int64), ("ld", C.c_int64),
                ("mode", C.c_int), ("codes", C.c_void_p), ("scales", C.c_void_p)]


class AttnDims(C.Structure):
    _fields_ = [("B", C.c_int32), ("Hq", C.c_int32), ("Hkv", C.c_int32), ("S", C.c_int32), ("D", C.c_int32),
                ("softmax_scale", C.c_float), ("pv_format", C.c_int32), ("mask", C.c_int32), ("global_scale_mode", C.c_int32)]


class Strides(C.Structure):
    _fields_ = [("batch", C.c_int64), ("head", C.c_int64), ("seq", C.c_int64)]


class WsLayout(C.Structure):
    _fields_ = [(n, C.c_size_t) for n in (
        "q_codes", "q_scales", "q_global", "k_codes", "k_scales", "k_global", "v_fp8", "k_fp8", "q_fp8",
        "amax_bits", "status", "saved_total", "do_fp8", "dstat", "lstat", "dq_accum", "dkv_accum", "total")]


class AttnPrepareArgs(C.Structure):
    _fields_ = [("dims", AttnDims), ("q", C.c_void_p), ("q_strides", Strides), ("k", C.c_void_p), ("k_strides", Strides),
                ("v", C.c_void_p), ("v_strides", Strides), ("ws", C.c_void_p), ("phase", C.c_int32)]


class AttnFwdArgs(C.Structure):
    _fields_ = [("dims", AttnDims), ("q", C.c_void_p), ("q_strides", Strides), ("k", C.c_void_p), ("k_strides", Strides),
                ("v", C.c_void_p), ("v_strides", Strides), ("o", C.c_void_p), ("o_strides", Strides),
                ("lse", C.c_void_p), ("ws", C.c_void_p), ("prepared", C.c_int32), ("ev_before", C.c_void_p),
                ("ev_after", C.c_void_p), ("kv_ws", C.c_void_p)]


class AttnBwdArgs(C.Structure):
    _fields_ = [("dims", AttnDims), ("o", C.c_void_p), ("o_strides", Strides), ("dout", C.c_void_p), ("do_strides", Strides),
                ("lse", C.c_void_p), ("dq", C.c_void_p), ("dq_strides", Strides), ("dk", C.c_void_p), ("dk_strides", Strides),
                ("dv", C.c_void_p), ("dv_strides", Strides), ("ws", C.c_void_p), ("preprocessed", C.c_int32),
                ("ev_before", C.c_void_p), ("ev_after", C.c_void_p), ("kv_ws", C.c_void_p), ("flags", C.c_int32),
                ("scratch", C.c_void_p)]


class BwdPlan(C.Structure):
    _fields_ = [("chunk", C.c_int32), ("items_per_head", C.c_int32), ("split_rows", C.c_int32), ("head_group", C.c_int32),
                ("grid", C.c_int64)]


class Info(C.Structure):
    _fields_ = [(n, C.c_int) for n in (
        "abi_version", "build_sm", "fwd_threads", "fwd_smem_bytes", "fwd_tmem_columns", "fwd_kv_stages",
        "bwd_threads", "bwd_smem_bytes", "bwd_tmem_columns", "tile_q", "tile_kv", "wait_limit")]


EXPORTS = (
    "fa4b_status_string", "fa4b_last_error", "fa4b_query", "fa4b_amax", "fa4b_quant_nvfp4", "fa4b_quant_check_status", "fa4b_quant_nvfp4_weight", "fa4b_project_nvfp4", "fa4b_project_qkv_publish", "fa4b_project_dout_publish", "fa4b_rope_pair", "fa4b_pack_qkv_grads",
    "fa4b_rmsnorm_quant_nvfp4", "fa4b_quant_mxfp4", "fa4b_dequant_nvfp4", "fa4b_dequant_mxfp4",
    "fa4b_attn_workspace_bytes", "fa4b_attn_ws_layout_query", "fa4b_attn_prepare", "fa4b_attn_fwd",
    "fa4b_attn_fwd_static", "fa4b_attn_bwd_preprocess", "fa4b_attn_bwd", "fa4b_attn_bwd_plan", "fa4b_attn_bwd_plan_item", "fa4b_attn_check_status", "fa4b_attn_merge", "fa4b_attn_accumulate", "fa4b_rmsnorm_bwd", "fa4b_rmsnorm_bwd_workspace_bytes", "fa4b_microgate", "fa4b_tensor_peak", "fa4b_wait_selftest",
)

_lib = None


def lib() -> C.CDLL:
    """The loaded library; raises if it has not been built."""
    global _lib
    if _lib is None:
        if not _LIB_PATH.exists():
            raise Fa4bError(f"{_LIB_PATH} is missing: build it with `make -C {_LIB_PATH.parents[1] / 'csrc'}`")
        handle = C.CDLL(str(_LIB_PATH))
        handle.fa4b_status_string.restype = C.c_char_p
        handle.fa4b_last_error.restype = C.c_char_p
        handle.fa4b_attn_workspace_bytes.restype = C.c_size_t
        handle.fa4b_rmsnorm_bwd_workspace_bytes.restype = C.c_size_t
        handle.fa4b_rmsnorm_bwd_workspace_bytes.argtypes = [C.c_int64]
        for name in EXPORTS:
            getattr(handle, name)  # AttributeError if the ABI is incomplete
        _lib = handle
    return _lib


def check(status: int, what: str) -> None:
    if status == 0:
        return
    handle = lib()
    reason = handle.fa4b_last_error().decode(errors="replace")
    kind = handle.fa4b_status_string(status).decode()
    raise STATUS_EXC.get(status, Fa4bError)(f"{what}: {kind}: {reason}")


def ptr(t) -> int:
    return 0 if t is None else t.data_ptr()


def current_stream() -> int:
    import torch

    return torch.cuda.current_stream().cuda_stream

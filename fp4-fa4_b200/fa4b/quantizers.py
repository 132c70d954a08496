"""Block quantizer operators, named after the reference's pybind entry points
(TK_quantisation/nvfp4_v6/tk_quantize.cu:3172-3234,
TK_quantisation/mxfp4_v3/tk_quantize.cu:2052-2054)."""

from __future__ import annotations

import ctypes as C

import torch

from . import _lib
from ._lib import check, current_stream, lib, ptr

MX_MODES = {"ceil": 0, "rte_mantissa": 1, "floor": 2, 0: 0, 1: 1, 2: 2}


def _require_matrix(x: torch.Tensor, name: str) -> None:
    if not isinstance(x, torch.Tensor) or x.ndim != 2:
        raise ValueError(f"{name} must be a 2-D tensor")
    if x.dtype != torch.bfloat16:
        raise TypeError(f"{name} must be bfloat16, got {x.dtype}")
    if not x.is_cuda:
        raise RuntimeError(f"{name} must live on a CUDA device (there is no CPU path)")
    if x.stride(1) != 1:
        raise ValueError(f"{name} must have a contiguous last dimension")
    if x.shape[0] % 128 or x.shape[1] % 128:
        raise ValueError(f"{name} shape {tuple(x.shape)} must be multiples of 128")


def amax(x: torch.Tensor) -> torch.Tensor:
    """max |x| of a contiguous bf16 tensor -> f32 [1]."""
    if x.dtype != torch.bfloat16 or not x.is_cuda or not x.is_contiguous():
        raise ValueError("amax needs a contiguous CUDA bfloat16 tensor")
    out = torch.empty(1, dtype=torch.float32, device=x.device)
    check(lib().fa4b_amax(C.c_void_p(ptr(x)), C.c_int64(x.numel()), C.c_void_p(ptr(out)), C.c_void_p(current_stream())), "fa4b_amax")
    return out


def _alloc_outputs(rows, cols, transpose, dev, block=16):
    fp4_row = torch.empty(rows, cols // 2, dtype=torch.uint8, device=dev)
    sc_row = torch.empty(rows // 128, cols // (4 * block), 512, dtype=torch.uint8, device=dev)
    fp4_col = sc_col = None
    if transpose:
        fp4_col = torch.empty(cols, rows // 2, dtype=torch.uint8, device=dev)
        sc_col = torch.empty(cols // 128, rows // (4 * block), 512, dtype=torch.uint8, device=dev)
    return fp4_row, sc_row, fp4_col, sc_col


def tk_quantize_for_gemm(input: torch.Tensor, return_transpose: bool = True, encode_centric: bool = True, *,
                         amax_in: torch.Tensor | None = None):
    """NVFP4 of ``input [M,K]``: returns ``(fp4_row [M,K/2], sc_row [M/128,K/64,512],
    fp4_col [K,M/2] | None, sc_col [K/128,M/64,512] | None, sg [1], amax [1])``.
    ``sg = amax/2688``; scale bytes are E4M3.  Positional arguments and defaults are the reference binding's
    (``tk_quantize_for_gemm(input, return_transpose, encode_centric=true)``,
    TK_quantisation/nvfp4_v6/tk_quantize.cu:3170-3172): ``encode_centric=True`` rounds the block multiplier and
    stores the E4M3 of its reciprocal; ``False`` is the decode-centric arithmetic of the reference's Python oracle
    (``fake_quantize_nvfp4``), which the attention block's projections use.  ``amax_in`` (keyword only, not in the
    reference) supplies the tensor amax instead of a statistics pass."""
    _require_matrix(input, "input")
    rows, cols = input.shape
    fp4_row, sc_row, fp4_col, sc_col = _alloc_outputs(rows, cols, return_transpose, input.device)
    am = torch.empty(1, dtype=torch.float32, device=input.device) if amax_in is None else amax_in
    sg = torch.empty(1, dtype=torch.float32, device=input.device)
    a = _lib.QuantNvfp4Args(ptr(input), rows, cols, input.stride(0), ptr(am), int(amax_in is not None), ptr(sg),
                            ptr(fp4_row), ptr(sc_row), ptr(fp4_col), ptr(sc_col), int(bool(encode_centric)))
    check(lib().fa4b_quant_nvfp4(C.byref(a), C.c_void_p(current_stream())), "fa4b_quant_nvfp4")
    return fp4_row, sc_row, fp4_col, sc_col, sg, am


def check_status() -> None:
    """Synchronise the current stream and raise if a quantizer kernel's bounded wait for its tile ran out since the
    last check (``fa4b_quant_check_status``; the kernels record the event instead of spinning)."""
    check(lib().fa4b_quant_check_status(C.c_void_p(current_stream())), "fa4b_quant_check_status")


def prepare_nvfp4_projection_weight(tensor: torch.Tensor):
    """Learned projection weight ``[N,K]`` with 16x16 NVFP4 scaling: ``(payload [N,K/2], scales
    [N/128,K/64,512], global [1])`` (b300_prepare_nvfp4_projection_weight, tk_fa4/interface.py:1221-1244)."""
    fwd, _ = _prepare_weight(tensor, dual=False)
    return fwd


def prepare_nvfp4_projection_weight_dual(tensor: torch.Tensor):
    """The weight and its exact physical transpose, quantised once: ``(forward, transpose)``, each a
    ``(payload, scales, global)`` triple; both share one global decode scale tensor
    (b300_prepare_nvfp4_projection_weight_dual, tk_fa4/interface.py:1247-1313)."""
    return _prepare_weight(tensor, dual=True)


def _prepare_weight(tensor: torch.Tensor, dual: bool):
    _require_matrix(tensor, "tensor")
    if not tensor.is_contiguous():
        raise ValueError("tensor must be contiguous")
    rows, cols = tensor.shape
    fp4_row, sc_row, fp4_col, sc_col = _alloc_outputs(rows, cols, dual, tensor.device)
    am = torch.empty(1, dtype=torch.float32, device=tensor.device)
    sg = torch.empty(1, dtype=torch.float32, device=tensor.device)
    a = _lib.QuantNvfp4Args(ptr(tensor), rows, cols, tensor.stride(0), ptr(am), 0, ptr(sg),
                            ptr(fp4_row), ptr(sc_row), ptr(fp4_col), ptr(sc_col))
    check(lib().fa4b_quant_nvfp4_weight(C.byref(a), C.c_void_p(current_stream())), "fa4b_quant_nvfp4_weight")
    return (fp4_row, sc_row, sg), ((fp4_col, sc_col, sg) if dual else None)


def project_nvfp4(input_operand, weight_operand, out: torch.Tensor | None = None, status: torch.Tensor | None = None) -> torch.Tensor:
    """``[M,K] x [N,K]^T -> bf16 [M,N]`` for two prepared NVFP4 operands ``(payload, scale pages, global)``
    (b300_project_nvfp4, tk_fa4/interface.py:1619-1640).  ``status`` (u32 [4], device) receives the kernel's
    wait status; when it is not supplied the call synchronises and raises if a device-side wait gave up."""
    if len(input_operand) != 3 or len(weight_operand) != 3:
        raise ValueError("NVFP4 operands must contain packed data, block scales, and one global scale")
    a, a_sc, a_g = input_operand
    w, w_sc, w_g = weight_operand
    for name, t in (("payload", a), ("scales", a_sc), ("weight payload", w), ("weight scales", w_sc)):
        if not t.is_cuda or t.element_size() != 1 or not t.is_contiguous():
            raise ValueError(f"{name} must be a contiguous byte-sized CUDA tensor")
    M, K = a.shape[0], a.shape[1] * 2
    N = w.shape[0]
    if w.shape[1] * 2 != K:
        raise ValueError(f"inner dimensions differ: activation K={K}, weight K={w.shape[1] * 2}")
    if tuple(a_sc.shape) != (M // 128, K // 64, 512) or tuple(w_sc.shape) != (N // 128, K // 64, 512):
        raise ValueError("scale pages have an invalid shape")
    if a_g.numel() != 1 or w_g.numel() != 1 or a_g.dtype != torch.float32 or w_g.dtype != torch.float32:
        raise ValueError("global scales must be one float32 each")
    if out is None:
        out = torch.empty(M, N, dtype=torch.bfloat16, device=a.device)
    elif out.dtype != torch.bfloat16 or tuple(out.shape) != (M, N) or out.stride(1) != 1:
        raise ValueError("out must be bfloat16 [M, N] with a contiguous last dimension")
    own = status is None
    if own:
        status = torch.empty(4, dtype=torch.int32, device=a.device)
    args = _lib.ProjectNvfp4Args(ptr(a), ptr(a_sc), ptr(a_g), ptr(w), ptr(w_sc), ptr(w_g), M, N, K, ptr(out), out.stride(0), ptr(status))
    check(lib().fa4b_project_nvfp4(C.byref(args), C.c_void_p(current_stream())), "fa4b_project_nvfp4")
    if own:
        st = status.cpu().tolist()
        if st[0] != 0:
            raise RuntimeError(f"fa4b_project_nvfp4: a device-side wait gave up (site {st[1]}, block {st[2]}, detail {st[3]})")
    return out


def project_qkv_publish(input_operand, weight_operand, rope_cos: torch.Tensor, rope_sin: torch.Tensor, workspace,
                        status: torch.Tensor | None = None) -> None:
    """QKV projection with the attention operands published from its epilogue: after the call ``workspace`` (an
    ``attention.Workspace`` whose dims have ``D = 128``, FP8 P.V and ``global_scale="one"``) holds what
    ``project_nvfp4`` + ``rope_pair_`` on Q and K + ``attention.attn_prepare`` would have put there, and the forward
    runs with ``attention.attn_forward_prepared``.  Weight rows: Hq query heads, Hkv key heads, Hkv value heads."""
    a, a_sc, a_g = input_operand
    w, w_sc, w_g = weight_operand
    M, K, N = a.shape[0], a.shape[1] * 2, w.shape[0]
    if w.shape[1] * 2 != K:
        raise ValueError(f"inner dimensions differ: activation K={K}, weight K={w.shape[1] * 2}")
    d = workspace.dims
    for name, t in (("rope_cos", rope_cos), ("rope_sin", rope_sin)):
        if t.dtype != torch.bfloat16 or tuple(t.shape) != (d.S, 64) or not t.is_contiguous() or not t.is_cuda:
            raise ValueError(f"{name} must be a contiguous CUDA bfloat16 [S, 64] tensor")
    own = status is None
    if own:
        status = torch.empty(4, dtype=torch.int32, device=a.device)
    args = _lib.ProjectNvfp4Args(ptr(a), ptr(a_sc), ptr(a_g), ptr(w), ptr(w_sc), ptr(w_g), M, N, K, 0, 0, ptr(status))
    check(lib().fa4b_project_qkv_publish(C.byref(args), C.byref(d), C.c_void_p(ptr(rope_cos)), C.c_void_p(ptr(rope_sin)),
                                         C.c_void_p(ptr(workspace.buf)), C.c_void_p(current_stream())), "fa4b_project_qkv_publish")
    if own:
        st = status.cpu().tolist()
        if st[0] != 0:
            raise RuntimeError(f"fa4b_project_qkv_publish: a device-side wait gave up (site {st[1]}, block {st[2]}, detail {st[3]})")


def project_dout_publish(grad_operand, weight_t_operand, o_rows: torch.Tensor, lse: torch.Tensor, workspace,
                         status: torch.Tensor | None = None) -> None:
    """Input-gradient GEMM of the output projection (``dO = dY . Wo``, the weight operand being the transposed one of
    the dual publication) with the attention backward's publication in its epilogue: ``workspace`` receives E5M2(4 dO)
    and the row statistics that ``attention.attn_bwd_preprocess`` would compute from a BF16 dO, which is never
    written; the backward then runs with ``attention.attn_backward_prepared``.  ``o_rows`` bf16 ``[B*S, Hq*128]``
    (the forward's output), ``lse`` f32 ``[B, Hq, S]``."""
    a, a_sc, a_g = grad_operand
    w, w_sc, w_g = weight_t_operand
    M, K, N = a.shape[0], a.shape[1] * 2, w.shape[0]
    if w.shape[1] * 2 != K:
        raise ValueError(f"inner dimensions differ: gradient K={K}, weight K={w.shape[1] * 2}")
    d = workspace.dims
    if o_rows.dtype != torch.bfloat16 or tuple(o_rows.shape) != (M, N) or not o_rows.is_contiguous() or not o_rows.is_cuda:
        raise ValueError(f"o_rows must be a contiguous CUDA bfloat16 {(M, N)} tensor")
    if lse.dtype != torch.float32 or tuple(lse.shape) != (d.B, d.Hq, d.S) or not lse.is_contiguous():
        raise ValueError(f"lse must be a contiguous float32 {(d.B, d.Hq, d.S)} tensor")
    own = status is None
    if own:
        status = torch.empty(4, dtype=torch.int32, device=a.device)
    args = _lib.ProjectNvfp4Args(ptr(a), ptr(a_sc), ptr(a_g), ptr(w), ptr(w_sc), ptr(w_g), M, N, K, 0, 0, ptr(status))
    check(lib().fa4b_project_dout_publish(C.byref(args), C.byref(d), C.c_void_p(ptr(o_rows)), C.c_void_p(ptr(lse)),
                                          C.c_void_p(ptr(workspace.buf)), C.c_void_p(current_stream())), "fa4b_project_dout_publish")
    if own:
        st = status.cpu().tolist()
        if st[0] != 0:
            raise RuntimeError(f"fa4b_project_dout_publish: a device-side wait gave up (site {st[1]}, block {st[2]}, detail {st[3]})")


def rope_pair_(x: torch.Tensor, rope_cos: torch.Tensor, rope_sin: torch.Tensor, inverse: bool = False) -> torch.Tensor:
    """In-place pair-native rotary embedding of ``x [B,S,H,D]`` bf16 (any strides with a contiguous last dimension)
    with bf16 tables ``[S, D/2]``; ``inverse=True`` turns the other way (gradients).  One tensor of
    ``b300_rope_pair_qk_`` / ``b300_inverse_rope_interleaved_qkv_grad_`` (tk_fa4/interface.py:6584, 6564)."""
    if x.ndim != 4 or x.dtype != torch.bfloat16 or not x.is_cuda or x.stride(3) != 1:
        raise ValueError("x must be a CUDA bfloat16 [B,S,H,D] tensor with a contiguous last dimension")
    B, S, H, D = x.shape
    for name, t in (("rope_cos", rope_cos), ("rope_sin", rope_sin)):
        if t.dtype != torch.bfloat16 or tuple(t.shape) != (S, D // 2) or not t.is_contiguous() or t.device != x.device:
            raise ValueError(f"{name} must be a contiguous bfloat16 [S, D/2] tensor on the device of x")
    a = _lib.RopePairArgs(ptr(x), B, S, H, D, x.stride(0), x.stride(1), x.stride(2), ptr(rope_cos), ptr(rope_sin), int(inverse))
    check(lib().fa4b_rope_pair(C.byref(a), C.c_void_p(current_stream())), "fa4b_rope_pair")
    return x


def pack_qkv_grads(dq: torch.Tensor, dk: torch.Tensor, dv: torch.Tensor, rope_cos: torch.Tensor, rope_sin: torch.Tensor,
                   return_transpose: bool = True, encode_centric: bool = False, *, amax_in: torch.Tensor | None = None):
    """The NVFP4 operand of the QKV projection's backward GEMMs from the attention gradients ``dq [B,S,Hq,D]``,
    ``dk``, ``dv [B,S,Hkv,D]`` (bf16; token-major, a token's heads contiguous -- column ranges of one
    ``[B*S, (Hq+2Hkv)D]`` buffer qualify): ``[dQ | dK | dV]`` with dQ and dK turned back through the pair-native
    rotation, as the 6-tuple of :func:`tk_quantize_for_gemm` (``rows = B*S``, ``cols = (Hq+2Hkv)D``).  One pass over
    the gradients (two when the amax is not given) instead of two in-place rotations, a statistics pass and the
    quantiser; the results are byte-identical.  The producer behind
    ``b300_pack_gqa_d128_hierarchical_qkv_gradient_nvfp4_tiles`` (tk_fa4/interface.py:4864-4912;
    tk_fa4/lowp_fa4_bwd/gqa_d128_hierarchical_qkv_nvfp4_quantize.cuh), which takes its global scale as an input
    like ``amax_in`` here."""
    for name, t in (("dq", dq), ("dk", dk), ("dv", dv)):
        if t.ndim != 4 or t.dtype != torch.bfloat16 or not t.is_cuda or t.stride(3) != 1 or t.stride(2) != t.shape[3] or (t.shape[0] > 1 and t.stride(0) != t.shape[1] * t.stride(1)):
            raise ValueError(f"{name} must be a CUDA bfloat16 [B,S,H,D] tensor, a token's heads contiguous and batches token-major")
    B, S, Hq, D = dq.shape
    Hkv = dk.shape[2]
    if tuple(dk.shape) != (B, S, Hkv, D) or tuple(dv.shape) != (B, S, Hkv, D):
        raise ValueError("dk and dv must be [B,S,Hkv,D] with the batch, length and head size of dq")
    for name, t in (("rope_cos", rope_cos), ("rope_sin", rope_sin)):
        if t.dtype != torch.bfloat16 or tuple(t.shape) != (S, D // 2) or not t.is_contiguous() or t.device != dq.device:
            raise ValueError(f"{name} must be a contiguous bfloat16 [S, D/2] tensor on the device of dq")
    rows, cols = B * S, (Hq + 2 * Hkv) * D
    if rows % 128 or cols % 128:
        raise ValueError(f"B*S={rows} and (Hq+2Hkv)*D={cols} must be multiples of 128")
    fp4_row, sc_row, fp4_col, sc_col = _alloc_outputs(rows, cols, return_transpose, dq.device)
    am = torch.empty(1, dtype=torch.float32, device=dq.device) if amax_in is None else amax_in
    sg = torch.empty(1, dtype=torch.float32, device=dq.device)
    a = _lib.PackQkvGradsArgs(ptr(dq), ptr(dk), ptr(dv), dq.stride(1), dk.stride(1), dv.stride(1), B, S, Hq, Hkv, D, ptr(rope_cos), ptr(rope_sin),
                              ptr(am), int(amax_in is not None), ptr(sg), ptr(fp4_row), ptr(sc_row), ptr(fp4_col), ptr(sc_col), int(bool(encode_centric)))
    check(lib().fa4b_pack_qkv_grads(C.byref(a), C.c_void_p(current_stream())), "fa4b_pack_qkv_grads")
    return fp4_row, sc_row, fp4_col, sc_col, sg, am


def tk_fused_norm_quantize(input: torch.Tensor, gamma: torch.Tensor, epsilon: float = 1e-6, with_silu: bool = False,
                           return_transpose: bool = True, *, return_normalized: bool = False, encode_centric: bool = True):
    """Fused RMSNorm + NVFP4: returns ``(fp4_row, sc_row, fp4_col, sc_col, sg,
    inv_rms [M], amax [1])`` (plus the bf16 normalised tensor when asked)."""
    _require_matrix(input, "input")
    if with_silu:
        raise NotImplementedError("the SiLU variant feeds the FFN GEMMs and is outside this attention path")
    if gamma.dtype != torch.bfloat16 or gamma.ndim != 1 or gamma.shape[0] != input.shape[1] or not gamma.is_cuda:
        raise ValueError("gamma must be a CUDA bfloat16 vector of length K")
    rows, cols = input.shape
    fp4_row, sc_row, fp4_col, sc_col = _alloc_outputs(rows, cols, return_transpose, input.device)
    dev = input.device
    inv_rms = torch.empty(rows, dtype=torch.float32, device=dev)
    am = torch.empty(1, dtype=torch.float32, device=dev)
    sg = torch.empty(1, dtype=torch.float32, device=dev)
    y = torch.empty(rows, cols, dtype=torch.bfloat16, device=dev) if return_normalized else None
    a = _lib.RmsnormQuantArgs(ptr(input), ptr(gamma.contiguous()), rows, cols, input.stride(0), float(epsilon), ptr(inv_rms), ptr(y),
                              ptr(am), ptr(sg), ptr(fp4_row), ptr(sc_row), ptr(fp4_col), ptr(sc_col), int(bool(encode_centric)))
    check(lib().fa4b_rmsnorm_quant_nvfp4(C.byref(a), C.c_void_p(current_stream())), "fa4b_rmsnorm_quant_nvfp4")
    out = (fp4_row, sc_row, fp4_col, sc_col, sg, inv_rms, am)
    return out + (y,) if return_normalized else out


def rmsnorm_backward_bf16(tensor: torch.Tensor, gamma: torch.Tensor, inv_rms: torch.Tensor, gradient: torch.Tensor):
    """Backward of the fused RMSNorm: ``(dx [M,K] bf16, dgamma [K] bf16)`` from the input, gamma, the saved
    ``inv_rms [M]`` f32 and the gradient of the normalised output (same name and argument order as the
    reference's ``rmsnorm_backward_bf16``, ``tk_fa4/interface.py:1144-1150``)."""
    _require_matrix(tensor, "tensor")
    _require_matrix(gradient, "gradient")
    if gradient.shape != tensor.shape:
        raise ValueError(f"gradient {tuple(gradient.shape)} does not match tensor {tuple(tensor.shape)}")
    rows, cols = tensor.shape
    if gamma.dtype != torch.bfloat16 or gamma.shape != (cols,) or not gamma.is_cuda or not gamma.is_contiguous():
        raise ValueError("gamma must be a contiguous CUDA bfloat16 vector of length K")
    if inv_rms.dtype != torch.float32 or inv_rms.shape != (rows,) or not inv_rms.is_cuda or not inv_rms.is_contiguous():
        raise ValueError("inv_rms must be a contiguous CUDA float32 vector of length M")
    nbytes = lib().fa4b_rmsnorm_bwd_workspace_bytes(cols)
    dev = tensor.device
    partials = torch.empty(max(nbytes // 4, 1), dtype=torch.float32, device=dev)
    dx = torch.empty(rows, cols, dtype=torch.bfloat16, device=dev)
    dgamma = torch.empty(cols, dtype=torch.bfloat16, device=dev)
    a = _lib.RmsnormBwdArgs(ptr(tensor), ptr(gamma), ptr(inv_rms), ptr(gradient), rows, cols, tensor.stride(0), gradient.stride(0),
                            ptr(dx), ptr(dgamma), ptr(partials))
    check(lib().fa4b_rmsnorm_bwd(C.byref(a), C.c_void_p(current_stream())), "fa4b_rmsnorm_bwd")
    return dx, dgamma


def mxfp4_quantize_for_gemm(input: torch.Tensor, mode: int | str = "ceil"):
    """MXFP4 (1x32, E8M0) of ``input [M,K]``: ``(fp4 [M,K/2], scales [M/128,K/128,512])``."""
    _require_matrix(input, "input")
    if mode not in MX_MODES:
        raise ValueError(f"unknown MXFP4 scale mode {mode!r}")
    rows, cols = input.shape
    fp4, sc, _, _ = _alloc_outputs(rows, cols, False, input.device, block=32)
    a = _lib.QuantMxfp4Args(ptr(input), rows, cols, input.stride(0), MX_MODES[mode], ptr(fp4), ptr(sc))
    check(lib().fa4b_quant_mxfp4(C.byref(a), C.c_void_p(current_stream())), "fa4b_quant_mxfp4")
    return fp4, sc


def dequant_nvfp4(codes: torch.Tensor, scale_pages: torch.Tensor, sg: torch.Tensor) -> torch.Tensor:
    rows, cols = codes.shape[0], codes.shape[1] * 2
    out = torch.empty(rows, cols, dtype=torch.float32, device=codes.device)
    check(lib().fa4b_dequant_nvfp4(C.c_void_p(ptr(codes)), C.c_void_p(ptr(scale_pages)), C.c_void_p(ptr(sg)), C.c_int64(rows),
                                   C.c_int64(cols), C.c_void_p(ptr(out)), C.c_void_p(current_stream())), "fa4b_dequant_nvfp4")
    return out


def dequant_mxfp4(codes: torch.Tensor, scale_pages: torch.Tensor) -> torch.Tensor:
    rows, cols = codes.shape[0], codes.shape[1] * 2
    out = torch.empty(rows, cols, dtype=torch.float32, device=codes.device)
    check(lib().fa4b_dequant_mxfp4(C.c_void_p(ptr(codes)), C.c_void_p(ptr(scale_pages)), C.c_int64(rows), C.c_int64(cols),
                                   C.c_void_p(ptr(out)), C.c_void_p(current_stream())), "fa4b_dequant_mxfp4")
    return out

"""Attention operators over the C ABI: operand publication, forward, backward.

Tensors are ``[B,H,S,D]`` bf16 views (any batch/head/sequence strides, last
dimension contiguous), the layout ``FA4AttentionWrapper.forward`` receives
(torchtitan/experiments/fa4/fa4_attention.py:507-548)."""

from __future__ import annotations

import ctypes as C
from dataclasses import dataclass

import torch

from . import _lib
from ._lib import check, current_stream, lib, ptr

PV_FORMATS = {"e4m3_fp8": 0, "mxfp4_e8m0_block32": 1}


def _strides(t: torch.Tensor) -> _lib.Strides:
    return _lib.Strides(t.stride(0), t.stride(1), t.stride(2))


def _check_bhsd(t: torch.Tensor, name: str) -> None:
    if not isinstance(t, torch.Tensor) or t.ndim != 4:
        raise ValueError(f"{name} must be a [B,H,S,D] tensor")
    if t.dtype != torch.bfloat16:
        raise TypeError(f"{name} must be bfloat16, got {t.dtype}")
    if not t.is_cuda:
        raise RuntimeError(f"{name} must live on a CUDA device (there is no CPU path)")
    if t.stride(3) != 1:
        raise ValueError(f"{name} must have a contiguous head dimension")


@dataclass
class Workspace:
    """Operand cache of one attention call (see fa4b_attn_ws_layout).

    ``buf`` holds the saved section (what the forward publishes and the backward replays) and, unless ``scratch``
    is given, the transient section behind it (E5M2 dO, row statistics, FP32 accumulators of one backward call).
    ``scratch`` is that transient section as a buffer of its own, which many workspaces may share."""

    dims: _lib.AttnDims
    layout: _lib.WsLayout
    buf: torch.Tensor
    scratch: torch.Tensor | None = None

    def _view(self, off: int, nbytes: int) -> torch.Tensor:
        if off >= self.layout.saved_total and self.scratch is not None:
            off -= self.layout.saved_total
            return self.scratch[off:off + nbytes]
        if off + nbytes > self.buf.numel():
            raise RuntimeError("this workspace holds the saved section only; the transient section needs a scratch buffer")
        return self.buf[off:off + nbytes]

    def saved(self) -> torch.Tensor:
        """The bytes a training step keeps from forward to backward (a view)."""
        return self.buf[:self.layout.saved_total]

    def with_scratch(self, scratch: torch.Tensor) -> "Workspace":
        need = self.layout.total - self.layout.saved_total
        if scratch.numel() < need or scratch.data_ptr() % 1024:
            raise ValueError(f"scratch must hold {need} bytes and be 1024-byte aligned")
        return Workspace(self.dims, self.layout, self.buf, scratch[:need])

    def operands(self):
        d = self.dims
        nq, nk, S, D = d.B * d.Hq, d.B * d.Hkv, d.S, d.D
        L = self.layout
        ops = {}
        if d.pv_format == PV_FORMATS["mxfp4_e8m0_block32"]:
            # the V section then holds sequence-grouped MXFP4: codes [B,Hkv,D,S/2], then (1024-aligned) E8M0 pages
            n_codes = nk * D * S // 2
            pages_at = L.v_fp8 + (n_codes + 1023) // 1024 * 1024
            ops["v_mx_codes"] = self._view(L.v_fp8, n_codes).view(d.B, d.Hkv, D, S // 2)
            ops["v_mx_scales"] = self._view(pages_at, nk * (S // 128) * 512).view(d.B, d.Hkv, S // 128, 512)
        return ops | {
            "q_codes": self._view(L.q_codes, nq * S * D // 2).view(d.B, d.Hq, S, D // 2),
            "q_scales": self._view(L.q_scales, nq * (S // 128) * (D // 64) * 512).view(d.B, d.Hq, S // 128, D // 64, 512),
            "q_global": self._view(L.q_global, nq * 4).view(torch.float32).view(d.B, d.Hq),
            "k_codes": self._view(L.k_codes, nk * S * D // 2).view(d.B, d.Hkv, S, D // 2),
            "k_scales": self._view(L.k_scales, nk * (S // 128) * (D // 64) * 512).view(d.B, d.Hkv, S // 128, D // 64, 512),
            "k_global": self._view(L.k_global, nk * 4).view(torch.float32).view(d.B, d.Hkv),
            "v_fp8": self._view(L.v_fp8, nk * S * D).view(torch.float8_e4m3fn).view(d.B, d.Hkv, S, D),
            "q_fp8": self._view(L.q_fp8, nq * S * D).view(torch.float8_e4m3fn).view(d.B, d.Hq, S, D),
            "k_fp8": self._view(L.k_fp8, nk * S * D).view(torch.float8_e4m3fn).view(d.B, d.Hkv, S, D),
            "do_fp8": self._view(L.do_fp8, nq * S * D).view(torch.float8_e5m2).view(d.B, d.Hq, S, D),
            "dstat": self._view(L.dstat, nq * S * 4).view(torch.float32).view(d.B, d.Hq, S),
            "lstat": self._view(L.lstat, nq * S * 4).view(torch.float32).view(d.B, d.Hq, S),
        }

    def amax(self) -> torch.Tensor:
        """The per-(batch, head) amax words of q (B*Hq) then k (B*Hkv), f32, as a view."""
        d = self.dims
        return self._view(self.layout.amax_bits, (d.B * d.Hq + d.B * d.Hkv) * 4).view(torch.float32)

    def kv_bytes(self) -> torch.Tensor:
        """The K and V operands (codes, scale pages, global scales, V) as one contiguous byte range: what a
        sequence-sharded run sends to the next rank."""
        return self._view(self.layout.k_codes, self.layout.q_fp8 - self.layout.k_codes)

    def check_status(self) -> None:
        check(lib().fa4b_attn_check_status(C.byref(self.dims), C.c_void_p(ptr(self.buf)), C.c_void_p(current_stream())),
              "fa4b_attn_check_status")


GLOBAL_SCALE_MODES = {"amax_per_bh": 0, "one": 1}


def make_dims(q: torch.Tensor, k: torch.Tensor, softmax_scale: float | None, pv_format: str, causal: bool = True,
              global_scale: str = "amax_per_bh") -> _lib.AttnDims:
    if pv_format not in PV_FORMATS:
        raise ValueError(f"unknown pv_format {pv_format!r}; expected one of {sorted(PV_FORMATS)}")
    if global_scale not in GLOBAL_SCALE_MODES:
        raise ValueError(f"unknown global_scale {global_scale!r}; expected one of {sorted(GLOBAL_SCALE_MODES)}")
    B, Hq, S, D = q.shape
    return _lib.AttnDims(B, Hq, k.shape[1], S, D, float(softmax_scale) if softmax_scale else 0.0, PV_FORMATS[pv_format],
                         0 if causal else 1, GLOBAL_SCALE_MODES[global_scale])


def ws_layout(dims: _lib.AttnDims) -> _lib.WsLayout:
    layout = _lib.WsLayout()
    check(lib().fa4b_attn_ws_layout_query(C.byref(dims), C.byref(layout)), "fa4b_attn_ws_layout_query")
    return layout


def _aligned_bytes(n: int, device) -> torch.Tensor:
    buf = torch.empty(n + 1024, dtype=torch.uint8, device=device)
    shift = (-buf.data_ptr()) % 1024
    return buf[shift:shift + n]


def alloc_workspace(dims: _lib.AttnDims, device, saved_only: bool = False) -> Workspace:
    """A workspace for ``dims``.  ``saved_only``: just the section the backward replays (Q/K codes, scale pages, E4M3
    operands); the backward then needs a scratch buffer (:func:`alloc_scratch`, :meth:`Workspace.with_scratch`)."""
    layout = ws_layout(dims)
    return Workspace(dims, layout, _aligned_bytes(layout.saved_total if saved_only else layout.total, device))


def alloc_scratch(dims: _lib.AttnDims, device) -> torch.Tensor:
    """The transient section of a backward call for ``dims`` as a buffer of its own."""
    layout = ws_layout(dims)
    return _aligned_bytes(layout.total - layout.saved_total, device)


_scratch_cache: dict = {}


def shared_scratch(dims: _lib.AttnDims, device) -> torch.Tensor:
    """One grow-only transient buffer per device, shared by every layer's backward (backward calls on one device are
    serial on the stream they share)."""
    layout = ws_layout(dims)
    need = layout.total - layout.saved_total
    key = torch.device(device)
    if key.index is None:
        key = torch.device("cuda", torch.cuda.current_device())
    have = _scratch_cache.get(key)
    if have is None or have.numel() < need:
        have = _aligned_bytes(need, key)
        _scratch_cache[key] = have
    return have[:need]


def backward_plan(dims: _lib.AttnDims, n_sm: int = 0) -> _lib.BwdPlan:
    """The work list :func:`attn_backward` launches for ``dims`` (host-only query; ``n_sm = 0``: the current device):
    ``chunk`` query tiles per work item, ``items_per_head``, ``grid`` and ``split_rows`` -- the leading key rows of
    every kv head whose dK / dV are summed in FP32 over several CTAs."""
    plan = _lib.BwdPlan()
    check(lib().fa4b_attn_bwd_plan(C.byref(dims), C.c_int32(n_sm), C.byref(plan)), "fa4b_attn_bwd_plan")
    return plan


def _ev(e) -> int:
    return 0 if e is None else e.cuda_event


def attn_forward(q, k, v, softmax_scale: float | None = None, pv_format: str = "e4m3_fp8", workspace: Workspace | None = None,
                 prepared: bool = False, events=(None, None), causal: bool = True, out: torch.Tensor | None = None,
                 global_scale: str = "amax_per_bh"):
    """O ``[B,Hq,S,D]`` bf16, LSE ``[B,Hq,S]`` f32 and the workspace holding the quantised operands.
    ``causal=False`` (forward only) lets every query see every key.  ``out`` receives O when given: a
    ``[B,Hq,S,D]``-shaped bf16 view with any strides (e.g. a permuted ``[B,S,Hq,D]`` buffer).
    ``global_scale="one"`` quantises Q and K with a unit global decode scale (block scale ``E4M3(block amax / 6)``,
    no statistics pass), as the reference's attention route does."""
    for t, n in ((q, "q"), (k, "k"), (v, "v")):
        _check_bhsd(t, n)
    if k.shape != v.shape or q.shape[0] != k.shape[0] or q.shape[2:] != k.shape[2:]:
        raise ValueError(f"inconsistent shapes q{tuple(q.shape)} k{tuple(k.shape)} v{tuple(v.shape)}")
    dims = make_dims(q, k, softmax_scale, pv_format, causal, global_scale)
    ws = workspace or alloc_workspace(dims, q.device)
    B, Hq, S, D = q.shape
    if out is None:
        o = torch.empty(B, Hq, S, D, dtype=torch.bfloat16, device=q.device)
    else:
        _check_bhsd(out, "out")
        if tuple(out.shape) != (B, Hq, S, D):
            raise ValueError(f"out must be shaped {(B, Hq, S, D)}, got {tuple(out.shape)}")
        o = out
    lse = torch.empty(B, Hq, S, dtype=torch.float32, device=q.device)
    a = _lib.AttnFwdArgs(dims, ptr(q), _strides(q), ptr(k), _strides(k), ptr(v), _strides(v), ptr(o), _strides(o), ptr(lse),
                         ptr(ws.buf), int(prepared), _ev(events[0]), _ev(events[1]))
    check(lib().fa4b_attn_fwd(C.byref(a), C.c_void_p(current_stream())), "fa4b_attn_fwd")
    return o, lse, ws


PREPARE_PHASES = {"all": 0, "amax": 1, "quantize": 2}


def attn_prepare(q, k, v, ws: Workspace, phase: str = "all") -> None:
    """Publish the quantised operands of q, k, v into ``ws`` (the first half of :func:`attn_forward`).
    ``phase="amax"`` only fills the per-(batch, head) amax words (``ws.amax()``), ``phase="quantize"`` publishes
    with the words found there: a sequence-sharded caller maximises them over shards and ranks in between."""
    a = _lib.AttnPrepareArgs(ws.dims, ptr(q), _strides(q), ptr(k), _strides(k), ptr(v), _strides(v), ptr(ws.buf), PREPARE_PHASES[phase])
    check(lib().fa4b_attn_prepare(C.byref(a), C.c_void_p(current_stream())), "fa4b_attn_prepare")


def attn_forward_prepared(ws: Workspace, kv_ws: Workspace | None = None, causal: bool = True, out: torch.Tensor | None = None):
    """Forward on operands already published: queries from ``ws``, keys and values from ``kv_ws`` (default ``ws``).
    ``causal=False`` lets every query see every key (an off-diagonal block of a sequence-sharded run); ``out`` as in
    :func:`attn_forward`."""
    d = ws.dims
    dims = _lib.AttnDims(d.B, d.Hq, d.Hkv, d.S, d.D, d.softmax_scale, d.pv_format, 0 if causal else 1, d.global_scale_mode)
    dev = ws.buf.device
    if out is None:
        o = torch.empty(d.B, d.Hq, d.S, d.D, dtype=torch.bfloat16, device=dev)
    else:
        _check_bhsd(out, "out")
        if tuple(out.shape) != (d.B, d.Hq, d.S, d.D):
            raise ValueError(f"out must be shaped {(d.B, d.Hq, d.S, d.D)}, got {tuple(out.shape)}")
        o = out
    lse = torch.empty(d.B, d.Hq, d.S, dtype=torch.float32, device=dev)
    z = _lib.Strides()
    a = _lib.AttnFwdArgs(dims, 0, z, 0, z, 0, z, ptr(o), _strides(o), ptr(lse), ptr(ws.buf), 1, 0, 0,
                         ptr(kv_ws.buf) if kv_ws is not None else 0)
    check(lib().fa4b_attn_fwd(C.byref(a), C.c_void_p(current_stream())), "fa4b_attn_fwd")
    return o, lse


def attn_merge(o_acc: torch.Tensor, lse_acc: torch.Tensor, o_part: torch.Tensor, lse_part: torch.Tensor, out: torch.Tensor | None = None):
    """Fold the partial result ``(o_part bf16, lse_part)`` into the running ``(o_acc f32, lse_acc)`` in place; with
    ``out`` (bf16) also write the merged rows there."""
    D = o_acc.shape[-1]
    n_rows = o_acc.numel() // D
    for t in (o_acc, lse_acc, o_part, lse_part) + ((out,) if out is not None else ()):
        if not t.is_contiguous():
            raise ValueError("attn_merge needs contiguous tensors")
    check(lib().fa4b_attn_merge(C.c_void_p(ptr(o_acc)), C.c_void_p(ptr(lse_acc)), C.c_void_p(ptr(o_part)), C.c_void_p(ptr(lse_part)),
                                C.c_int64(n_rows), C.c_int32(D), C.c_void_p(ptr(out) if out is not None else 0),
                                C.c_void_p(current_stream())), "fa4b_attn_merge")


def attn_backward(o, lse, dout, ws: Workspace, preprocessed: bool = False, events=(None, None), out=None,
                  dq_sums_fp32: bool = False):
    """dQ ``[B,Hq,S,D]``, dK, dV ``[B,Hkv,S,D]`` bf16, replaying the operands the forward cached in ``ws``.
    ``out=(dq, dk, dv)`` supplies the destinations: bf16 views of those shapes with any strides (e.g. the column
    ranges of one ``[B*S, (Hq + 2 Hkv) D]`` buffer).  At D = 128 the key tiles' partial dQ sums meet as f16 pairs
    (half the reduction traffic of FP32 sums; the sums of two runs differ in the last bits of bf16);
    ``dq_sums_fp32`` keeps them in FP32."""
    for t, n in ((o, "o"), (dout, "dout")):
        _check_bhsd(t, n)
    d = ws.dims
    if out is None:
        dq = torch.empty(d.B, d.Hq, d.S, d.D, dtype=torch.bfloat16, device=o.device)
        dk = torch.empty(d.B, d.Hkv, d.S, d.D, dtype=torch.bfloat16, device=o.device)
        dv = torch.empty_like(dk)
    else:
        dq, dk, dv = out
        for t, n, h in ((dq, "dq", d.Hq), (dk, "dk", d.Hkv), (dv, "dv", d.Hkv)):
            _check_bhsd(t, n)
            if tuple(t.shape) != (d.B, h, d.S, d.D):
                raise ValueError(f"{n} must be shaped {(d.B, h, d.S, d.D)}, got {tuple(t.shape)}")
    a = _lib.AttnBwdArgs(d, ptr(o), _strides(o), ptr(dout), _strides(dout), ptr(lse), ptr(dq), _strides(dq), ptr(dk), _strides(dk),
                         ptr(dv), _strides(dv), ptr(ws.buf), int(preprocessed), _ev(events[0]), _ev(events[1]), 0,
                         BWD_DQ_SUMS_FP32 if dq_sums_fp32 else 0, ptr(ws.scratch))
    check(lib().fa4b_attn_bwd(C.byref(a), C.c_void_p(current_stream())), "fa4b_attn_bwd")
    return dq, dk, dv


BWD_KEEP_DQ_ACCUM, BWD_SKIP_DQ_OUT, BWD_DQ_SUMS_FP32 = 1, 2, 4


def attn_backward_prepared(ws: Workspace, kv_ws: Workspace | None = None, causal: bool = True, keep_dq_accum: bool = False,
                           write_dq: bool = True, out=None):
    """Backward block call on published operands and statistics: queries, dO and the row statistics from ``ws``
    (:func:`attn_bwd_preprocess` has run on it with the LSE and O of the whole sequence), keys and values from
    ``kv_ws`` (default ``ws``).  Returns ``(dq | None, dk, dv)``: dK and dV of this block alone (bf16); the query
    gradient accumulates in ``ws``'s FP32 scratch across calls with ``keep_dq_accum`` and is only converted into
    ``dq`` when ``write_dq`` (a sum over several calls starts with ``write_dq=False``; a single call with the
    defaults forms its sum as f16 pairs, as :func:`attn_backward` does).  ``out=(dq, dk, dv)`` supplies strided destinations as in :func:`attn_backward`."""
    d = ws.dims
    dims = _lib.AttnDims(d.B, d.Hq, d.Hkv, d.S, d.D, d.softmax_scale, d.pv_format, 0 if causal else 1, d.global_scale_mode)
    dev = ws.buf.device
    if out is None:
        dq = torch.empty(d.B, d.Hq, d.S, d.D, dtype=torch.bfloat16, device=dev) if write_dq else None
        dk = torch.empty(d.B, d.Hkv, d.S, d.D, dtype=torch.bfloat16, device=dev)
        dv = torch.empty_like(dk)
    else:
        dq, dk, dv = out
        for t, n, h in ((dq, "dq", d.Hq), (dk, "dk", d.Hkv), (dv, "dv", d.Hkv)):
            if t is None and n == "dq" and not write_dq:
                continue
            _check_bhsd(t, n)
            if tuple(t.shape) != (d.B, h, d.S, d.D):
                raise ValueError(f"{n} must be shaped {(d.B, h, d.S, d.D)}, got {tuple(t.shape)}")
    z = _lib.Strides()
    flags = (BWD_KEEP_DQ_ACCUM if keep_dq_accum else 0) | (0 if write_dq else BWD_SKIP_DQ_OUT)
    a = _lib.AttnBwdArgs(dims, 0, z, 0, z, 0, ptr(dq) if write_dq else 0, _strides(dq) if write_dq else z, ptr(dk), _strides(dk),
                         ptr(dv), _strides(dv), ptr(ws.buf), 1, 0, 0, ptr(kv_ws.buf) if kv_ws is not None else 0, flags, ptr(ws.scratch))
    check(lib().fa4b_attn_bwd(C.byref(a), C.c_void_p(current_stream())), "fa4b_attn_bwd")
    return dq, dk, dv


def attn_accumulate(acc: torch.Tensor, part: torch.Tensor, out: torch.Tensor | None = None) -> None:
    """``acc (f32) += part (bf16)`` in place; with ``out`` (bf16) also write the sums there."""
    for t in (acc, part) + ((out,) if out is not None else ()):
        if not t.is_contiguous():
            raise ValueError("attn_accumulate needs contiguous tensors")
    check(lib().fa4b_attn_accumulate(C.c_void_p(ptr(acc)), C.c_void_p(ptr(part)), C.c_int64(acc.numel()),
                                     C.c_void_p(ptr(out) if out is not None else 0), C.c_void_p(current_stream())), "fa4b_attn_accumulate")


def attn_bwd_preprocess(o, lse, dout, ws: Workspace):
    d = ws.dims
    a = _lib.AttnBwdArgs(d, ptr(o), _strides(o), ptr(dout), _strides(dout), ptr(lse), 0, _lib.Strides(), 0, _lib.Strides(), 0,
                         _lib.Strides(), ptr(ws.buf), 0, 0, 0, 0, 0, ptr(ws.scratch))
    check(lib().fa4b_attn_bwd_preprocess(C.byref(a), C.c_void_p(current_stream())), "fa4b_attn_bwd_preprocess")
    ops = ws.operands()
    return ops["do_fp8"], ops["dstat"], ops["lstat"]

"""Drop-in operator boundary: the attention-op signature, ModelConverter and
``fa4.*`` config fields of torchtitan/experiments/fa4 in the reference
(fa4_attention.py:358-608, job_config.py:33-96, exact_lowp_attention.py:60-95).

``FA4AttentionWrapper.forward(q, k, v, *, score_mod=None, scale=None)`` takes
``[B,H,S,D]`` tensors, is always causal, and returns ``[B,Hq,S,D]``.  The
operator is registered with ``torch.library`` as ``fa4b::attn_fwd`` /
``fa4b::attn_bwd`` so that it composes with autograd; both run the CUDA
kernels through the C ABI and raise on anything unsupported -- there is no
fallback to another attention implementation.
"""

from __future__ import annotations

import threading
from dataclasses import dataclass
from typing import Callable, Literal

import torch
import torch.nn as nn

from . import attention

_EXACT_FP8_PV = "e4m3_fp8"
_EXACT_MXFP4_PV = "mxfp4_e8m0_block32"
_EXACT_PV_FORMATS = (_EXACT_FP8_PV, _EXACT_MXFP4_PV)
_EXACT_LEARNED_PROJECTION_FORMATS = ("e4m3", "nvfp4")
# (projection format, P/V format) -> route name, as in exact_lowp_attention.py:84-95
EXACT_ROUTE_BY_FORMATS = {
    ("nvfp4", _EXACT_FP8_PV): "nvfp4_qk_fp8_pv",
    ("nvfp4", _EXACT_MXFP4_PV): "nvfp4_qk_mxfp4_pv",
    ("e4m3", _EXACT_FP8_PV): "e4m3_proj_nvfp4_qk_fp8_pv",
    ("e4m3", _EXACT_MXFP4_PV): "e4m3_proj_nvfp4_qk_mxfp4_pv",
}


@dataclass
class FA4:
    """The ``[fa4]`` table of the job config; only the fields that select the attention route
    are kept (job_config.py:33-96 of the reference)."""

    enabled: bool = True
    mode: Literal["softmax", "softcap", "sigmoid_attention"] = "softmax"
    exact_pv_format: Literal["e4m3_fp8", "mxfp4_e8m0_block32"] | None = "e4m3_fp8"
    exact_learned_projection_format: Literal["e4m3", "nvfp4"] = "e4m3"
    exact_forward_batch_size: int = 1


@dataclass(frozen=True)
class ResolvedFA4Config:
    mode: str
    pv_format: str
    route: str


def resolve_fa4_config(cfg) -> ResolvedFA4Config:
    """Fail closed on anything but the softmax low-precision routes."""
    fa4 = getattr(cfg, "fa4", cfg)
    if not getattr(fa4, "enabled", True):
        raise ValueError("fa4.enabled is false but the fa4 attention converter was requested")
    mode = getattr(fa4, "mode", "softmax")
    if mode != "softmax":
        raise ValueError(f"Unsupported fa4.mode={mode!r}: this build has the softmax route only")
    pv = getattr(fa4, "exact_pv_format", _EXACT_FP8_PV) or _EXACT_FP8_PV
    if pv not in _EXACT_PV_FORMATS:
        raise ValueError(f"fa4.exact_pv_format must be one of {_EXACT_PV_FORMATS}, got {pv!r}")
    proj = getattr(fa4, "exact_learned_projection_format", "e4m3")
    if proj not in _EXACT_LEARNED_PROJECTION_FORMATS:
        raise ValueError(f"fa4.exact_learned_projection_format must be one of {_EXACT_LEARNED_PROJECTION_FORMATS}, got {proj!r}")
    return ResolvedFA4Config(mode=mode, pv_format=pv, route=EXACT_ROUTE_BY_FORMATS[(proj, pv)])


# --------------------------------------------------------------------------- torch.library ops
_PV_CODE = attention.PV_FORMATS


@torch.library.custom_op("fa4b::attn_fwd", mutates_args=())
def _attn_fwd_op(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float, pv_code: int) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    pv = _EXACT_FP8_PV if pv_code == 0 else _EXACT_MXFP4_PV
    # only the saved section of the operand cache is allocated here and kept for the backward: the quantised
    # operands, as the reference saves them (release/routes.json:443-447); the backward's dO / statistics /
    # FP32 accumulators live in one scratch buffer per device that every layer shares
    dims = attention.make_dims(q, k, scale if scale > 0 else None, pv)
    ws = attention.alloc_workspace(dims, q.device, saved_only=True)
    o, lse, ws = attention.attn_forward(q, k, v, softmax_scale=scale if scale > 0 else None, pv_format=pv, workspace=ws)
    return o, lse, ws.buf


@_attn_fwd_op.register_fake
def _(q, k, v, scale, pv_code):
    B, Hq, S, D = q.shape
    dims = attention._lib.AttnDims(B, Hq, k.shape[1], S, D, scale if scale > 0 else 0.0, pv_code)
    saved = attention.ws_layout(dims).saved_total  # host-only query: the real op returns exactly these bytes
    return (q.new_empty(B, Hq, S, D), q.new_empty(B, Hq, S, dtype=torch.float32), q.new_empty(saved, dtype=torch.uint8))


@torch.library.custom_op("fa4b::attn_bwd", mutates_args=("ws",))
def _attn_bwd_op(o: torch.Tensor, lse: torch.Tensor, dout: torch.Tensor, ws: torch.Tensor, Hkv: int, scale: float,
                 pv_code: int) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    B, Hq, S, D = o.shape
    dims = attention._lib.AttnDims(B, Hq, Hkv, S, D, scale if scale > 0 else 0.0, pv_code)
    layout = attention.ws_layout(dims)
    if ws.numel() != layout.saved_total or ws.data_ptr() % 1024:
        raise RuntimeError("the saved operand cache does not match this call's shape")
    work = attention.Workspace(dims, layout, ws).with_scratch(attention.shared_scratch(dims, o.device))
    grads = attention.attn_backward(o, lse, dout, work)
    return grads


@_attn_bwd_op.register_fake
def _(o, lse, dout, ws, Hkv, scale, pv_code):
    B, Hq, S, D = o.shape
    return o.new_empty(B, Hq, S, D), o.new_empty(B, Hkv, S, D), o.new_empty(B, Hkv, S, D)


def _setup_context(ctx, inputs, output):
    q, k, v, scale, pv_code = inputs
    o, lse, ws = output
    ctx.save_for_backward(o, lse, ws)
    ctx.Hkv, ctx.scale, ctx.pv_code = k.shape[1], scale, pv_code
    ctx.stream = torch.cuda.current_stream() if q.is_cuda else None


def _backward(ctx, do, _dlse, _dws):
    o, lse, ws = ctx.saved_tensors
    # backward must run on the forward's stream (benchmark_llama12b_e2e.py:6206-6210 of the reference)
    if ctx.stream is not None and torch.cuda.current_stream() != ctx.stream:
        raise RuntimeError("fa4b attention backward must run on the stream of its forward")
    if do.stride(-1) != 1:
        do = do.contiguous()
    dq, dk, dv = torch.ops.fa4b.attn_bwd(o, lse, do, ws, ctx.Hkv, ctx.scale, ctx.pv_code)
    return dq, dk, dv, None, None


_attn_fwd_op.register_autograd(_backward, setup_context=_setup_context)


def fa4_func(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, *, softmax_scale: float | None = None, causal: bool = True,
             pv_format: str = _EXACT_FP8_PV) -> torch.Tensor:
    """Causal low-precision attention on ``[B,H,S,D]`` views; differentiable."""
    if not causal:
        raise NotImplementedError("only the causal training route is built")
    if pv_format not in _PV_CODE:
        raise ValueError(f"unknown pv_format {pv_format!r}")
    o, _lse, _ws = torch.ops.fa4b.attn_fwd(q, k, v, float(softmax_scale) if softmax_scale else 0.0, _PV_CODE[pv_format])
    return o


class FA4AttentionWrapper(nn.Module):
    """``inner_attention`` replacement (fa4_attention.py:507-548 of the reference)."""

    def __init__(self, config: ResolvedFA4Config, head_dim: int):
        super().__init__()
        self.config = config
        self.head_dim = head_dim

    def forward(self, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, *, score_mod: Callable | None = None,
                scale: float | None = None, **unused) -> torch.Tensor:
        if score_mod is not None:
            raise NotImplementedError(
                "FA4AttentionWrapper does not accept an external score_mod; configure low_bits_training.fa4 instead.")
        if unused.get("block_mask") is not None or unused.get("attention_masks") is not None:
            raise NotImplementedError("FA4AttentionWrapper is causal-only and takes no attention mask")
        if q.shape[-1] != self.head_dim:
            raise ValueError(f"head dim {q.shape[-1]} does not match the converted module's {self.head_dim}")
        target = torch.get_autocast_dtype("cuda") if torch.is_autocast_enabled() else q.dtype
        if target != torch.bfloat16:
            raise TypeError(f"the low-precision route runs on bfloat16 activations, got {target}")
        q, k, v = (t.to(target) if t.dtype != target else t for t in (q, k, v))
        # no transposes or copies: the kernels read [B,H,S,D] views through their strides
        return fa4_func(q, k, v, softmax_scale=scale, causal=True, pv_format=self.config.pv_format)


_patch_lock = threading.Lock()


def patch_attention_modules(model: nn.Module, config: ResolvedFA4Config) -> int:
    """Replace ``inner_attention`` on every module that has it and a ``head_dim``
    (fa4_attention.py:551-570 of the reference)."""
    patched = 0
    with _patch_lock:
        for module in model.modules():
            if not hasattr(module, "inner_attention") or not hasattr(module, "head_dim"):
                continue
            if isinstance(module.inner_attention, FA4AttentionWrapper):
                continue
            if module.head_dim not in (64, 128):
                raise ValueError(f"head_dim {module.head_dim} is not built (64 and 128 are)")
            module.inner_attention = FA4AttentionWrapper(config=config, head_dim=module.head_dim)
            if hasattr(module, "use_flex_attn"):
                module.use_flex_attn = False
            if hasattr(module, "attn_score_modifier"):
                module.attn_score_modifier = None
            patched += 1
    return patched


class FA4AttentionConverter:
    """TorchTitan ModelConverter (torchtitan/protocols/model_converter.py): select it with
    ``model.converters = ["fa4_attention"]``."""

    def __init__(self, job_config, parallel_dims=None):
        self.config = resolve_fa4_config(job_config)

    def convert(self, model: nn.Module):
        patched = patch_attention_modules(model, self.config)
        if patched == 0:
            raise RuntimeError("fa4_attention found no module with inner_attention and head_dim to patch")
        self.patched = patched

    def post_optimizer_hook(self, model):
        pass


def register_with_torchtitan(name: str = "fa4_attention") -> bool:
    """Register the converter under the reference's name when TorchTitan is importable."""
    try:
        from torchtitan.protocols.model_converter import _registry_model_converter_cls, register_model_converter
    except Exception:
        return False
    if name not in _registry_model_converter_cls:
        register_model_converter(FA4AttentionConverter, name)
    return True

"""Module-level forward of the low-precision attention block: hidden states in, hidden states out.

Mirrors the forward of ``ExactLowpFA4Attention.forward(x, freqs_cis, None)``
(torchtitan/experiments/fa4/exact_lowp_attention.py:3789-3969) with the operand formats of the reference's D128
NVFP4 projection route (tk_fa4/interface.py:5238, b300_project_qkv_gqa_d128_unified_lowp_nvfp4): the activation
rows are quantised to NVFP4 (1x16 blocks), the stacked Q/K/V weight and the output weight to NVFP4 with one scale
per 16x16 tile, both projections run as block-scaled FP4 GEMMs, Q and K rotate in the pair-native order in packed
BF16, and the attention core is the NVFP4 Q.K^T / FP8 P.V kernel.  The reference fuses rotation, quantisation and
publication into the projection epilogues; here they are separate launches on the same stream.
"""

from __future__ import annotations

import torch

from . import attention
from .quantizers import prepare_nvfp4_projection_weight_dual, project_nvfp4, rope_pair_, tk_quantize_for_gemm


def pair_interleave_qk_rows(weight: torch.Tensor, n_heads: int, head_dim: int) -> torch.Tensor:
    """Reorder the output rows of a Q or K projection weight ``[n_heads*head_dim, hidden]`` from the split-half
    rotary order ``[x_0 .. x_{D/2-1}, y_0 .. y_{D/2-1}]`` to adjacent pairs ``[x_0, y_0, x_1, y_1, ...]`` per head
    (b300_pair_interleave_qk_projection_weights, tk_fa4/interface.py:6496-6533).  Q.K^T does not see the common
    permutation."""
    if weight.ndim != 2 or weight.shape[0] != n_heads * head_dim or head_dim % 2:
        raise ValueError("weight must be [n_heads*head_dim, hidden] with an even head_dim")
    w = weight.reshape(n_heads, 2, head_dim // 2, weight.shape[1])
    return w.permute(0, 2, 1, 3).reshape(n_heads * head_dim, weight.shape[1]).contiguous()


class LowpFA4AttentionBlock:
    """Prepared weights plus the forward pass.  Weights are ``nn.Linear``-style ``[out, in]`` bf16 CUDA tensors; the
    rows of ``wq`` / ``wk`` are expected in the pair-native rotary order (see :func:`pair_interleave_qk_rows`)."""

    def __init__(self, wq: torch.Tensor, wk: torch.Tensor, wv: torch.Tensor, wo: torch.Tensor, n_heads: int, n_kv_heads: int,
                 head_dim: int):
        hidden = wq.shape[1]
        if head_dim not in (64, 128):
            raise ValueError(f"head_dim {head_dim}: the attention core supports 64 and 128")
        if n_heads % n_kv_heads:
            raise ValueError("n_heads must be a multiple of n_kv_heads")
        for name, w, rows in (("wq", wq, n_heads * head_dim), ("wk", wk, n_kv_heads * head_dim), ("wv", wv, n_kv_heads * head_dim)):
            if tuple(w.shape) != (rows, hidden):
                raise ValueError(f"{name} must be {(rows, hidden)}, got {tuple(w.shape)}")
        if tuple(wo.shape) != (hidden, n_heads * head_dim):
            raise ValueError(f"wo must be {(hidden, n_heads * head_dim)}, got {tuple(wo.shape)}")
        n_qkv = (n_heads + 2 * n_kv_heads) * head_dim
        if n_qkv % 256 or hidden % 256 or (n_heads * head_dim) % 256:
            raise ValueError("projection widths must be multiples of 256 (tile width of the FP4 GEMM)")
        self.n_heads, self.n_kv_heads, self.head_dim, self.hidden = n_heads, n_kv_heads, head_dim, hidden
        # quantised once; a cached result is valid only until the next optimizer update of the weight
        self.w_qkv, self.w_qkv_t = prepare_nvfp4_projection_weight_dual(torch.cat((wq, wk, wv), dim=0).contiguous())
        self.w_o, self.w_o_t = prepare_nvfp4_projection_weight_dual(wo.contiguous())

    def forward(self, x: torch.Tensor, rope_cos: torch.Tensor, rope_sin: torch.Tensor, attention_masks=None,
                softmax_scale: float | None = None, return_intermediates: bool = False):
        """``x [B,S,hidden]`` bf16 -> ``[B,S,hidden]`` bf16; causal attention only (``attention_masks`` must be None,
        as in the reference module)."""
        if attention_masks is not None:
            raise ValueError("causal attention_masks=None only")
        if x.ndim != 3 or x.shape[2] != self.hidden or x.dtype != torch.bfloat16 or not x.is_cuda:
            raise ValueError(f"x must be a CUDA bfloat16 [B, S, {self.hidden}] tensor")
        B, S, _ = x.shape
        if (B * S) % 128 or S % 128:
            raise ValueError("B*S and S must be multiples of 128")
        Hq, Hkv, D = self.n_heads, self.n_kv_heads, self.head_dim
        rows = x.reshape(B * S, self.hidden)
        if not rows.is_contiguous():
            rows = rows.contiguous()
        a_codes, a_pages, _, _, a_g, _ = tk_quantize_for_gemm(rows, return_transpose=False)
        qkv = project_nvfp4((a_codes, a_pages, a_g), self.w_qkv)                 # [B*S, (Hq + 2 Hkv) D]
        q = qkv[:, :Hq * D].view(B, S, Hq, D)
        k = qkv[:, Hq * D:(Hq + Hkv) * D].view(B, S, Hkv, D)
        v = qkv[:, (Hq + Hkv) * D:].view(B, S, Hkv, D)
        rope_pair_(q, rope_cos, rope_sin)
        rope_pair_(k, rope_cos, rope_sin)
        o_rows = torch.empty(B * S, Hq * D, dtype=torch.bfloat16, device=x.device)
        o, lse, ws = attention.attn_forward(q.permute(0, 2, 1, 3), k.permute(0, 2, 1, 3), v.permute(0, 2, 1, 3), softmax_scale,
                                            out=o_rows.view(B, S, Hq, D).permute(0, 2, 1, 3))
        o_codes, o_pages, _, _, o_g, _ = tk_quantize_for_gemm(o_rows, return_transpose=False)
        y = project_nvfp4((o_codes, o_pages, o_g), self.w_o).view(B, S, self.hidden)
        if return_intermediates:
            return y, {"qkv": qkv, "o": o_rows, "lse": lse, "workspace": ws}
        return y

    __call__ = forward

"""Module-level forward of the low-precision attention block: hidden states in, hidden states out.

Mirrors the forward of ``ExactLowpFA4Attention.forward(x, freqs_cis, None)``
(torchtitan/experiments/fa4/exact_lowp_attention.py:3789-3969) with the operand formats of the reference's D128
NVFP4 projection route (tk_fa4/interface.py:5238, b300_project_qkv_gqa_d128_unified_lowp_nvfp4): the activation
rows are quantised to NVFP4 (1x16 blocks), the stacked Q/K/V weight and the output weight to NVFP4 with one scale
per 16x16 tile, both projections run as block-scaled FP4 GEMMs, Q and K rotate in the pair-native order in packed
BF16, and the attention core is the NVFP4 Q.K^T / FP8 P.V kernel.  With ``fused_publish=True`` rotation, Q/K/V
quantisation and publication run in the QKV projection's epilogue and the dO / statistics publication in the output
projection's input-gradient epilogue, as in the reference; otherwise they are separate launches on the same stream.
The projections write their wait status into one status tensor of the block and never synchronise the host;
``check_status()`` reads it (and a workspace's) on demand.
"""

from __future__ import annotations

import torch

from . import attention
from . import _lib
from .quantizers import (pack_qkv_grads, prepare_nvfp4_projection_weight_dual, project_dout_publish, project_nvfp4, project_qkv_publish, rope_pair_,
                         tk_quantize_for_gemm)


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
                 head_dim: int, fused_publish: bool = False, global_scale: str | None = None):
        """``fused_publish`` runs the QKV projection with rotation, quantisation and publication of the attention
        operands in its epilogue (head_dim 128; implies the unit global scale of the reference's attention route);
        ``global_scale`` ("amax_per_bh" or "one") chooses the Q/K recipe of the unfused path."""
        hidden = wq.shape[1]
        if fused_publish and head_dim != 128:
            raise ValueError("the fused publication serves head_dim 128")
        if fused_publish and global_scale not in (None, "one"):
            raise ValueError("the fused publication quantises Q and K at the unit global scale")
        self.fused_publish = bool(fused_publish)
        self.global_scale = "one" if fused_publish else (global_scale or "amax_per_bh")
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
        self._status = None  # [6, 4] u32 on the block's device: one slot per projection GEMM of a step

    def _slot(self, device, i: int) -> torch.Tensor:
        if self._status is None or self._status.device != torch.device(device):
            self._status = torch.zeros(6, 4, dtype=torch.int32, device=device)
        return self._status[i]

    def check_status(self, workspace=None) -> None:
        """One host synchronisation: raises if a device-side wait of any projection since the last check (or of the
        attention kernels that last used ``workspace``) gave up."""
        if self._status is not None:
            st = self._status.cpu()
            bad = [(i, st[i].tolist()) for i in range(st.shape[0]) if int(st[i, 0]) != 0]
            if bad:
                raise TimeoutError(f"projection GEMM wait status (slot, [flag, site, block, detail]): {bad}")
        if workspace is not None:
            workspace.check_status()

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
        # with a backward to follow, the token-major (column) operand of the weight-gradient GEMM comes from the same pass
        a_codes, a_pages, x_c, x_cp, a_g, _ = tk_quantize_for_gemm(rows, return_transpose=return_intermediates, encode_centric=False)
        x_cols = (x_c, x_cp, a_g) if return_intermediates else None
        o_rows = torch.empty(B * S, Hq * D, dtype=torch.bfloat16, device=x.device)
        o_view = o_rows.view(B, S, Hq, D).permute(0, 2, 1, 3)
        if self.fused_publish:
            dims = _lib.AttnDims(B, Hq, Hkv, S, D, float(softmax_scale) if softmax_scale else 0.0, attention.PV_FORMATS["e4m3_fp8"], 0,
                                 attention.GLOBAL_SCALE_MODES["one"])
            ws = attention.alloc_workspace(dims, x.device)
            project_qkv_publish((a_codes, a_pages, a_g), self.w_qkv, rope_cos, rope_sin, ws, status=self._slot(x.device, 0))
            _, lse = attention.attn_forward_prepared(ws, out=o_view)
            qkv = None
            return self._finish(o_rows, lse, ws, qkv, rows, x_cols, B, S, return_intermediates)
        qkv = project_nvfp4((a_codes, a_pages, a_g), self.w_qkv, status=self._slot(x.device, 0))                 # [B*S, (Hq + 2 Hkv) D]
        q = qkv[:, :Hq * D].view(B, S, Hq, D)
        k = qkv[:, Hq * D:(Hq + Hkv) * D].view(B, S, Hkv, D)
        v = qkv[:, (Hq + Hkv) * D:].view(B, S, Hkv, D)
        rope_pair_(q, rope_cos, rope_sin)
        rope_pair_(k, rope_cos, rope_sin)
        _, lse, ws = attention.attn_forward(q.permute(0, 2, 1, 3), k.permute(0, 2, 1, 3), v.permute(0, 2, 1, 3), softmax_scale,
                                            out=o_view, global_scale=self.global_scale)
        return self._finish(o_rows, lse, ws, qkv, rows, x_cols, B, S, return_intermediates)

    def _finish(self, o_rows, lse, ws, qkv, rows, x_cols, B, S, return_intermediates):
        o_codes, o_pages, o_c, o_cp, o_g, _ = tk_quantize_for_gemm(o_rows, return_transpose=return_intermediates, encode_centric=False)
        y = project_nvfp4((o_codes, o_pages, o_g), self.w_o, status=self._slot(o_rows.device, 1)).view(B, S, self.hidden)
        if return_intermediates:
            return y, {"qkv": qkv, "o": o_rows, "lse": lse, "workspace": ws, "x_rows": rows, "x_cols": x_cols, "o_cols": (o_c, o_cp, o_g)}
        return y

    __call__ = forward

    def backward(self, dy: torch.Tensor, saved: dict, rope_cos: torch.Tensor, rope_sin: torch.Tensor):
        """Gradients of :meth:`forward` from ``dy [B,S,hidden]`` and the intermediates the forward returned:
        ``(dx [B,S,hidden], dwq, dwk, dwv, dwo)``, all bf16.  Every GEMM is the NVFP4 projection kernel: the input
        gradients multiply the row-quantised upstream gradient with the transposed weight operand of the dual
        publication, the weight gradients multiply the two column-quantised (token-major blocks) activations --
        the operand formats of b300_mha_bwd_adaptive_lowp_hierarchical_nvfp4_qkv_projection_dgrad
        (tk_fa4/interface.py:6313-6441); the query and key gradients turn back through the inverse rotation."""
        Hq, Hkv, D = self.n_heads, self.n_kv_heads, self.head_dim
        B, S, _ = dy.shape
        M = B * S
        if M % 256:
            raise ValueError("B*S must be a multiple of 256 (the weight-gradient GEMMs contract over the tokens)")
        dy_rows = dy.reshape(M, self.hidden)
        if not dy_rows.is_contiguous():
            dy_rows = dy_rows.contiguous()
        o_rows, lse, ws = saved["o"], saved["lse"], saved["workspace"]
        # output projection: dO = dY . Wo, dWo = dY^T . O
        dy_r, dy_rp, dy_c, dy_cp, dy_g, _ = tk_quantize_for_gemm(dy_rows, return_transpose=True, encode_centric=False)
        fused = self.fused_publish
        if fused:  # dO goes straight into the workspace as E5M2 with its row statistics
            project_dout_publish((dy_r, dy_rp, dy_g), self.w_o_t, o_rows, lse, ws, status=self._slot(dy.device, 2))
        else:
            do_rows = project_nvfp4((dy_r, dy_rp, dy_g), self.w_o_t, status=self._slot(dy.device, 2))                           # [M, Hq D]
        dwo = project_nvfp4((dy_c, dy_cp, dy_g), saved["o_cols"], status=self._slot(dy.device, 3))                              # [hidden, Hq D]
        # attention core, gradients written into the columns of one [M, (Hq + 2 Hkv) D] buffer
        dqkv = torch.empty(M, (Hq + 2 * Hkv) * D, dtype=torch.bfloat16, device=dy.device)
        dq = dqkv[:, :Hq * D].view(B, S, Hq, D)
        dk = dqkv[:, Hq * D:(Hq + Hkv) * D].view(B, S, Hkv, D)
        dv = dqkv[:, (Hq + Hkv) * D:].view(B, S, Hkv, D)
        grads = (dq.permute(0, 2, 1, 3), dk.permute(0, 2, 1, 3), dv.permute(0, 2, 1, 3))
        if fused:
            attention.attn_backward_prepared(ws, out=grads)
        else:
            attention.attn_backward(o_rows.view(B, S, Hq, D).permute(0, 2, 1, 3), lse, do_rows.view(B, S, Hq, D).permute(0, 2, 1, 3), ws,
                                    out=grads)
        # QKV projection: dX = dQKV . Wqkv, dWqkv = dQKV^T . X; the inverse rotation of dQ and dK happens while the
        # gradients are packed
        g_r, g_rp, g_c, g_cp, g_g, _ = pack_qkv_grads(dq, dk, dv, rope_cos, rope_sin, return_transpose=True, encode_centric=False)
        dx = project_nvfp4((g_r, g_rp, g_g), self.w_qkv_t, status=self._slot(dy.device, 4)).view(B, S, self.hidden)
        dwqkv = project_nvfp4((g_c, g_cp, g_g), saved["x_cols"], status=self._slot(dy.device, 5))                               # [(Hq + 2 Hkv) D, hidden]
        return dx, dwqkv[:Hq * D], dwqkv[Hq * D:(Hq + Hkv) * D], dwqkv[(Hq + Hkv) * D:], dwo


class _BlockFunction(torch.autograd.Function):
    """Autograd binding of :class:`LowpFA4AttentionBlock` (the role of _LowpAttentionFunction,
    tk_fa4/lowp_fa4_bwd/benchmark_llama12b_e2e.py:5841-6546); backward runs on the stream of the forward."""

    @staticmethod
    def forward(ctx, x, wq, wk, wv, wo, block, rope_cos, rope_sin):
        y, saved = block.forward(x, rope_cos, rope_sin, return_intermediates=True)
        ctx.block, ctx.saved, ctx.tables = block, saved, (rope_cos, rope_sin)
        return y

    @staticmethod
    def backward(ctx, dy):
        dx, dwq, dwk, dwv, dwo = ctx.block.backward(dy, ctx.saved, *ctx.tables)
        ctx.saved = None
        return dx, dwq, dwk, dwv, dwo, None, None, None


class LowpFA4Attention(torch.nn.Module):
    """Trainable module: ``forward(x, (rope_cos, rope_sin), attention_masks=None) -> [B,S,hidden]``.  The parameters
    keep the names of TorchTitan's Llama ``Attention`` (``wq``, ``wk``, ``wv``, ``wo`` as ``nn.Linear`` without
    bias), so a checkpoint of the original module loads unchanged; ``wq`` / ``wk`` rows are expected in the
    pair-native rotary order.  The quantised weight operands are rebuilt whenever a parameter has changed
    (optimizer step, ``load_state_dict``), as the reference requires of a cached preparation."""

    def __init__(self, hidden: int, n_heads: int, n_kv_heads: int, head_dim: int, device="cuda", linears=None, fused_publish: bool = False):
        super().__init__()
        self.fused_publish = bool(fused_publish)
        self.n_heads, self.n_kv_heads, self.head_dim = n_heads, n_kv_heads, head_dim
        self.n_rep = n_heads // n_kv_heads
        self.use_flex_attn = False
        if linears is None:
            mk = lambda o, i: torch.nn.Linear(i, o, bias=False, device=device, dtype=torch.bfloat16)
            linears = (mk(n_heads * head_dim, hidden), mk(n_kv_heads * head_dim, hidden), mk(n_kv_heads * head_dim, hidden),
                       mk(hidden, n_heads * head_dim))
        self.wq, self.wk, self.wv, self.wo = linears
        self._block, self._versions = None, None
        self._tables = None

    @classmethod
    def from_attention(cls, original: torch.nn.Module) -> "LowpFA4Attention":
        """Take over the projections of a TorchTitan Llama ``Attention`` (same ``nn.Linear`` objects, so the
        state-dict keys and the optimizer's parameters stay what they were), as ``ExactLowpFA4Attention(original, ...)``
        does (exact_lowp_attention.py:3792-3830).  TorchTitan rotates adjacent pairs, the order used here."""
        for name in ("wq", "wk", "wv", "wo", "n_heads", "n_kv_heads", "head_dim"):
            if not hasattr(original, name):
                raise TypeError(f"{type(original).__name__} has no attribute {name!r}: not a Llama-style attention module")
        for lin in (original.wq, original.wk, original.wv, original.wo):
            if not isinstance(lin, torch.nn.Linear) or lin.bias is not None:
                raise TypeError("the projections must be bias-free nn.Linear modules")
            if lin.weight.dtype != torch.bfloat16:
                raise TypeError(f"the low-precision block runs on bfloat16 weights, got {lin.weight.dtype}")
        return cls(original.wq.in_features, int(original.n_heads), int(original.n_kv_heads), int(original.head_dim),
                   linears=(original.wq, original.wk, original.wv, original.wo))

    def _rope_tables(self, freqs):
        """(cos, sin) bf16 [S, D/2] from a pair of tables or from TorchTitan's complex ``freqs_cis [S, D/2]``."""
        if isinstance(freqs, (tuple, list)):
            return freqs
        if not torch.is_complex(freqs) or freqs.ndim != 2:
            raise TypeError("freqs must be (cos, sin) tables or a complex [S, D/2] tensor")
        key = (freqs.data_ptr(), tuple(freqs.shape), freqs._version)
        if self._tables is None or self._tables[0] != key:
            self._tables = (key, freqs.real.to(torch.bfloat16).contiguous(), freqs.imag.to(torch.bfloat16).contiguous())
        return self._tables[1], self._tables[2]

    def _prepared(self) -> LowpFA4AttentionBlock:
        ws = (self.wq.weight, self.wk.weight, self.wv.weight, self.wo.weight)
        versions = tuple((w.data_ptr(), w._version) for w in ws)
        if self._block is None or versions != self._versions:
            with torch.no_grad():
                self._block = LowpFA4AttentionBlock(*(w.detach() for w in ws), self.n_heads, self.n_kv_heads, self.head_dim,
                                                    fused_publish=self.fused_publish)
            self._versions = versions
        return self._block

    def forward(self, x: torch.Tensor, freqs, attention_masks=None) -> torch.Tensor:
        if attention_masks is not None:
            raise ValueError("causal attention_masks=None only")
        rope_cos, rope_sin = self._rope_tables(freqs)
        S = x.shape[1]
        if rope_cos.shape[0] != S:  # TorchTitan hands over the table of the longest sequence
            rope_cos, rope_sin = rope_cos[:S].contiguous(), rope_sin[:S].contiguous()
        return _BlockFunction.apply(x, self.wq.weight, self.wk.weight, self.wv.weight, self.wo.weight, self._prepared(), rope_cos, rope_sin)


def replace_attention_modules(model: torch.nn.Module) -> int:
    """Swap every Llama-style attention module of ``model`` (attributes ``wq, wk, wv, wo, n_heads, n_kv_heads,
    head_dim``) for a :class:`LowpFA4Attention` that shares its projections; returns how many were replaced.  The
    module-level counterpart of ``patch_attention_modules`` (which only replaces the inner attention op)."""
    replaced = 0
    for parent in list(model.modules()):
        for name, child in list(parent.named_children()):
            if isinstance(child, LowpFA4Attention):
                continue
            if all(hasattr(child, a) for a in ("wq", "wk", "wv", "wo", "n_heads", "n_kv_heads", "head_dim")):
                setattr(parent, name, LowpFA4Attention.from_attention(child))
                replaced += 1
    return replaced

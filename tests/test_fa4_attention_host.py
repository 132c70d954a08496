"""Host logic of the operator boundary (no GPU): config resolution, converter
patching, fail-closed behaviour -- the CPU contract style of the reference's
tests (tests/unit_tests/test_fa4_reproduction.py)."""

import types

import pytest
import torch
import torch.nn as nn

from fa4b import fa4_attention as F


def test_route_names_follow_the_reference_table():
    assert F.resolve_fa4_config(F.FA4(exact_learned_projection_format="nvfp4")).route == "nvfp4_qk_fp8_pv"
    assert F.resolve_fa4_config(F.FA4()).route == "e4m3_proj_nvfp4_qk_fp8_pv"
    cfg = F.FA4(exact_pv_format="mxfp4_e8m0_block32", exact_learned_projection_format="nvfp4")
    assert F.resolve_fa4_config(types.SimpleNamespace(fa4=cfg)).route == "nvfp4_qk_mxfp4_pv"
    with pytest.raises(ValueError, match="fa4.mode"):
        F.resolve_fa4_config(F.FA4(mode="softcap"))
    with pytest.raises(ValueError, match="exact_pv_format"):
        F.resolve_fa4_config(types.SimpleNamespace(fa4=types.SimpleNamespace(enabled=True, mode="softmax", exact_pv_format="bf16")))
    with pytest.raises(ValueError, match="enabled"):
        F.resolve_fa4_config(F.FA4(enabled=False))


class _Attn(nn.Module):
    def __init__(self, head_dim=128):
        super().__init__()
        self.head_dim = head_dim
        self.inner_attention = nn.Identity()
        self.use_flex_attn = True
        self.attn_score_modifier = object()


def test_converter_patches_every_attention_module_once():
    model = nn.Sequential(_Attn(), nn.Linear(4, 4), _Attn(64))
    conv = F.FA4AttentionConverter(types.SimpleNamespace(fa4=F.FA4()))
    conv.convert(model)
    assert conv.patched == 2
    for m in (model[0], model[2]):
        assert isinstance(m.inner_attention, F.FA4AttentionWrapper)
        assert m.use_flex_attn is False and m.attn_score_modifier is None
    assert F.patch_attention_modules(model, conv.config) == 0  # idempotent
    with pytest.raises(RuntimeError, match="found no module"):
        F.FA4AttentionConverter(types.SimpleNamespace(fa4=F.FA4())).convert(nn.Linear(2, 2))
    with pytest.raises(ValueError, match="head_dim"):
        F.FA4AttentionConverter(types.SimpleNamespace(fa4=F.FA4())).convert(nn.Sequential(_Attn(96)))


def test_wrapper_fails_closed():
    w = F.FA4AttentionWrapper(F.resolve_fa4_config(F.FA4()), head_dim=64)
    q = torch.zeros(1, 2, 128, 64, dtype=torch.bfloat16)
    with pytest.raises(NotImplementedError, match="score_mod"):
        w(q, q, q, score_mod=lambda *a: a)
    with pytest.raises(TypeError, match="bfloat16"):
        w(q.float(), q.float(), q.float())
    with pytest.raises(ValueError, match="head dim"):
        w(q[..., :32], q[..., :32], q[..., :32])
    with pytest.raises(RuntimeError, match="no CPU path"):
        w(q, q, q)  # CPU tensors: no fallback
    with pytest.raises(NotImplementedError, match="causal"):
        F.fa4_func(q, q, q, causal=False)


def test_fake_kernels_give_shapes_for_meta_tracing():
    q = torch.empty(2, 8, 256, 128, dtype=torch.bfloat16, device="meta")
    k = torch.empty(2, 2, 256, 128, dtype=torch.bfloat16, device="meta")
    o, lse, ws = torch.ops.fa4b.attn_fwd(q, k, k, 0.0, 0)
    assert o.shape == q.shape and lse.shape == (2, 8, 256) and lse.dtype == torch.float32
    dq, dk, dv = torch.ops.fa4b.attn_bwd(o, lse, o, ws, 2, 0.0, 0)
    assert dq.shape == q.shape and dk.shape == k.shape and dv.shape == k.shape


def test_registers_under_the_reference_converter_name_when_torchtitan_is_present():
    ok = F.register_with_torchtitan("fa4_attention")
    if ok:
        from torchtitan.protocols.model_converter import _registry_model_converter_cls

        assert _registry_model_converter_cls["fa4_attention"] is F.FA4AttentionConverter

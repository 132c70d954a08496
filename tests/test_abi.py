"""CPU checks of the C-ABI library: it loads, exports every symbol the public
header declares, and rejects bad arguments before touching a device."""

import ctypes as C
import pathlib
import re

import pytest

from fa4b import _lib

ROOT = pathlib.Path(__file__).resolve().parents[1]


def test_library_exports_every_declared_symbol():
    header = (ROOT / "include" / "fa4b.h").read_text()
    declared = set(re.findall(r"\b(fa4b_[a-z0-9_]+)\s*\(", header))
    assert declared, "no declarations found"
    handle = _lib.lib()
    missing = [n for n in sorted(declared) if not hasattr(handle, n)]
    assert not missing, missing
    assert declared == set(_lib.EXPORTS), declared ^ set(_lib.EXPORTS)


def test_query_reports_build_facts():
    info = _lib.Info()
    assert _lib.lib().fa4b_query(C.byref(info)) == 0
    assert info.abi_version == 2 and info.build_sm == 100
    assert info.tile_q == 128 and info.tile_kv == 128
    assert info.fwd_tmem_columns == 512 and info.fwd_threads == 352
    assert 0 < info.wait_limit <= 1 << 24


def test_backward_flags_agree_between_the_header_and_the_python_side():
    from fa4b import attention

    header = (ROOT / "include" / "fa4b.h").read_text()
    values = {m.group(1): int(m.group(2)) for m in re.finditer(r"(FA4B_BWD_[A-Z0-9_]+) = (\d+)", header)}
    assert values == {"FA4B_BWD_KEEP_DQ_ACCUM": 1, "FA4B_BWD_SKIP_DQ_OUT": 2, "FA4B_BWD_DQ_SUMS_FP32": 4}
    assert (attention.BWD_KEEP_DQ_ACCUM, attention.BWD_SKIP_DQ_OUT, attention.BWD_DQ_SUMS_FP32) == (1, 2, 4)


def test_status_strings():
    h = _lib.lib()
    assert h.fa4b_status_string(0) == b"ok"
    assert h.fa4b_status_string(5) == b"device wait timed out"


def test_quantizer_rejects_bad_shapes_without_a_device():
    h = _lib.lib()
    a = _lib.QuantNvfp4Args(0x1000, 100, 128, 128, 0x1000, 0, 0x1000, 0x1000, 0x1000, 0, 0)
    assert h.fa4b_quant_nvfp4(C.byref(a), None) == 1  # BAD_SHAPE
    assert b"multiples of 128" in h.fa4b_last_error()
    a = _lib.QuantNvfp4Args(0x1001, 128, 128, 128, 0x1000, 0, 0x1000, 0x1000, 0x1000, 0, 0)
    assert h.fa4b_quant_nvfp4(C.byref(a), None) == 2  # BAD_ALIGN
    a = _lib.QuantNvfp4Args(0x1000, 128, 128, 128, 0x1000, 0, 0x1000, 0x1000, 0x1000, 0x1000, 0)
    assert h.fa4b_quant_nvfp4(C.byref(a), None) == 6  # codes_col without scales_col
    m = _lib.QuantMxfp4Args(0x1000, 128, 128, 128, 9, 0x1000, 0x1000)
    assert h.fa4b_quant_mxfp4(C.byref(m), None) == 3  # UNSUPPORTED mode
    with pytest.raises(ValueError):
        _lib.check(1, "x")
    with pytest.raises(TimeoutError):
        _lib.check(5, "x")


def test_attention_dims_are_validated_on_the_host():
    h = _lib.lib()
    layout = _lib.WsLayout()
    good = _lib.AttnDims(2, 32, 8, 8192, 128, 0.0, 0)
    assert h.fa4b_attn_ws_layout_query(C.byref(good), C.byref(layout)) == 0
    assert layout.total == h.fa4b_attn_workspace_bytes(C.byref(good))
    assert layout.q_codes == 0 and layout.k_codes > layout.q_scales > 0 and layout.total % 1024 == 0
    # Q codes 32 MiB, Q scale pages 4 MiB at the benchmark shape
    assert layout.q_scales - layout.q_codes == 32 << 20 and layout.q_global - layout.q_scales == 4 << 20
    for bad in (_lib.AttnDims(2, 32, 8, 8192, 96, 0.0, 0), _lib.AttnDims(2, 32, 8, 8100, 128, 0.0, 0),
                _lib.AttnDims(2, 32, 5, 8192, 128, 0.0, 0)):
        assert h.fa4b_attn_ws_layout_query(C.byref(bad), C.byref(layout)) == 1
    assert h.fa4b_attn_ws_layout_query(C.byref(_lib.AttnDims(2, 32, 8, 8192, 128, 0.0, 7)), C.byref(layout)) == 3
    assert h.fa4b_attn_ws_layout_query(C.byref(_lib.AttnDims(2, 32, 8, 8192, 128, 0.0, 0, 0, 5)), C.byref(layout)) == 3  # global_scale_mode
    assert h.fa4b_attn_workspace_bytes(C.byref(_lib.AttnDims(2, 32, 8, 8100, 128, 0.0, 0))) == 0
    # saved section (what a training step keeps from forward to backward): codes + pages + globals + three E4M3
    # operands + amax and status words; the transient section holds E5M2 dO, two statistics and the FP32 accumulators
    nq, nk, S, D = 64, 16, 8192, 128
    assert layout.saved_total == layout.do_fp8 < layout.dq_accum < layout.dkv_accum < layout.total
    assert layout.status < layout.saved_total and layout.amax_bits < layout.saved_total
    assert layout.saved_total < 260 << 20  # 36 + 9 MiB of NVFP4, 176 MiB of E4M3 (the whole cache is 0.98 GiB)
    assert layout.total - layout.dkv_accum == 2 * nk * S * D * 4 and layout.dkv_accum - layout.dq_accum == nq * S * D * 4


def test_attention_entry_points_reject_a_bad_workspace_before_any_launch():
    """NULL or misaligned workspace / scratch pointers come back as a status code whatever the prepared /
    preprocessed flags say; nothing is launched, so no device is needed."""
    h = _lib.lib()
    d = _lib.AttnDims(1, 4, 1, 256, 128, 0.0, 0)
    z = _lib.Strides(256 * 128 * 4, 256 * 128, 128)
    for prepared in (0, 1):
        for ws, want in ((0, 2), (0x10000 + 512, 2)):
            f = _lib.AttnFwdArgs(d, 0x10000, z, 0x10000, z, 0x10000, z, 0x10000, z, 0x10000, ws, prepared, 0, 0, 0)
            assert h.fa4b_attn_fwd(C.byref(f), None) == want, (prepared, ws)
            assert b"workspace" in h.fa4b_last_error()
            b = _lib.AttnBwdArgs(d, 0x10000, z, 0x10000, z, 0x10000, 0x10000, z, 0x10000, z, 0x10000, z, ws, prepared, 0, 0, 0, 0, 0)
            assert h.fa4b_attn_bwd(C.byref(b), None) == want, (prepared, ws)
    b = _lib.AttnBwdArgs(d, 0x10000, z, 0x10000, z, 0x10000, 0x10000, z, 0x10000, z, 0x10000, z, 0x10000, 1, 0, 0, 0, 0, 0x10000 + 256)
    assert h.fa4b_attn_bwd(C.byref(b), None) == 2 and b"scratch" in h.fa4b_last_error()
    b = _lib.AttnBwdArgs(d, 0x10000, z, 0x10000, z, 0x10000, 0x10000, z, 0x10000, z, 0x10000, z, 0x10000, 1, 0, 0, 0x10000 + 8, 0, 0)
    assert h.fa4b_attn_bwd(C.byref(b), None) == 2 and b"kv_ws" in h.fa4b_last_error()


def test_backward_work_list_tiles_every_key_tile_once():
    """fa4b_attn_bwd_plan / _plan_item (host only): the items of a launch cover, for every (batch, kv head) and key
    tile, the tile's query range exactly once, in parts no longer than the chunk; launch order: groups of heads, inside
    a group key tiles, then parts, then the group's heads."""
    h = _lib.lib()
    out = (C.c_int32 * 5)()
    for (B, Hkv, S, n_sm, mask) in ((2, 8, 8192, 148, 0), (1, 2, 8192, 148, 0), (1, 1, 256, 148, 0), (1, 2, 384, 148, 0),
                                    (1, 1, 1024, 148, 0), (1, 1, 512, 148, 1), (16, 8, 4096, 148, 0), (1, 1, 2048, 7, 1),
                                    (1, 3, 1152, 33, 0), (1, 6, 8192, 148, 0)):  # the last: head groups of 4 and 2
        d = _lib.AttnDims(B, 4 * Hkv, Hkv, S, 128, 0.0, 0, mask, 0)
        p = _lib.BwdPlan()
        assert h.fa4b_attn_bwd_plan(C.byref(d), n_sm, C.byref(p)) == 0
        n = S // 128
        assert p.grid == B * Hkv * p.items_per_head and 1 <= p.chunk <= n and 1 <= p.head_group <= B * Hkv
        cover, order = {}, []
        for i in range(p.grid):
            assert h.fa4b_attn_bwd_plan_item(C.byref(d), n_sm, i, out) == 0
            bhk, kt, lo, hi, parts = list(out)
            assert 0 < hi - lo <= p.chunk
            cover.setdefault((bhk, kt), []).append((lo, hi, parts))
            order.append((bhk // p.head_group, kt, lo, bhk))
        assert order == sorted(order) and len(cover) == B * Hkv * n
        for (bhk, kt), segs in cover.items():
            first = kt if mask == 0 else 0
            assert segs[0][0] == first and segs[-1][1] == n and all(a[1] == b_[0] for a, b_ in zip(segs, segs[1:]))
            assert all(s[2] == len(segs) for s in segs)
            assert (len(segs) > 1) == (kt * 128 < p.split_rows)
        assert h.fa4b_attn_bwd_plan_item(C.byref(d), n_sm, p.grid, out) == 6
    # the benchmark configuration on 148 SMs, and one eighth of it (what one of eight GPUs holds)
    p = _lib.BwdPlan()
    h.fa4b_attn_bwd_plan(C.byref(_lib.AttnDims(2, 32, 8, 8192, 128, 0.0, 0)), 148, C.byref(p))
    assert (p.chunk, p.items_per_head, p.grid, p.split_rows, p.head_group) == (64, 64, 1024, 0, 4)  # 6.9 CTAs per SM: no cut; 4 x 16.8 MB of dQ rows per group
    h.fa4b_attn_bwd_plan(C.byref(_lib.AttnDims(1, 8, 2, 8192, 128, 0.0, 0)), 148, C.byref(p))
    assert (p.chunk, p.grid) == (8, 576)  # about four items per SM


def test_python_operators_fail_loudly_on_cpu_tensors():
    import torch

    import fa4b
    from fa4b import attention

    x = torch.zeros(128, 128, dtype=torch.bfloat16)
    with pytest.raises(RuntimeError, match="no CPU path"):
        fa4b.tk_quantize_for_gemm(x, encode_centric=False)
    with pytest.raises(TypeError):
        fa4b.tk_quantize_for_gemm(x.float(), encode_centric=False)
    q = torch.zeros(1, 4, 128, 64, dtype=torch.bfloat16)
    with pytest.raises(RuntimeError, match="no CPU path"):
        attention.attn_forward(q, q, q)


def test_quantizer_operators_keep_the_reference_bindings_positional_arguments():
    """TK_quantisation/nvfp4_v6/tk_quantize.cu:3170-3172, 3219-3222 of the reference: a caller written against
    tk_quantize_for_gemm(input, return_transpose, encode_centric=true) and tk_fused_norm_quantize(input, gamma,
    epsilon, with_silu, return_transpose) keeps working; what this build adds is keyword-only."""
    import inspect

    import fa4b

    p = list(inspect.signature(fa4b.tk_quantize_for_gemm).parameters.values())
    assert [x.name for x in p[:3]] == ["input", "return_transpose", "encode_centric"] and p[2].default is True
    assert all(x.kind is inspect.Parameter.KEYWORD_ONLY for x in p[3:])
    p = list(inspect.signature(fa4b.tk_fused_norm_quantize).parameters.values())
    assert [x.name for x in p[:5]] == ["input", "gamma", "epsilon", "with_silu", "return_transpose"]
    assert all(x.kind is inspect.Parameter.KEYWORD_ONLY for x in p[5:])
    p = list(inspect.signature(fa4b.mxfp4_quantize_for_gemm).parameters.values())
    assert [x.name for x in p[:2]] == ["input", "mode"]

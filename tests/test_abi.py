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
    assert info.abi_version == 1 and info.build_sm == 100
    assert info.tile_q == 128 and info.tile_kv == 128
    assert info.fwd_tmem_columns == 512 and info.fwd_threads == 352
    assert 0 < info.wait_limit <= 1 << 24


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


def test_python_operators_fail_loudly_on_cpu_tensors():
    import torch

    import fa4b
    from fa4b import attention

    x = torch.zeros(128, 128, dtype=torch.bfloat16)
    with pytest.raises(RuntimeError, match="no CPU path"):
        fa4b.tk_quantize_for_gemm(x)
    with pytest.raises(TypeError):
        fa4b.tk_quantize_for_gemm(x.float())
    q = torch.zeros(1, 4, 128, 64, dtype=torch.bfloat16)
    with pytest.raises(RuntimeError, match="no CPU path"):
        attention.attn_forward(q, q, q)

"""The forward entry point that allocates nothing (fa4b_attn_fwd_static).

It serves hosts that may launch kernels but not allocate device memory at the
point where attention runs; its operand cache is a fixed array inside the
library.  Checked here through the C ABI against the regular entry point, on
two calls in a row that share that array, and for its size limit.  This file
sorts last on purpose: a run that stops at the first failure has then already
run every other test."""

import ctypes as C

import pytest
import torch

import fa4b_oracle as O
from fa4b import _lib, attention

DEV = "cuda"


def _static_forward(q, k, v, scale=None):
    dims = attention.make_dims(q, k, scale, "e4m3_fp8")
    B, Hq, S, D = q.shape
    o = torch.empty(B, Hq, S, D, dtype=torch.bfloat16, device=q.device)
    lse = torch.empty(B, Hq, S, dtype=torch.float32, device=q.device)
    st = attention._strides
    a = _lib.AttnFwdArgs(dims, q.data_ptr(), st(q), k.data_ptr(), st(k), v.data_ptr(), st(v), o.data_ptr(), st(o), lse.data_ptr(),
                         0, 0, 0, 0)  # no workspace pointer at all
    _lib.check(_lib.lib().fa4b_attn_fwd_static(C.byref(a), C.c_void_p(_lib.current_stream())), "fa4b_attn_fwd_static")
    return o, lse


def test_static_entry_point_rejects_shapes_beyond_its_scratch():
    # host-side check, needs no device: the benchmark shape wants ~918 MiB of operand cache
    big = _lib.AttnDims(2, 32, 8, 8192, 128, 0.0, 0)
    a = _lib.AttnFwdArgs(big, 0x1000, _lib.Strides(), 0x1000, _lib.Strides(), 0x1000, _lib.Strides(), 0x1000, _lib.Strides(),
                         0x1000, 0, 0, 0, 0)
    h = _lib.lib()
    assert h.fa4b_attn_fwd_static(C.byref(a), None) == 1  # FA4B_BAD_SHAPE
    msg = h.fa4b_last_error().decode()
    assert "FA4B_STATIC_WS_BYTES" in msg and str(8 << 20) in msg
    assert h.fa4b_attn_fwd_static(None, None) == 6


@pytest.mark.gpu
def test_static_entry_point_matches_the_regular_forward_on_two_calls_in_a_row():
    cases = [(1, 4, 1, 256, 128, 51), (1, 4, 4, 512, 64, 52)]  # the second call finds the first call's leftovers
    for B, Hq, Hkv, S, D, seed in cases:
        q, k, v, _ = O.make_attention_inputs(B, Hq, Hkv, S, D, seed=seed, rope=(D == 128))
        qd, kd, vd = q.to(DEV), k.to(DEV), v.to(DEV)
        o_ref, lse_ref, ws = attention.attn_forward(qd, kd, vd)
        ws.check_status()
        o, lse = _static_forward(qd, kd, vd)
        torch.cuda.synchronize()
        # same kernels, same operands: the tolerance of the forward parity tests is met with room to spare
        assert O.rel_l2(o_ref, o) < 1e-2 and (lse_ref - lse).abs().max().item() < 1e-3
        assert torch.equal(o_ref, o) and torch.equal(lse_ref, lse)
        fwd = O.attn_forward(q, k, v)
        assert O.rel_l2(fwd.o, o.cpu()) < 1e-2

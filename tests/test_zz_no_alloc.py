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


def _static_forward(q, k, v, scale=None, out=None):
    dims = attention.make_dims(q, k, scale, "e4m3_fp8")
    B, Hq, S, D = q.shape
    if out is None:
        out = (torch.empty(B, Hq, S, D, dtype=torch.bfloat16, device=q.device), torch.empty(B, Hq, S, dtype=torch.float32, device=q.device))
    o, lse = out
    st = attention._strides
    a = _lib.AttnFwdArgs(dims, q.data_ptr(), st(q), k.data_ptr(), st(k), v.data_ptr(), st(v), o.data_ptr(), st(o), lse.data_ptr(),
                         0, 0, 0, 0)  # no workspace pointer at all
    _lib.check(_lib.lib().fa4b_attn_fwd_static(C.byref(a), C.c_void_p(_lib.current_stream())), "fa4b_attn_fwd_static")
    return o, lse


def test_static_entry_point_rejects_shapes_beyond_its_scratch():
    # host-side check, needs no device: the benchmark shape's forward operands take ~222 MiB
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
    first_call = True
    for B, Hq, Hkv, S, D, seed in cases:
        q, k, v, _ = O.make_attention_inputs(B, Hq, Hkv, S, D, seed=seed, rope=(D == 128))
        qd, kd, vd = q.to(DEV), k.to(DEV), v.to(DEV)
        o_ref, lse_ref, ws = attention.attn_forward(qd, kd, vd)
        ws.check_status()
        o_buf = torch.empty(B, Hq, S, D, dtype=torch.bfloat16, device=DEV)  # outputs are the caller's: allocated first
        lse_buf = torch.empty(B, Hq, S, dtype=torch.float32, device=DEV)
        if first_call:
            # the first call on a device looks the array's address up, and the driver may load the module that holds
            # the array only now: set-up that the header tells callers to do before they freeze their memory
            _static_forward(qd, kd, vd, out=(o_buf, lse_buf))
            first_call = False
        torch.cuda.synchronize()
        free_before, reserved_before = torch.cuda.mem_get_info()[0], torch.cuda.memory_reserved()
        o, lse = _static_forward(qd, kd, vd, out=(o_buf, lse_buf))
        torch.cuda.synchronize()
        # the property in the entry point's name: the call took no device memory, from the driver or from torch's pool
        assert torch.cuda.mem_get_info()[0] == free_before and torch.cuda.memory_reserved() == reserved_before
        # a bounded wait that ran out inside the call would be reported here (NULL = the built-in cache)
        _lib.check(_lib.lib().fa4b_attn_check_status(C.byref(attention.make_dims(qd, kd, None, "e4m3_fp8")), None,
                                                     C.c_void_p(_lib.current_stream())), "fa4b_attn_check_status")
        # same kernels, same operands: the tolerance of the forward parity tests is met with room to spare
        assert O.rel_l2(o_ref, o) < 1e-2 and (lse_ref - lse).abs().max().item() < 1e-3
        assert torch.equal(o_ref, o) and torch.equal(lse_ref, lse)
        fwd = O.attn_forward(q, k, v)
        assert O.rel_l2(fwd.o, o.cpu()) < 1e-2

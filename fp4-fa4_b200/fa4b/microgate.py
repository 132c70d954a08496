"""Tensor-core self tests (one 128x128xK product per call); see fa4b_microgate."""

from __future__ import annotations

import ctypes as C

import torch

from ._lib import check, current_stream, lib, ptr

KINDS = {"nvfp4": 0, "e4m3_kk": 1, "e4m3_e5m2_kk": 2, "e4m3_k_mn": 3, "e4m3_mn_mn": 4, "e4m3_ts_mn": 5, "mxfp4": 6,
         "e4m3_kk_tma": 7}


def run(kind: str, K: int, a: torch.Tensor, b: torch.Tensor, sfa: torch.Tensor | None = None, sfb: torch.Tensor | None = None):
    out = torch.zeros(128, 128, dtype=torch.float32, device=a.device)
    status = torch.zeros(4, dtype=torch.int32, device=a.device)
    check(lib().fa4b_microgate(C.c_int(KINDS[kind]), C.c_int(K), C.c_void_p(ptr(a)), C.c_void_p(ptr(b)), C.c_void_p(ptr(sfa)),
                               C.c_void_p(ptr(sfb)), C.c_void_p(ptr(out)), C.c_void_p(ptr(status)), C.c_void_p(current_stream())),
          "fa4b_microgate")
    torch.cuda.synchronize()
    if int(status[0]) != 0:
        raise TimeoutError(f"microgate {kind}: device wait ran out at site {int(status[1])}")
    return out


def tensor_peak(kind: str, iters: int = 8192, reps: int = 3) -> float:
    """Measured dense tensor-core rate of the current GPU in TFLOP/s for ``kind`` in {"fp8", "nvfp4"}
    (all SMs, operands resident in shared memory, CUDA events, best of ``reps``)."""
    k = {"fp8": 0, "nvfp4": 1}[kind]
    status = torch.zeros(4, dtype=torch.int32, device="cuda")
    sms = torch.cuda.get_device_properties(torch.cuda.current_device()).multi_processor_count
    flops = sms * iters * 2.0 * 128 * 256 * (32 if k == 0 else 64)
    best = float("inf")
    for _ in range(reps + 1):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        check(lib().fa4b_tensor_peak(C.c_int(k), C.c_int(iters), C.c_void_p(ptr(status)), C.c_void_p(current_stream())), "fa4b_tensor_peak")
        e1.record()
        e1.synchronize()
        if int(status[0]) != 0:
            raise TimeoutError(f"tensor_peak {kind}: device wait ran out")
        best = min(best, e0.elapsed_time(e1))
    return flops / (best * 1e-3) / 1e12


def wait_selftest(limit_cycles: int = 1_000_000) -> torch.Tensor:
    """Make a bounded device-side wait run out on purpose (an unarmed barrier, nothing in flight) and return the
    8 status words; raises unless the library reports exactly FA4B_TIMEOUT."""
    status = torch.zeros(8, dtype=torch.int32, device="cuda")
    rc = lib().fa4b_wait_selftest(C.c_int64(limit_cycles), C.c_void_p(ptr(status)), C.c_void_p(current_stream()))
    if rc != 5:
        check(rc, "fa4b_wait_selftest")
        raise RuntimeError("fa4b_wait_selftest returned FA4B_OK: the wait did not run out")
    return status

"""Context-parallel forward on the GPU: the operand-level entry points (two-phase prepare with an external amax,
prepared forward against a second K/V cache, unmasked blocks, the merge kernel) against the single-kernel run of
the whole sequence; and, where the box has several GPUs, the NCCL ring itself."""

import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import fa4b_oracle as O
from fa4b import attention
from fa4b import context_parallel as cp

pytestmark = pytest.mark.gpu
DEV = "cuda"


@pytest.mark.parametrize("pv", ["e4m3_fp8", "mxfp4_e8m0_block32"])
@pytest.mark.parametrize("B,Hq,Hkv,S,D", [(1, 4, 1, 512, 128), (2, 4, 2, 768, 64)])
def test_one_rank_ring_matches_the_single_kernel(B, Hq, Hkv, S, D, pv):
    """world = 1: chunk 0 causal, chunk 1 against chunk 0 unmasked, chunk 1 causal, merged."""
    q, k, v, _ = (t.to(DEV) for t in O.make_attention_inputs(B, Hq, Hkv, S, D, seed=123 + S, rope=(D == 128)))
    o_ref, lse_ref, ws = attention.attn_forward(q, k, v, pv_format=pv)
    ws.check_status()
    o, lse = cp.ring_attention_forward(q, k, v, cp.KernelEngine(pv_format=pv))
    torch.cuda.synchronize()
    assert O.rel_l2(o_ref.float().cpu(), o.float().cpu()) < 4e-3
    assert (lse_ref - lse).abs().max().item() < 2e-3 if pv != "e4m3_fp8" else (lse_ref - lse).abs().max().item() < 1e-4
    # the first chunk is one causal block call with the whole-sequence amax: identical to the single kernel's rows
    assert torch.equal(o[:, :, :S // 2], o_ref[:, :, :S // 2])


def test_one_rank_ring_backward_matches_the_single_kernel():
    """world = 1: three block calls per direction; dQ folded in the FP32 scratch, dK / dV through fa4b_attn_accumulate."""
    B, Hq, Hkv, S, D = 1, 8, 2, 1024, 128
    q, k, v, do = (t.to(DEV) for t in O.make_attention_inputs(B, Hq, Hkv, S, D, seed=77, rope=True, do_std=0.01))
    o_ref, lse_ref, ws = attention.attn_forward(q, k, v)
    want = attention.attn_backward(o_ref, lse_ref, do, ws)
    ws.check_status()
    engine = cp.KernelEngine()
    o, lse, state = cp.ring_attention_forward(q, k, v, engine, return_state=True)
    got = cp.ring_attention_backward(o, lse, do, state, engine)
    for w_ in state:
        w_.check_status()
    for w, g_, name in zip(want, got, ("dq", "dk", "dv")):
        assert O.rel_l2(w.float().cpu(), g_.float().cpu()) < 1e-2, (name, O.rel_l2(w.float().cpu(), g_.float().cpu()))


def test_merge_kernel_against_fp32_formula():
    g = torch.Generator(device=DEV).manual_seed(5)
    rows, D = 1000, 128
    o_acc = torch.randn(rows, D, device=DEV, generator=g)
    lse_acc = torch.randn(rows, device=DEV, generator=g) * 3
    lse_acc[::7] = float("-inf")
    o_acc[::7] = 0
    o_part = torch.randn(rows, D, device=DEV, generator=g).bfloat16()
    lse_part = torch.randn(rows, device=DEV, generator=g) * 3
    m = torch.maximum(lse_acc, lse_part)
    ea, ep = torch.exp(lse_acc - m), torch.exp(lse_part - m)
    want_o = o_acc * (ea / (ea + ep))[:, None] + o_part.float() * (ep / (ea + ep))[:, None]
    want_l = m + torch.log(ea + ep)
    out = torch.empty(rows, D, dtype=torch.bfloat16, device=DEV)
    attention.attn_merge(o_acc, lse_acc, o_part, lse_part, out=out)
    assert torch.allclose(o_acc, want_o, rtol=1e-5, atol=1e-6)
    assert torch.allclose(lse_acc, want_l, rtol=1e-5, atol=1e-5)
    assert torch.equal(out, o_acc.bfloat16())


def _worker(rank, world, port, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        B, Hq, Hkv, D = 1, 8, 2, 128
        S = 256 * 2 * world
        q, k, v, _ = O.make_attention_inputs(B, Hq, Hkv, S, D, seed=31, rope=True, heavy_tail=True)
        ql, kl, vl = (cp.shard_sequence(t, rank, world).cuda() for t in (q, k, v))
        engine = cp.KernelEngine()
        o, lse, state = cp.ring_attention_forward(ql, kl, vl, engine, return_state=True)
        _, _, _, do = O.make_attention_inputs(B, Hq, Hkv, S, D, seed=31, rope=True, heavy_tail=True, do_std=0.01)
        grads = []
        for t in cp.ring_attention_backward(o, lse, cp.shard_sequence(do, rank, world).cuda(), state, engine):
            parts = [torch.empty_like(t) for _ in range(world)]
            dist.all_gather(parts, t.contiguous())  # checking only
            grads.append(cp.unshard_sequence(parts))
        parts_o = [torch.empty_like(o) for _ in range(world)]
        parts_l = [torch.empty_like(lse) for _ in range(world)]
        dist.all_gather(parts_o, o.contiguous())  # checking only
        dist.all_gather(parts_l, lse.contiguous())
        if rank == 0:
            o_ref, lse_ref, ws = attention.attn_forward(q.cuda(), k.cuda(), v.cuda())
            ws.check_status()
            got_o, got_l = cp.unshard_sequence(parts_o), cp.unshard_sequence(parts_l, dim=2)
            want = attention.attn_backward(o_ref, lse_ref, do.cuda(), ws)
            ws.check_status()
            g_err = max(O.rel_l2(w.float().cpu(), g_.float().cpu()) for w, g_ in zip(want, grads))
            out.put((O.rel_l2(o_ref.float().cpu(), got_o.float().cpu()), float((lse_ref - got_l).abs().max()), g_err))
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="the NCCL ring needs at least two GPUs")
def test_nccl_ring_matches_the_single_device_kernel():
    world = min(torch.cuda.device_count(), 4)
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, world, port, out)) for r in range(world)]
    for p in procs:
        p.start()
    o_err, lse_err, g_err = out.get(timeout=300)
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    # gradients: the ring's O carries the bf16 rounding of its partial results into dstat (heavy-tailed inputs here)
    assert o_err < 4e-3 and lse_err < 1e-4 and g_err < 2e-2, (o_err, lse_err, g_err)

"""GPU parity at the configurations and through the entry points that the other files do not reach: the operator
boundary (FA4AttentionWrapper, the torch.library ops and their autograd) against the oracle; a (batch, kv-head) unit
of the D = 64 configuration at its full size; the long-context route's block calls on heavy-tailed inputs against
the oracle's MXFP4 P.V emulation; the reference's own forward gate; and the backward's split work list at the shape
an 8-GPU shard of the benchmark configuration has.  Tolerances are the path's: O and LSE rel-L2 1e-2 / abs 1e-3,
dQ, dK, dV rel-L2 2e-2."""

import pytest
import torch

import fa4b_oracle as O
from fa4b import attention, fa4_attention
from fa4b import context_parallel as cp

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _wrapper(D, pv="e4m3_fp8"):
    cfg = fa4_attention.resolve_fa4_config(fa4_attention.FA4(exact_pv_format=pv))
    return fa4_attention.FA4AttentionWrapper(cfg, head_dim=D)


@pytest.mark.parametrize("B,Hq,Hkv,S,D,do_layout", [
    (1, 4, 4, 512, 64, "contiguous"),   # the CPU-runnable reference configuration
    (1, 8, 2, 384, 128, "bshd"),        # GQA, D = 128, upstream gradient stored [B,S,H,D]
    (2, 8, 2, 256, 128, "strided"),     # upstream gradient with a non-unit last stride
])
def test_wrapper_forward_and_autograd_backward_match_the_oracle(B, Hq, Hkv, S, D, do_layout):
    q, k, v, do = O.make_attention_inputs(B, Hq, Hkv, S, D, seed=4242 + S + D, rope=(D == 128), do_std=0.01)
    fwd = O.attn_forward(q, k, v)
    want = O.attn_backward(q, k, v, fwd.o, fwd.lse, do)
    qd, kd, vd = (t.to(DEV).requires_grad_(True) for t in (q, k, v))
    out = _wrapper(D)(qd, kd, vd)
    assert out.shape == (B, Hq, S, D) and out.dtype == torch.bfloat16
    if do_layout == "bshd":
        dod = do.permute(0, 2, 1, 3).contiguous().to(DEV).permute(0, 2, 1, 3)
        assert not dod.is_contiguous()
    elif do_layout == "strided":
        wide = torch.zeros(B, Hq, S, 2 * D, dtype=torch.bfloat16, device=DEV)
        wide[..., ::2] = do.to(DEV)
        dod = wide[..., ::2]
        assert dod.stride(-1) == 2
    else:
        dod = do.to(DEV)
    out.backward(dod)
    torch.cuda.synchronize()
    assert O.rel_l2(fwd.o, out.detach().cpu()) < 1e-2
    for name, got, w in (("dq", qd.grad, want[0]), ("dk", kd.grad, want[1]), ("dv", vd.grad, want[2])):
        assert got.shape == w.shape and O.rel_l2(w, got.cpu()) < 2e-2, (name, O.rel_l2(w, got.cpu()))


def test_custom_op_saves_only_the_operand_section_and_checks_it_on_the_way_back():
    B, Hq, Hkv, S, D = 1, 4, 2, 256, 128
    q, k, v, do = (t.to(DEV) for t in O.make_attention_inputs(B, Hq, Hkv, S, D, seed=5, do_std=0.01))
    o, lse, saved = torch.ops.fa4b.attn_fwd(q, k, v, 0.0, 0)
    layout = attention.ws_layout(attention.make_dims(q, k, None, "e4m3_fp8"))
    assert saved.numel() == layout.saved_total < layout.total and saved.data_ptr() % 1024 == 0
    fwd = O.attn_forward(q.cpu(), k.cpu(), v.cpu())
    assert O.rel_l2(fwd.o, o.cpu()) < 1e-2 and (fwd.lse - lse.cpu()).abs().max() < 1e-3
    dq, dk, dv = torch.ops.fa4b.attn_bwd(o, lse, do, saved, Hkv, 0.0, 0)
    want = O.attn_backward(q.cpu(), k.cpu(), v.cpu(), fwd.o, fwd.lse, do.cpu())
    for w, g_ in zip(want, (dq, dk, dv)):
        assert O.rel_l2(w, g_.cpu()) < 2e-2
    with pytest.raises(RuntimeError, match="does not match"):
        torch.ops.fa4b.attn_bwd(o, lse, do, saved[:-1024], Hkv, 0.0, 0)
    # the same backward with the transient section as a caller-owned buffer, through the Python operator
    ws = attention.Workspace(attention.make_dims(q, k, None, "e4m3_fp8"), layout, saved)
    dq2, dk2, dv2 = attention.attn_backward(o, lse, do, ws.with_scratch(attention.alloc_scratch(ws.dims, DEV)))
    assert torch.equal(dk2, dk) and torch.equal(dv2, dv) and O.rel_l2(dq.float().cpu(), dq2.float().cpu()) < 4e-3  # f16 partial sums, other order


def test_wrapper_mxfp4_route_forward():
    q, k, v, _ = O.make_attention_inputs(1, 4, 1, 256, 128, seed=8, rope=True)
    fwd = O.attn_forward(q, k, v, pv_format="mxfp4_e8m0_block32")
    with torch.no_grad():
        out = _wrapper(128, "mxfp4_e8m0_block32")(q.to(DEV), k.to(DEV), v.to(DEV))
    assert O.rel_l2(fwd.o, out.cpu()) < 1e-2


def test_d64_configuration_unit_at_full_size():
    """B16, Hq32, Hkv8, S4096, D64 (N(0,1) inputs with RoPE).  Too large for the CPU oracle as a whole; every
    statistic is local to a (batch, kv-head) unit, so the oracle of one unit checks that unit's rows of the full run.
    The 16 batches are two generated ones with their kv groups rotated, so that the unit sits somewhere else in every
    batch and equal units can also be compared with each other bit for bit."""
    B, Hq, Hkv, S, D = 16, 32, 8, 4096, 64
    G = Hq // Hkv
    q2, k2, v2, do2 = O.make_attention_inputs(2, Hq, Hkv, S, D, seed=20260826, rope=True, do_std=0.01)
    qd = torch.cat([torch.roll(q2, i * G, dims=1) for i in range(8)]).to(DEV)
    kd = torch.cat([torch.roll(k2, i, dims=1) for i in range(8)]).to(DEV)
    vd = torch.cat([torch.roll(v2, i, dims=1) for i in range(8)]).to(DEV)
    dod = torch.cat([torch.roll(do2, i * G, dims=1) for i in range(8)]).to(DEV)
    o, lse, ws = attention.attn_forward(qd, kd, vd)
    ws.check_status()
    dq, dk, dv = attention.attn_backward(o, lse, dod, ws)
    ws.check_status()
    # source unit (batch 1, kv head 2) sits at kv head (2 + i) % 8 of batch 2 i + 1
    b0, hk0 = 1, 2
    hq0 = slice(hk0 * G, (hk0 + 1) * G)
    qu, ku, vu, dou = q2[b0:b0 + 1, hq0], k2[b0:b0 + 1, hk0:hk0 + 1], v2[b0:b0 + 1, hk0:hk0 + 1], do2[b0:b0 + 1, hq0]
    fwd = O.attn_forward(qu, ku, vu, query_chunk=512)
    want = O.attn_backward(qu, ku, vu, fwd.o, fwd.lse, dou, query_chunk=512)
    for i in (0, 5):
        b, hk = 2 * i + b0, (hk0 + i) % Hkv
        hq = slice(hk * G, (hk + 1) * G)
        assert O.rel_l2(fwd.o, o[b:b + 1, hq].cpu()) < 1e-2 and (fwd.lse - lse[b:b + 1, hq].cpu()).abs().max() < 1e-3
        for w, g_, name in zip(want, (dq[b:b + 1, hq], dk[b:b + 1, hk:hk + 1], dv[b:b + 1, hk:hk + 1]), ("dq", "dk", "dv")):
            assert O.rel_l2(w, g_.cpu()) < 2e-2, (name, i, O.rel_l2(w, g_.cpu()))
    assert torch.equal(o[b0, hq0], o[2 * 5 + b0, ((hk0 + 5) % Hkv) * G:((hk0 + 5) % Hkv + 1) * G])
    assert torch.equal(lse[b0, hq0], lse[2 * 5 + b0, ((hk0 + 5) % Hkv) * G:((hk0 + 5) % Hkv + 1) * G])


def test_long_context_block_calls_on_heavy_tailed_inputs_against_the_oracle():
    """The long-context route (MXFP4 P.V, Student-t Q and K) as one rank runs it: the sequence in two chunks, chunk 0
    causal, chunk 1 against chunk 0 unmasked, chunk 1 causal, partial results folded by their log-sum-exp --
    against the oracle's emulation of the whole sequence, not against the single kernel."""
    B, Hq, Hkv, S, D = 1, 4, 1, 8192, 128
    q, k, v, _ = O.make_attention_inputs(B, Hq, Hkv, S, D, seed=20260829, rope=True, heavy_tail=True)
    fwd = O.attn_forward(q, k, v, pv_format="mxfp4_e8m0_block32", query_chunk=512)
    engine = cp.KernelEngine(pv_format="mxfp4_e8m0_block32")
    o, lse, state = cp.ring_attention_forward(q.to(DEV), k.to(DEV), v.to(DEV), engine, return_state=True)
    for w in state:
        w.check_status()
    assert O.rel_l2(fwd.o, o.cpu()) < 1e-2, O.rel_l2(fwd.o, o.cpu())
    err = (fwd.lse - lse.cpu()).abs()
    # LSE sums FP4-represented probabilities: a term that lands on the other side of an E2M1 boundary moves its row
    assert O.rel_l2(fwd.lse, lse.cpu()) < 1e-2 and (err > 1e-3).float().mean() < 1e-3 and err.max() < 2e-2, (
        float((err > 1e-3).float().mean()), float(err.max()))
    # the FP8 route on the same inputs, forward and backward through the block calls
    engine8 = cp.KernelEngine()
    S8 = 2048
    q, k, v, do = O.make_attention_inputs(B, Hq, Hkv, S8, D, seed=20260830, rope=True, heavy_tail=True, do_std=0.01)
    fwd8 = O.attn_forward(q, k, v, query_chunk=512)
    o8, lse8, state8 = cp.ring_attention_forward(q.to(DEV), k.to(DEV), v.to(DEV), engine8, return_state=True)
    assert O.rel_l2(fwd8.o, o8.cpu()) < 1e-2 and (fwd8.lse - lse8.cpu()).abs().max() < 1e-3
    got = cp.ring_attention_backward(o8, lse8, do.to(DEV), state8, engine8)
    want = O.attn_backward(q, k, v, o8.cpu(), lse8.cpu(), do, query_chunk=512)
    for w, g_, name in zip(want, got, ("dq", "dk", "dv")):
        assert O.rel_l2(w, g_.cpu()) < 2e-2, (name, O.rel_l2(w, g_.cpu()))


@pytest.mark.parametrize("B,Hq,Hkv,S,D,gs", [(1, 4, 1, 1024, 128, "amax_per_bh"), (1, 4, 4, 512, 64, "amax_per_bh"),
                                             (2, 8, 2, 512, 128, "one")])
def test_kernel_passes_the_reference_forward_gate(B, Hq, Hkv, S, D, gs):
    """validate_causal_gqa_fp8pv_batch.py:268-324, 705-706 of the reference: the kernel's O against exact attention on
    the decoded operands, cosine >= 0.999 and rel-L2 <= 0.03."""
    q, k, v, _ = O.make_attention_inputs(B, Hq, Hkv, S, D, seed=99 + S, rope=(D == 128))
    fwd = O.attn_forward(q, k, v, global_scale=gs)  # its operands equal the kernel's byte for byte (checked elsewhere)
    o, lse, ws = attention.attn_forward(q.to(DEV), k.to(DEV), v.to(DEV), global_scale=gs)
    ws.check_status()
    assert torch.equal(ws.operands()["q_codes"].cpu(), fwd.q_codes) and torch.equal(ws.operands()["k_codes"].cpu(), fwd.k_codes)
    cosine, rel = O.represented_forward_gate(o.cpu(), fwd)
    assert cosine >= 0.999 and rel <= 0.03, (cosine, rel)


def test_backward_split_work_list_at_the_shape_of_an_eight_gpu_shard():
    """B1, Hq8, Hkv2, S8192, D128: two (batch, kv-head) units, what one of eight GPUs holds of the benchmark
    configuration.  The backward cuts every key tile's query range into short parts here (64 key tiles over
    148 SMs otherwise), so dK and dV of every tile are FP32 sums over several CTAs."""
    B, Hq, Hkv, S, D = 1, 8, 2, 8192, 128
    q, k, v, do = O.make_attention_inputs(B, Hq, Hkv, S, D, seed=20260827, rope=True, do_std=0.01)
    o, lse, ws = attention.attn_forward(q.to(DEV), k.to(DEV), v.to(DEV))
    ws.check_status()
    plan = attention.backward_plan(ws.dims)
    assert plan.chunk < 16 and plan.split_rows > S // 2 and plan.grid > 3 * 148  # on a B200: chunk 8, 576 CTAs
    dq, dk, dv = attention.attn_backward(o, lse, do.to(DEV), ws)
    ws.check_status()
    fwd = O.attn_forward(q, k, v, query_chunk=512)
    assert O.rel_l2(fwd.o, o.cpu()) < 1e-2 and (fwd.lse - lse.cpu()).abs().max() < 1e-3
    want = O.attn_backward(q, k, v, fwd.o, fwd.lse, do, query_chunk=512)
    for w, g_, name in zip(want, (dq, dk, dv), ("dq", "dk", "dv")):
        assert O.rel_l2(w, g_.cpu()) < 2e-2, (name, O.rel_l2(w, g_.cpu()))
    # the unmasked block call of a sequence-sharded run splits too
    dims_nc = attention.make_dims(q.to(DEV), k.to(DEV), None, "e4m3_fp8", causal=False)
    assert attention.backward_plan(dims_nc).split_rows == S

"""GPU parity of the attention path against the CPU oracle on the same seeded
inputs: quantised operands bit-exact; O and LSE within rel-L2 1e-2 / abs 1e-3;
dQ, dK, dV within rel-L2 2e-2."""

import pytest
import torch

import fa4b_oracle as O
from fa4b import attention

pytestmark = pytest.mark.gpu
DEV = "cuda"
# dQ of two runs of the same problem: the key tiles' partial sums meet as f16 pairs in an order that differs from run
# to run (7.5e-4 measured at S = 2048 ... 8192); with dq_sums_fp32 the difference is FP32 summation order only
DQ_RERUN_TOL = 4e-3


def _pages(scales):  # [B,H,S,D/16] bytes -> [B,H,S/128,D/64,512]
    B, H = scales.shape[:2]
    return torch.stack([torch.stack([O.scales_to_pages(scales[b, h]) for h in range(H)]) for b in range(B)])


def _check_operands(ws, fwd):
    ops = ws.operands()
    assert torch.equal(ops["q_global"].cpu(), fwd.q_global)
    assert torch.equal(ops["k_global"].cpu(), fwd.k_global)
    for name, want in (("q_codes", fwd.q_codes), ("k_codes", fwd.k_codes), ("q_scales", _pages(fwd.q_scales)),
                       ("k_scales", _pages(fwd.k_scales)), ("v_fp8", fwd.v_fp8.view(torch.uint8))):
        got = ops[name].cpu().view(torch.uint8)
        bad = (got != want.view(torch.uint8)).sum().item()
        assert bad == 0, f"{name}: {bad} bytes differ"


def _assert_dkv_reproduce(dims, a, b, name):
    """dK / dV of two runs of the same problem: bit for bit where a key tile's query range is handled by one CTA or
    two (a + b = b + a), within FP32 summation order where three or more partial sums meet."""
    plan = attention.backward_plan(dims)
    n = dims.S // 128
    causal = dims.mask == 0
    many = max(0, (n - 2 * plan.chunk) * 128) if causal else (dims.S if n > 2 * plan.chunk else 0)
    assert torch.equal(a[:, :, many:], b[:, :, many:]), name
    if many:
        assert O.rel_l2(a[:, :, :many].float().cpu(), b[:, :, :many].float().cpu()) < 1e-4, name


def _check_forward(o, lse, fwd):
    torch.cuda.synchronize()
    assert O.rel_l2(fwd.lse, lse.cpu()) < 1e-2 and (fwd.lse - lse.cpu()).abs().max() < 1e-3
    assert O.rel_l2(fwd.o, o.cpu()) < 1e-2, O.rel_l2(fwd.o, o.cpu())


FWD_CASES = [
    # B, Hq, Hkv, S, D, rope
    (1, 4, 4, 512, 64, False),   # the CPU-runnable reference configuration
    (1, 4, 1, 256, 128, False),  # one GQA group, D128
    (2, 8, 2, 384, 128, True),   # RoPE'd, ragged tile count, batch > 1
    (1, 2, 2, 128, 64, False),   # single tile (diagonal only)
]


@pytest.mark.parametrize("B,Hq,Hkv,S,D,rope", FWD_CASES)
def test_forward_matches_oracle(B, Hq, Hkv, S, D, rope):
    q, k, v, _ = O.make_attention_inputs(B, Hq, Hkv, S, D, seed=20260825 + S + D, rope=rope)
    fwd = O.attn_forward(q, k, v)
    o, lse, ws = attention.attn_forward(q.to(DEV), k.to(DEV), v.to(DEV))
    ws.check_status()
    _check_operands(ws, fwd)
    _check_forward(o, lse, fwd)


@pytest.mark.parametrize("B,Hq,Hkv,S,D", [(1, 4, 1, 256, 128), (1, 4, 4, 256, 64)])
def test_unit_global_scale_route_matches_oracle_forward_and_backward(B, Hq, Hkv, S, D):
    # the reference's attention route: global decode scale 1, block scale E4M3(block amax / 6), no statistics pass
    q, k, v, do = O.make_attention_inputs(B, Hq, Hkv, S, D, seed=77 + D)
    q[0, 0, 5, :16] *= 3000.0  # a block whose amax / 6 is beyond E4M3: the scale byte saturates, the codes clip
    fwd = O.attn_forward(q, k, v, global_scale="one")
    assert float(fwd.q_global.min()) == 1.0 == float(fwd.k_global.max())
    o, lse, ws = attention.attn_forward(q.to(DEV), k.to(DEV), v.to(DEV), global_scale="one")
    ws.check_status()
    _check_operands(ws, fwd)
    _check_forward(o, lse, fwd)
    dq, dk, dv = attention.attn_backward(o, lse, do.to(DEV), ws)
    ws.check_status()
    rq, rk, rv = O.attn_backward(q, k, v, fwd.o, fwd.lse, do, global_scale="one")
    for name, got, want in (("dq", dq, rq), ("dk", dk, rk), ("dv", dv, rv)):
        assert O.rel_l2(want.float(), got.float().cpu()) < 2e-2, name


def test_forward_accepts_bshd_strides_and_custom_scale():
    q, k, v, _ = O.make_attention_inputs(1, 4, 2, 256, 128, seed=9)
    fwd = O.attn_forward(q, k, v, softmax_scale=0.05)
    # [B,S,H,D] storage viewed as [B,H,S,D]
    qd, kd, vd = (t.permute(0, 2, 1, 3).contiguous().to(DEV).permute(0, 2, 1, 3) for t in (q, k, v))
    o, lse, ws = attention.attn_forward(qd, kd, vd, softmax_scale=0.05)
    ws.check_status()
    _check_forward(o, lse, fwd)


def test_forward_is_bitwise_reproducible():
    q, k, v, _ = O.make_attention_inputs(1, 4, 2, 512, 128, seed=4)
    a = attention.attn_forward(q.to(DEV), k.to(DEV), v.to(DEV))
    b = attention.attn_forward(q.to(DEV), k.to(DEV), v.to(DEV))
    assert torch.equal(a[0], b[0]) and torch.equal(a[1], b[1])


def test_forward_long_sequence_against_chunked_oracle():
    """S=2048: many kv tiles per query tile (stage ring wraps, maxima move)."""
    q, k, v, _ = O.make_attention_inputs(1, 4, 1, 2048, 128, seed=17, rope=True)
    fwd = O.attn_forward(q, k, v, query_chunk=512)
    o, lse, ws = attention.attn_forward(q.to(DEV), k.to(DEV), v.to(DEV))
    ws.check_status()
    _check_forward(o, lse, fwd)


def test_backward_preprocess_matches_oracle():
    q, k, v, do = O.make_attention_inputs(1, 4, 2, 256, 128, seed=21, do_std=0.01)
    fwd = O.attn_forward(q, k, v)
    _, _, ws = attention.attn_forward(q.to(DEV), k.to(DEV), v.to(DEV))
    do5, dstat, lstat = attention.attn_bwd_preprocess(fwd.o.to(DEV), fwd.lse.to(DEV), do.to(DEV), ws)
    r5, rd, rl = O.attn_bwd_preprocess(fwd.o, do, fwd.lse)
    assert torch.equal(do5.cpu().view(torch.uint8), r5.view(torch.uint8))
    assert torch.allclose(lstat.cpu(), rl, rtol=0, atol=1e-5)
    assert O.rel_l2(rd, dstat.cpu()) < 1e-5


BWD_CASES = [
    (1, 4, 4, 512, 64),    # the CPU-runnable reference configuration
    (1, 4, 1, 256, 128),   # one GQA group of four query heads
    (2, 8, 2, 384, 128),   # batch, several kv heads, three key tiles
    (1, 2, 2, 128, 64),
]


def _run_backward(q, k, v, do, scale=None):
    fwd = O.attn_forward(q, k, v, softmax_scale=scale)
    o, lse, ws = attention.attn_forward(q.to(DEV), k.to(DEV), v.to(DEV), softmax_scale=scale)
    # both sides consume their own forward results, as a training step does
    want = O.attn_backward(q, k, v, fwd.o, fwd.lse, do, softmax_scale=scale)
    got = attention.attn_backward(o, lse, do.to(DEV), ws)
    ws.check_status()
    return want, got


@pytest.mark.parametrize("B,Hq,Hkv,S,D", BWD_CASES)
def test_backward_matches_oracle(B, Hq, Hkv, S, D):
    q, k, v, do = O.make_attention_inputs(B, Hq, Hkv, S, D, seed=20260829 + S + D, rope=(D == 128), do_std=0.01)
    want, got = _run_backward(q, k, v, do)
    for w, g, name in zip(want, got, ("dq", "dk", "dv")):
        err = O.rel_l2(w, g.cpu())
        assert err < 2e-2, (name, err)


def test_backward_zero_dout_gives_exact_zero_gradients():
    # validate_native_tk_d128_backward.py:707-738 of the reference
    q, k, v, do = O.make_attention_inputs(1, 4, 1, 256, 128, seed=33)
    o, lse, ws = attention.attn_forward(q.to(DEV), k.to(DEV), v.to(DEV))
    dq, dk, dv = attention.attn_backward(o, lse, torch.zeros_like(do).to(DEV), ws)
    ws.check_status()
    assert not dq.any() and not dk.any() and not dv.any()


def test_backward_long_sequence():
    q, k, v, do = O.make_attention_inputs(1, 4, 1, 1024, 128, seed=41, rope=True, do_std=0.01)
    want, got = _run_backward(q, k, v, do)
    for w, g, name in zip(want, got, ("dq", "dk", "dv")):
        assert O.rel_l2(w, g.cpu()) < 2e-2, name


def test_partition_by_batch_and_kv_head_reproduces_the_unsharded_run():
    """The multi-GPU split (no collective): every "rank" runs its (batch, kv-head) units as an independent problem
    on views of the global tensors; O, LSE, dK, dV match the unsharded run bit for bit, dQ up to the order of its
    FP32 reductions."""
    from fa4b import parallel

    B, Hq, Hkv, S, D = 2, 8, 2, 384, 128
    q, k, v, do = (t.to(DEV) for t in O.make_attention_inputs(B, Hq, Hkv, S, D, seed=77, rope=True, do_std=0.01))
    o, lse, ws = attention.attn_forward(q, k, v)
    dq, dk, dv = attention.attn_backward(o, lse, do, ws)
    ws.check_status()
    world = 3  # uneven on purpose: 4 units over 3 ranks
    parts = {n: [] for n in ("o", "lse", "dq", "dk", "dv")}
    for rank in range(world):
        qs, ks, vs, dos = parallel.shard_attention_inputs(q, k, v, rank, world, do)
        o_r, lse_r, ws_r = attention.attn_forward(qs, ks, vs)
        dq_r, dk_r, dv_r = attention.attn_backward(o_r, lse_r, dos, ws_r)
        ws_r.check_status()
        for n, t in zip(parts, (o_r, lse_r, dq_r, dk_r, dv_r)):
            parts[n].append(t)
    assert torch.equal(parallel.unshard_q_like(parts["o"], B, Hq), o)
    assert torch.equal(parallel.unshard_q_like(parts["lse"], B, Hq), lse)
    _assert_dkv_reproduce(ws.dims, parallel.unshard_kv_like(parts["dk"], B, Hkv), dk, "dk")
    _assert_dkv_reproduce(ws.dims, parallel.unshard_kv_like(parts["dv"], B, Hkv), dv, "dv")
    assert O.rel_l2(dq.float().cpu(), parallel.unshard_q_like(parts["dq"], B, Hq).float().cpu()) < DQ_RERUN_TOL


@pytest.mark.parametrize("B,Hq,Hkv,S,D", [(1, 4, 1, 256, 128), (1, 4, 4, 512, 64), (2, 8, 2, 384, 128)])
def test_forward_mxfp4_pv_route_matches_oracle(B, Hq, Hkv, S, D):
    """The diagnostic route: P as MXFP4 in 32-key groups (E8M0, ceil), V as sequence-grouped MXFP4 (cut-off
    exponent), row sum over the represented P.  V codes and scale pages bit-exact; O and LSE as the FP8 route."""
    q, k, v, _ = O.make_attention_inputs(B, Hq, Hkv, S, D, seed=20260901 + S + D, rope=(D == 128))
    fwd = O.attn_forward(q, k, v, pv_format="mxfp4_e8m0_block32")
    o, lse, ws = attention.attn_forward(q.to(DEV), k.to(DEV), v.to(DEV), pv_format="mxfp4_e8m0_block32")
    ws.check_status()
    codes, scales, _ = O.mxfp4_v_sequence(v)
    ops = ws.operands()
    assert torch.equal(ops["v_mx_codes"].cpu(), codes)
    # pages: row = feature, k-block = 32-key group within the 128-key tile
    want_pages = torch.zeros(B, Hkv, S // 128, 512, dtype=torch.uint8)
    d_idx = torch.arange(D)
    for kb in range(4):
        off = (d_idx % 32) * 16 + ((d_idx % 128) // 32) * 4 + kb
        want_pages[..., off] = scales.reshape(B, Hkv, D, S // 128, 4)[..., kb].permute(0, 1, 3, 2)
    assert torch.equal(ops["v_mx_scales"].cpu(), want_pages)
    torch.cuda.synchronize()
    assert O.rel_l2(fwd.o, o.cpu()) < 1e-2, O.rel_l2(fwd.o, o.cpu())
    # LSE: the row sum is over FP4-represented probabilities, so where the 2-ulp ex2.approx lands on the other side of
    # an E2M1 rounding boundary than the oracle's exp2, one term of one row moves by up to two code steps.  Such rows
    # are rare (boundary hits at 1e-7 relative distance); all others meet the 1e-3 bound of the FP8 route.
    err = (fwd.lse - lse.cpu()).abs()
    assert O.rel_l2(fwd.lse, lse.cpu()) < 1e-2
    assert (err > 1e-3).float().mean() < 1e-4 and err.max() < 5e-3, (float((err > 1e-3).float().mean()), float(err.max()))


def test_backward_refuses_the_forward_only_mxfp4_route():
    q, k, v, do = (t.to(DEV) for t in O.make_attention_inputs(1, 4, 1, 256, 128, seed=3))
    o, lse, ws = attention.attn_forward(q, k, v, pv_format="mxfp4_e8m0_block32")
    with pytest.raises(Exception, match="forward only"):
        attention.attn_backward(o, lse, do, ws)


@pytest.mark.parametrize("B,Hq,Hkv,S,D,pv", [(1, 4, 1, 384, 128, "e4m3_fp8"), (1, 4, 2, 256, 64, "e4m3_fp8"),
                                             (1, 4, 1, 256, 128, "mxfp4_e8m0_block32")])
def test_forward_without_mask_matches_oracle(B, Hq, Hkv, S, D, pv):
    """FA4B_MASK_NONE: every query sees every key (the off-diagonal blocks of a sequence-sharded run, and the
    reference's non-causal inference shape)."""
    q, k, v, do = O.make_attention_inputs(B, Hq, Hkv, S, D, seed=606 + S, rope=(D == 128))
    fwd = O.attn_forward(q, k, v, pv_format=pv, causal=False)
    o, lse, ws = attention.attn_forward(q.to(DEV), k.to(DEV), v.to(DEV), pv_format=pv, causal=False)
    ws.check_status()
    torch.cuda.synchronize()
    assert O.rel_l2(fwd.o, o.cpu()) < 1e-2, O.rel_l2(fwd.o, o.cpu())
    assert O.rel_l2(fwd.lse, lse.cpu()) < 1e-2
    if pv == "e4m3_fp8":
        assert (fwd.lse - lse.cpu()).abs().max() < 1e-3
    if pv != "e4m3_fp8":
        with pytest.raises(Exception, match="forward only"):
            attention.attn_backward(o, lse, do.to(DEV), ws)
        return
    # the unmasked backward (the workspace remembers the mask of its forward)
    dq, dk, dv = attention.attn_backward(o, lse, do.to(DEV), ws)
    ws.check_status()
    do5, dstat, lstat = O.attn_bwd_preprocess(fwd.o, do, fwd.lse)
    want = O.attn_backward_operands(O.quantize_qk_heads(q)[3], O.fp8_operand(q).float(), O.quantize_qk_heads(k)[3], O.fp8_operand(k).float(),
                                    O.fp8_operand(v).float(), do5.float(), dstat, lstat, D ** -0.5, causal=False)
    for w, g_, name in zip(want, (dq, dk, dv), ("dq", "dk", "dv")):
        assert O.rel_l2(w / 1024, g_.float().cpu()) < 2e-2, (name, O.rel_l2(w / 1024, g_.float().cpu()))


def test_full_size_properties_at_the_benchmark_shape():
    """C2 (B2, Hq32, Hkv8, S8192, D128) is too large for the CPU oracle as a whole, so the full size is checked
    through (a) a property: permuting the kv groups permutes O and LSE bit for bit (every statistic is local to a
    (batch, head) slice); (b) a slab: by (a) one (batch, kv head) unit of the full run equals that unit run alone, so
    the oracle of one unit (4 query heads, S = 8192) checks O, LSE, dQ, dK, dV of its rows in the full run;
    (c) dK and dV reproduce from run to run (bit for bit where at most two partial sums meet) and zero dO gives
    exactly zero gradients."""
    B, Hq, Hkv, S, D = 2, 32, 8, 8192, 128
    q, k, v, do = O.make_attention_inputs(1, 4 * Hkv, Hkv, S, D, seed=20260825, rope=True, do_std=0.01)
    # batch 1 is batch 0 with the kv groups in reverse order: the permutation property and the slab in one run
    G = Hq // Hkv
    perm_kv = torch.arange(Hkv - 1, -1, -1)
    perm_q = (perm_kv[:, None] * G + torch.arange(G)[None, :]).reshape(-1)
    qd = torch.cat([q, q[:, perm_q]]).to(DEV)
    kd = torch.cat([k, k[:, perm_kv]]).to(DEV)
    vd = torch.cat([v, v[:, perm_kv]]).to(DEV)
    dod = torch.cat([do, do[:, perm_q]]).to(DEV)
    o, lse, ws = attention.attn_forward(qd, kd, vd)
    ws.check_status()
    dq, dk, dv = attention.attn_backward(o, lse, dod, ws)
    ws.check_status()
    # (a)
    pq, pk = perm_q.to(DEV), perm_kv.to(DEV)
    assert torch.equal(o[1], o[0][pq]) and torch.equal(lse[1], lse[0][pq])
    _assert_dkv_reproduce(ws.dims, dk[1:2], dk[0:1][:, pk], "dk")
    _assert_dkv_reproduce(ws.dims, dv[1:2], dv[0:1][:, pk], "dv")
    # (b) kv head 5 of batch 0 against the oracle of that unit alone
    hk = 5
    hq = slice(hk * G, (hk + 1) * G)
    qu, ku, vu, dou = q[:, hq], k[:, hk:hk + 1], v[:, hk:hk + 1], do[:, hq]
    fwd = O.attn_forward(qu, ku, vu, query_chunk=512)
    want = O.attn_backward(qu, ku, vu, fwd.o, fwd.lse, dou, query_chunk=512)
    assert O.rel_l2(fwd.o, o[0:1, hq].cpu()) < 1e-2 and (fwd.lse - lse[0:1, hq].cpu()).abs().max() < 1e-3
    for w, g_, name in zip(want, (dq[0:1, hq], dk[0:1, hk:hk + 1], dv[0:1, hk:hk + 1]), ("dq", "dk", "dv")):
        assert O.rel_l2(w, g_.cpu()) < 2e-2, (name, O.rel_l2(w, g_.cpu()))
    # (c)
    dq2, dk2, dv2 = attention.attn_backward(o, lse, dod, ws)
    ws.check_status()
    _assert_dkv_reproduce(ws.dims, dk2, dk, "dk")
    _assert_dkv_reproduce(ws.dims, dv2, dv, "dv")
    assert O.rel_l2(dq.float().cpu(), dq2.float().cpu()) < DQ_RERUN_TOL
    dq0, dk0, dv0 = attention.attn_backward(o, lse, torch.zeros_like(dod), ws)
    ws.check_status()
    assert not dq0.any() and not dk0.any() and not dv0.any()


def test_forward_and_backward_replay_from_a_cuda_graph():
    """The entry points only enqueue work on the caller's stream (memsets, kernels; tensor maps travel by value),
    so after one warm-up call a forward + backward pair can be captured once and replayed."""
    B, Hq, Hkv, S, D = 1, 8, 2, 1024, 128
    q, k, v, do = (t.to(DEV) for t in O.make_attention_inputs(B, Hq, Hkv, S, D, seed=91, rope=True, do_std=0.01))
    o_ref, lse_ref, ws = attention.attn_forward(q, k, v)
    grads_ref = attention.attn_backward(o_ref, lse_ref, do, ws)
    ws.check_status()
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        o, lse, ws_g = attention.attn_forward(q, k, v)
        dq, dk, dv = attention.attn_backward(o, lse, do, ws_g)
    for _ in range(2):
        o.zero_()
        dk.zero_()
        graph.replay()
        torch.cuda.synchronize()
        assert torch.equal(o, o_ref) and torch.equal(lse, lse_ref)
        _assert_dkv_reproduce(ws.dims, dk, grads_ref[1], "dk")
        _assert_dkv_reproduce(ws.dims, dv, grads_ref[2], "dv")
        assert O.rel_l2(grads_ref[0].float().cpu(), dq.float().cpu()) < DQ_RERUN_TOL
    ws_g.check_status()


def test_backward_block_calls_against_oracle_and_the_single_kernel():
    """The pieces a sequence-sharded backward is made of: an unmasked block call with the keys of another operand
    cache (against the oracle's operand-level arithmetic), and a causal run split into block calls over two
    sequence halves that accumulate dQ in the workspace and dK/dV through fa4b_attn_accumulate (against the single
    kernel over the whole sequence)."""
    B, Hq, Hkv, S, D = 1, 4, 1, 512, 128
    q, k, v, do = O.make_attention_inputs(B, Hq, Hkv, S, D, seed=515, rope=True, do_std=0.01)
    qd_, kd_, vd_, dod = (t.to(DEV) for t in (q, k, v, do))
    o, lse, ws = attention.attn_forward(qd_, kd_, vd_)
    dq_ref, dk_ref, dv_ref = attention.attn_backward(o, lse, dod, ws)
    ws.check_status()
    # the two halves as their own operand caches, quantised with the amax of the whole sequence
    h = S // 2
    halves = []
    for i in range(2):
        sl = slice(i * h, (i + 1) * h)
        qs, ks, vs = (t[:, :, sl].contiguous() for t in (qd_, kd_, vd_))
        w = attention.alloc_workspace(attention.make_dims(qs, ks, None, "e4m3_fp8"), DEV)
        attention.attn_prepare(qs, ks, vs, w, phase="amax")
        halves.append((w, qs, ks, vs))
    amax = torch.maximum(halves[0][0].amax(), halves[1][0].amax()).clone()
    assert torch.equal(amax, ws.amax())
    for i, (w, qs, ks, vs) in enumerate(halves):
        w.amax().copy_(amax)
        attention.attn_prepare(qs, ks, vs, w, phase="quantize")
        sl = slice(i * h, (i + 1) * h)
        attention.attn_bwd_preprocess(o[:, :, sl].contiguous(), lse[:, :, sl].contiguous(), dod[:, :, sl].contiguous(), w)
    w0, w1 = halves[0][0], halves[1][0]
    # unmasked block (queries of the late half, keys of the early half) against the oracle
    _, dk_blk, dv_blk = attention.attn_backward_prepared(w1, w0, causal=False, write_dq=False)
    w1.check_status()
    fwd = O.attn_forward(q, k, v)
    do5, dstat, lstat = O.attn_bwd_preprocess(fwd.o, do, fwd.lse)
    am_q, am_k = q.float().abs().amax(dim=(2, 3)), k.float().abs().amax(dim=(2, 3))
    qdq = O.quantize_qk_heads(q[:, :, h:], am_q)[3]
    kdq = O.quantize_qk_heads(k[:, :, :h], am_k)[3]
    want = O.attn_backward_operands(qdq, O.fp8_operand(q[:, :, h:]).float(), kdq, O.fp8_operand(k[:, :, :h]).float(),
                                    O.fp8_operand(v[:, :, :h]).float(), do5[:, :, h:].float(), dstat[:, :, h:], lstat[:, :, h:],
                                    D ** -0.5, causal=False)
    assert O.rel_l2(want[1] / 1024, dk_blk.float().cpu()) < 2e-2 and O.rel_l2(want[2] / 1024, dv_blk.float().cpu()) < 2e-2
    # the whole causal run as three block calls
    dk_acc = torch.zeros(B, Hkv, S, D, dtype=torch.float32, device=DEV)
    dv_acc = torch.zeros_like(dk_acc)
    dq0, dk00, dv00 = attention.attn_backward_prepared(w0, w0, causal=True)                      # early x early
    _, dk10, dv10 = attention.attn_backward_prepared(w1, w0, causal=False, write_dq=False)        # late x early
    dq1, dk11, dv11 = attention.attn_backward_prepared(w1, w1, causal=True, keep_dq_accum=True)   # late x late
    w0.check_status()
    w1.check_status()
    for acc, parts in ((dk_acc, (dk00, dk10, dk11)), (dv_acc, (dv00, dv10, dv11))):
        lo, hi = acc[:, :, :h].contiguous(), acc[:, :, h:].contiguous()
        attention.attn_accumulate(lo, parts[0])
        attention.attn_accumulate(lo, parts[1])
        attention.attn_accumulate(hi, parts[2])
        acc[:, :, :h], acc[:, :, h:] = lo, hi
    assert O.rel_l2(dq_ref.float().cpu(), torch.cat([dq0, dq1], dim=2).float().cpu()) < 2e-3
    assert O.rel_l2(dk_ref.float().cpu(), dk_acc.cpu()) < 4e-3 and O.rel_l2(dv_ref.float().cpu(), dv_acc.cpu()) < 4e-3


@pytest.mark.parametrize("D,S", [(128, 2048), (64, 1024)])
def test_dq_partial_sums_as_f16_pairs_or_fp32(D, S):
    """The default backward adds the key tiles' partial dQ sums as f16 pairs (half the reduction traffic); both that
    form and the FP32 form requested by dq_sums_fp32 stay within the dQ tolerance, the FP32 form an order of
    magnitude closer to the oracle, and dK / dV do not depend on the choice."""
    q, k, v, do = O.make_attention_inputs(1, 4, 1, S, D, seed=11, do_std=0.01)
    fwd = O.attn_forward(q, k, v)
    want = O.attn_backward(q, k, v, fwd.o, fwd.lse, do)
    o, lse, ws = attention.attn_forward(q.to(DEV), k.to(DEV), v.to(DEV))
    dq16, dk16, dv16 = attention.attn_backward(o, lse, do.to(DEV), ws)
    dq32, dk32, dv32 = attention.attn_backward(o, lse, do.to(DEV), ws, dq_sums_fp32=True)
    ws.check_status()
    e16, e32 = O.rel_l2(want[0], dq16.float().cpu()), O.rel_l2(want[0], dq32.float().cpu())
    assert e32 < 1e-3 and e16 < 4e-3, (e16, e32)
    assert O.rel_l2(dq32.float().cpu(), dq16.float().cpu()) < DQ_RERUN_TOL
    _assert_dkv_reproduce(ws.dims, dk16, dk32, "dk")
    _assert_dkv_reproduce(ws.dims, dv16, dv32, "dv")

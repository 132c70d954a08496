"""Pin the CPU oracle to the reference: its known-answer tests restated, and
fixtures produced by importing the reference's Python (tests/golden/make_golden.py).
Everything here is bit-exact unless a tolerance is written next to the check."""

import numpy as np
import torch

import fa4b_oracle as O


def _bf16(a):
    return torch.from_numpy(a.copy()).view(torch.bfloat16)


def test_e2m1_rne_midpoints_match_reference_kat(golden_dir):
    # tests/test_projection_quantization_reference.py:81-95 of the reference
    fx = np.load(golden_dir / "quantizers.npz")
    mid = torch.from_numpy(fx["e2m1_midpoints"])
    want = torch.from_numpy(fx["e2m1_midpoints_rne"])
    assert want.tolist() == [0.0, 1.0, 1.0, 2.0, 2.0, 4.0, 4.0]
    assert torch.equal(O.e2m1_decode(O.e2m1_rne_codes(mid)), want)
    assert torch.equal(O.e2m1_decode(O.e2m1_rne_codes(-mid)), -want)
    # sign bit is kept when the magnitude rounds to zero
    # (tests/test_e4m3_to_mxfp4_v_contract.py:465-478 of the reference)
    assert O.e2m1_rne_codes(torch.tensor([-0.1, -0.0, 0.1])).tolist() == [8, 8, 0]
    assert O.e2m1_rne_codes(torch.tensor([7.0, -100.0, 6.0])).tolist() == [7, 15, 7]


def test_nvfp4_rowwise_matches_reference_fixture(golden_dir):
    fx = np.load(golden_dir / "quantizers.npz")
    x = _bf16(fx["x"])
    q = O.nvfp4_quantize(x)
    assert torch.equal(q.dequant().bfloat16().view(torch.int16), torch.from_numpy(fx["nvfp4_values"]))
    assert torch.equal(q.scales.view(torch.float8_e4m3fn).float(), torch.from_numpy(fx["nvfp4_block_scales"]))
    assert float(q.global_scale) == float(fx["nvfp4_global_decode"])
    # the stock bucketize payload differs only at exact ties
    stock = _bf16(fx["nvfp4_stock_values"])
    differing = (stock != q.dequant().bfloat16()).sum().item()
    assert 0 < differing <= 64


def test_nvfp4_transposed_matches_reference_fixture(golden_dir):
    fx = np.load(golden_dir / "quantizers.npz")
    x = _bf16(fx["x"])
    q = O.nvfp4_quantize_transposed(x)
    assert q.codes.shape == (256, 64)
    assert torch.equal(q.dequant().bfloat16().view(torch.int16), torch.from_numpy(fx["nvfp4_t_values"]))
    assert torch.equal(q.scales.view(torch.float8_e4m3fn).float(), torch.from_numpy(fx["nvfp4_t_block_scales"]))


def test_nvfp4_weight_tiles_match_reference_fixture(golden_dir):
    # fake_quantize_nvfp4(block_shape=(16, 16)) and transpose_prepared_nvfp4_weight_reference, run by the generator
    fx = np.load(golden_dir / "quantizers.npz")
    x = _bf16(fx["x"])
    fwd, tr = O.nvfp4_quantize_weight(x)
    assert torch.equal(fwd.dequant().bfloat16().view(torch.int16), torch.from_numpy(fx["nvfp4_w2d_values"]))
    tile_scales = fwd.scales.view(torch.float8_e4m3fn).float()[0::16]
    assert torch.equal(tile_scales, torch.from_numpy(fx["nvfp4_w2d_block_scales"]))
    assert torch.equal(fwd.codes, torch.from_numpy(fx["nvfp4_w2d_payload"]))
    assert torch.equal(fwd.pages(), torch.from_numpy(fx["nvfp4_w2d_pages"]))
    # the operand of the transposed weight is the reference's byte-level transposition of the first
    assert torch.equal(tr.codes, torch.from_numpy(fx["nvfp4_w2d_t_payload"]))
    assert torch.equal(tr.pages(), torch.from_numpy(fx["nvfp4_w2d_t_pages"]))
    assert torch.equal(tr.dequant(), fwd.dequant().t())
    # a tile never has a larger error than the 1x16 recipe allows for its amax: codes stay within +-6
    assert float(fwd.dequant().abs().max()) <= float(x.float().abs().max()) * 1.07


def test_mxfp4_matches_reference_fixture(golden_dir):
    fx = np.load(golden_dir / "quantizers.npz")
    x = _bf16(fx["x"])
    for mode in ("ceil", "rte"):
        q = O.mxfp4_quantize(x, mode)
        assert torch.equal(q.dequant().bfloat16().view(torch.int16), torch.from_numpy(fx[f"mxfp4_{mode}_values"]))
        e = q.scales.float()
        scale = torch.where(e > 0, torch.exp2(e - 127.0), torch.zeros_like(e))
        assert torch.equal(scale, torch.from_numpy(fx[f"mxfp4_{mode}_block_scales"]))


def test_mxfp4_v_sequence_groups_match_reference_fixture(golden_dir):
    fx = np.load(golden_dir / "quantizers.npz")
    v = _bf16(fx["v"])  # [B,S,H,D]
    codes, scales, deq = O.mxfp4_v_sequence(v.permute(0, 2, 1, 3).contiguous())
    assert codes.shape == (1, 2, 32, 32) and scales.shape == (1, 2, 32, 2)
    got = deq.permute(0, 2, 1, 3).bfloat16().contiguous()
    assert torch.equal(got.view(torch.int16), torch.from_numpy(fx["v_values"]))
    e = scales.float()
    assert torch.equal(torch.where(e > 0, torch.exp2(e - 127.0), torch.zeros_like(e)),
                       torch.from_numpy(fx["v_block_scales"]))


def test_scale_page_byte_order():
    # projection_quantization_reference.py:314-322
    rows, kb = 256, 8
    s = torch.arange(rows * kb, dtype=torch.int64).remainder(251).to(torch.uint8).reshape(rows, kb)
    pages = O.scales_to_pages(s)
    assert pages.shape == (2, 2, 512)
    for r, c in ((0, 0), (31, 3), (32, 0), (127, 7), (128, 4), (200, 5), (255, 7)):
        off = (r % 32) * 16 + ((r % 128) // 32) * 4 + (c % 4)
        assert pages[r // 128, c // 4, off] == s[r, c]
    assert torch.equal(O.pages_to_scales(pages), s)


def test_nibble_packing_even_element_low():
    codes = torch.tensor([[1, 2, 15, 0]], dtype=torch.uint8)
    assert O.pack_nibbles(codes).tolist() == [[0x21, 0x0F]]
    assert torch.equal(O.unpack_nibbles(O.pack_nibbles(codes)), codes)


def test_all_zero_and_saturating_blocks():
    x = torch.zeros(128, 64).bfloat16()
    q = O.nvfp4_quantize(x)
    assert q.codes.sum() == 0 and q.scales.sum() == 0 and float(q.global_scale) == 0.0
    m = O.mxfp4_quantize(x)
    assert m.codes.sum() == 0 and m.scales.sum() == 0
    x[0, 0] = 3.0
    q = O.nvfp4_quantize(x)
    # the block holding the tensor maximum gets the E4M3 end point and code 6
    assert q.scales[0, 0] == 0x7E and (q.codes[0, 0] & 0xF) == 7


def test_backward_collapses_to_reference_fp32_backward(golden_dir):
    """With E4M3 scores and no P/dS rounding the emulation must equal the
    reference's represented-operand FP32 backward (S=128, one kv group)."""
    fx = np.load(golden_dir / "backward_s128.npz")
    def e4(a):  # [B,S,H,D] e4m3 bits of 4*x -> bf16 [B,H,S,D]
        t = torch.from_numpy(a.copy()).view(torch.float8_e4m3fn).float() / 4.0
        return t.permute(0, 2, 1, 3).contiguous().bfloat16()
    q, k, v, do = e4(fx["q"]), e4(fx["k"]), e4(fx["v"]), e4(fx["dout"])
    lstat = torch.from_numpy(fx["lstat"])[:, :, 0]
    dstat = torch.from_numpy(fx["dstat"])[:, :, 0]
    do5 = do.float() * 4.0  # the validator's dO is E4M3-represented; keep it exact (no E5M2 step)
    dq, dk, dv = O.attn_backward(q, k, v, None, None, do, softmax_scale=float(fx["softmax_scale"]),
                                 score_operands="e4m3", quantize_p_ds=False, stats=(do5, dstat, lstat))
    for got, name in ((dq, "dq"), (dk, "dk"), (dv, "dv")):
        want = torch.from_numpy(fx[name]).permute(0, 2, 1, 3)
        assert O.rel_l2(want, got) < 2e-5, name  # FP32 summation order only


def test_backward_quantised_route_stays_close_to_fp32_backward(golden_dir):
    fx = np.load(golden_dir / "backward_s128.npz")
    def e4(a):
        t = torch.from_numpy(a.copy()).view(torch.float8_e4m3fn).float() / 4.0
        return t.permute(0, 2, 1, 3).contiguous().bfloat16()
    q, k, v, do = e4(fx["q"]), e4(fx["k"]), e4(fx["v"]), e4(fx["dout"])
    fwd = O.attn_forward(q, k, v, softmax_scale=float(fx["softmax_scale"]))
    dq, dk, dv = O.attn_backward(q, k, v, fwd.o, fwd.lse, do, softmax_scale=float(fx["softmax_scale"]))
    for got, name, tol in ((dq, "dq", 0.25), (dk, "dk", 0.25), (dv, "dv", 0.1)):
        want = torch.from_numpy(fx[name]).permute(0, 2, 1, 3)
        assert O.rel_l2(want, got) < tol, (name, O.rel_l2(want, got))


def test_forward_tracks_fp32_attention_and_zero_dout_gives_zero_grads():
    q, k, v, do = O.make_attention_inputs(1, 4, 2, 256, 64, seed=3)
    fwd = O.attn_forward(q, k, v)
    ref_o, ref_lse = O.attn_reference_fp32(q, k, v)
    assert O.rel_l2(ref_o, fwd.o) < 0.12  # NVFP4 scores + FP8 P/V vs exact math
    assert (fwd.lse - ref_lse).abs().max() < 0.5
    # validate_native_tk_d128_backward.py:707-738: exact-zero dO => exact-zero gradients
    dq, dk, dv = O.attn_backward(q, k, v, fwd.o, fwd.lse, torch.zeros_like(do))
    assert not dq.any() and not dk.any() and not dv.any()


def test_forward_rounding_is_invariant_to_the_running_maximum():
    """The E4M3 probability of 2^(s - mhat + 8) does not depend on which
    integer mhat a streaming kernel happened to hold when it saw the tile."""
    g = torch.Generator().manual_seed(1)
    s2 = torch.randn(64, 256, generator=g) * 3.0
    mhat = torch.ceil(s2.amax(dim=1, keepdim=True))
    final = O.e4m3_round(torch.exp2(s2 - mhat + 8.0)).float()
    early = O.e4m3_round(torch.exp2(s2 - (mhat - 3.0) + 8.0).clamp(max=448.0)).float() / 8.0
    keep = torch.exp2(s2 - mhat + 8.0) >= 2.0 ** -6  # normal range of the final grid
    keep &= torch.exp2(s2 - (mhat - 3.0) + 8.0) <= 448.0
    assert torch.equal(final[keep], early[keep])


def test_rope_pair_reference_is_one_rounding_per_step_and_close_to_the_complex_rotation():
    # apply_rope_pair (projection_fp4_epilogue.cuh:447-479): t = bf16(pair * cos); out = bf16(fma(perp, sin, t))
    g = torch.Generator().manual_seed(7)
    x = torch.randn(1, 64, 3, 32, generator=g).bfloat16()
    cos, sin = O.rope_tables(64, 32)
    y = O.rope_pair_reference(x, cos, sin)
    xc = torch.view_as_complex(x.float().reshape(1, 64, 3, 16, 2))
    want = torch.view_as_real(xc * torch.complex(cos.float(), sin.float())[None, :, None, :]).flatten(3)
    assert O.rel_l2(want, y.float()) < 5e-3                       # bf16 tables and two bf16 roundings
    assert torch.equal(y[:, 0], x[:, 0])                         # position 0: cos = 1, sin = 0
    z = O.rope_pair_reference(y, cos, sin, inverse=True)
    assert O.rel_l2(x.float(), z.float()) < 1e-2
    # hand-checked pair: (x, y) = (1.5, -2), cos = 0.5, sin = 0.25 -> t = (0.75, -1); out = (0.75 + 0.5, -1 + 0.375)
    one = torch.tensor([1.5, -2.0]).bfloat16().reshape(1, 1, 1, 2)
    out = O.rope_pair_reference(one, torch.tensor([[0.5]]).bfloat16(), torch.tensor([[0.25]]).bfloat16())
    assert out.flatten().tolist() == [1.25, -0.625]


def test_float64_to_bf16_rounds_once():
    # 1 + 2^-8 is a bf16 tie (rounds to even: 1.0); a float64 just above it must round up although the detour through
    # float32 alone would first land on the tie
    v = torch.tensor([1.0 + 2.0 ** -8, 1.0 + 2.0 ** -8 + 2.0 ** -40, 1.0 + 2.0 ** -8 - 2.0 ** -40, 1.0 + 3 * 2.0 ** -8], dtype=torch.float64)
    got = O._round_f64_to_bf16(v).double().tolist()
    assert got == [1.0, 1.0 + 2.0 ** -7, 1.0, 1.0 + 2.0 ** -6]


def test_project_reference_and_block_composition_shapes():
    g = torch.Generator().manual_seed(8)
    x = torch.randn(128, 64, generator=g).bfloat16()
    w = (torch.randn(32, 64, generator=g) * 0.1).bfloat16()
    a, (wf, wt) = O.nvfp4_quantize(x), O.nvfp4_quantize_weight(w)
    y = O.project_nvfp4_reference(a, wf)
    assert y.shape == (128, 32) and y.dtype == torch.bfloat16
    assert O.rel_l2((a.dequant() @ wf.dequant().t()), y.float()) < 4e-3
    assert torch.equal(wt.dequant(), wf.dequant().t())


def test_encode_centric_recipe_against_blocks_worked_by_hand():
    """Known answers for the TK quantiser's default recipe, worked from core.cuh:47-60, 103-113 and
    fused_amax_quantize.cuh:235-256 of the reference without this repo's restatement:
    S_enc = 2688 / amax; M = E4M3(6 / (bamax S_enc)) (448 when bamax <= 1e-9); coeff = M S_enc;
    stored scale = E4M3(1 / M); code = E2M1_rne(x coeff).  The tensor's amax is 2688, so S_enc = 1.
    E4M3 bytes: 1 = 0x38, 2 = 0x40, 0.5 = 0x30, 1.25 = 0x3A, 0.8125 = 0x35, 448 = 0x7E, 2^-9 = 0x01.
    E2M1 codes: 0, .5, 1, 1.5, 2, 3, 4, 6 = 0..7 (ties to the even code)."""
    x = torch.zeros(2, 64)
    # block (0,0): bamax 6 -> M = 1, scale 1; elements exercise every tie of the payload grid
    x[0, :16] = torch.tensor([6, -3, 1.5, 0.75, 0.25, 1.25, 1.75, 2.5, 3.5, 5, -0.75, -5, 0, 0.5, 2, 4])
    want00 = [7, 8 + 5, 3, 2, 0, 2, 4, 4, 6, 6, 8 + 2, 8 + 6, 0, 1, 4, 6]
    # block (0,1): holds the tensor maximum 2688 -> M = 6/2688 = 0.00223 -> sub-normal E4M3 2^-9; the stored scale
    # 1/M = 512 saturates at 448; 2688 * 2^-9 = 5.25 -> 6; 1024 * 2^-9 = 2 -> 2; 512 * 2^-9 = 1
    x[0, 16:32] = torch.tensor([2688, 1024, 512, -2688] + [0] * 12)
    want01 = [7, 4, 2, 15] + [0] * 12
    # block (0,2): all zero -> M = 448, stored scale E4M3(1/448) = 2^-9 (not zero), codes zero
    # block (0,3): bamax 2^-10 -> M = 6144 saturates at 448; 2^-10 * 448 = 0.4375 -> 0.5; 2^-12 * 448 = 0.109 -> 0
    x[0, 48:64] = torch.tensor([2.0 ** -10, -(2.0 ** -10), 2.0 ** -12] + [0] * 13)
    want03 = [1, 9, 0] + [0] * 13
    # block (1,0): bamax 3 -> M = 2, scale 0.5; 0.375 * 2 = 0.75 (tie -> 1), 0.125 * 2 = 0.25 (tie -> 0), 3 * 2 = 6
    x[1, :16] = torch.tensor([3, 0.375, 0.125, -0.375] + [0] * 12)
    want10 = [7, 2, 0, 10] + [0] * 12
    # block (1,1): bamax 5 -> M = 1.2 -> E4M3 1.25; stored scale E4M3(0.8) = 0.8125; 5 * 1.25 = 6.25 -> 6;
    # 4 * 1.25 = 5 (tie between 4 and 6 -> 4); 1 * 1.25 = 1.25 (tie -> 1); 2 * 1.25 = 2.5 (tie -> 2)
    x[1, 16:32] = torch.tensor([5, 4, 1, 2, -4] + [0] * 11)
    want11 = [7, 6, 2, 4, 14] + [0] * 11
    q = O.nvfp4_quantize_encode_centric(x.bfloat16())
    codes = O.unpack_nibbles(q.codes)
    assert float(q.global_scale) == 1.0
    assert codes[0, :16].tolist() == want00 and codes[0, 16:32].tolist() == want01 and codes[0, 48:64].tolist() == want03
    assert codes[1, :16].tolist() == want10 and codes[1, 16:32].tolist() == want11
    assert not codes[0, 32:48].any() and not codes[1, 32:].any()
    assert q.scales[0].tolist() == [0x38, 0x7E, 0x01, 0x01]
    assert q.scales[1].tolist() == [0x30, 0x35, 0x01, 0x01]
    # an all-zero tensor: S_enc = 1, every block as the zero block above
    z = O.nvfp4_quantize_encode_centric(torch.zeros(1, 32).bfloat16())
    assert z.scales.tolist() == [[0x01, 0x01]] and not z.codes.any() and float(z.global_scale) == 0.0


def test_forward_emulation_passes_the_reference_forward_gate():
    """validate_causal_gqa_fp8pv_batch.py:268-324, 705-706 of the reference: O against exact attention on the decoded
    operands, cosine >= 0.999 and rel-L2 <= 0.03 -- the check that pins the one free choice of the forward emulation
    (integer reference point, 2^8 lift, exponential split) to what the reference accepts of its own kernel."""
    for (B, Hq, Hkv, S, D, rope) in ((1, 4, 1, 256, 128, True), (1, 4, 4, 512, 64, False)):
        q, k, v, _ = O.make_attention_inputs(B, Hq, Hkv, S, D, seed=20260825, rope=rope)
        for gs in ("amax_per_bh", "one"):
            fwd = O.attn_forward(q, k, v, global_scale=gs)
            cosine, rel = O.represented_forward_gate(fwd.o, fwd)
            assert cosine >= 0.999 and rel <= 0.03, (S, D, gs, cosine, rel)


def test_exponential_split_tracks_exp2_and_keeps_powers_of_two_scaling():
    x = torch.linspace(-40.0, 8.0, 20001)
    p, r = O.exp2_polynomial(x).double(), torch.exp2(x.double())
    assert ((p - r) / r).abs().max() < 8e-5
    # an integer shift of the exponent is an exact power-of-two factor: what makes the rounding of a probability
    # independent of the (integer) reference point a streaming kernel holds
    xe = torch.arange(-40 * 256, 5 * 256 + 1).float() / 256.0  # x + 3 is exact on this grid
    assert torch.equal(O.exp2_polynomial(xe + 3.0), O.exp2_polynomial(xe) * 8.0)
    e = torch.tensor([[0.0, 1.0, 2.5, 3.5, float("-inf"), 5.0] + [0.0] * 10])
    out = O.exp2_split(e)
    assert out[0, 4] == 0.0 and out[0, 0] == 1.0 and out[0, 1] == 2.0        # keys 0, 1: exponential unit
    assert out[0, 2] == O.exp2_polynomial(torch.tensor(2.5)) != 2.0 ** 2.5   # keys 2, 3 (pair 1): polynomial

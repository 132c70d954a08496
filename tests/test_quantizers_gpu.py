"""GPU parity of the block quantizers against the CPU oracle: codes, scale
pages and global scales bit-exact (integer/byte work, tolerance zero)."""

import pytest
import torch

import fa4b
import fa4b_oracle as O

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _same(a, b, what):
    a, b = a.cpu(), b.cpu()
    assert a.shape == b.shape, (what, a.shape, b.shape)
    bad = (a != b).sum().item()
    assert bad == 0, f"{what}: {bad} of {a.numel()} bytes differ"


@pytest.mark.parametrize("shape,seed", [((128, 128), 1), ((256, 512), 2), ((384, 1024), 3)])
def test_nvfp4_row_and_transposed_match_oracle(shape, seed):
    x, _ = O.make_quantizer_inputs(*shape, seed=seed)
    fp4_row, sc_row, fp4_col, sc_col, sg, am = fa4b.tk_quantize_for_gemm(x.to(DEV), return_transpose=True, encode_centric=False)
    ref = O.nvfp4_quantize(x)
    ref_t = O.nvfp4_quantize_transposed(x)
    assert float(am) == float(x.float().abs().amax())
    assert float(sg) == float(ref.global_scale)
    _same(fp4_row, ref.codes, "row codes")
    _same(sc_row, ref.pages(), "row scale pages")
    _same(fp4_col, ref_t.codes, "transposed codes")
    _same(sc_col, ref_t.pages(), "transposed scale pages")
    # decode utility agrees with the oracle's decode
    assert torch.equal(fa4b.dequant_nvfp4(fp4_row, sc_row, sg).cpu(), ref.dequant())


def test_nvfp4_edge_cases_zero_tensor_zero_blocks_ties_and_row_only():
    x = torch.zeros(128, 128, dtype=torch.bfloat16)
    out = fa4b.tk_quantize_for_gemm(x.to(DEV), return_transpose=False, encode_centric=False)
    assert out[2] is None and out[3] is None
    assert not out[0].any() and not out[1].any() and float(out[4]) == 0.0
    x, _ = O.make_quantizer_inputs(256, 256, seed=5)
    x[3, 32:64] = 0
    x[:, 17] = 0
    x[9, :16] = (torch.tensor([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0, 6.0] * 2) * float(x.float().abs().amax()) / 6.0).bfloat16()
    x[10, :16] = -x[9, :16]
    fp4_row, sc_row, fp4_col, sc_col, sg, _ = fa4b.tk_quantize_for_gemm(x.to(DEV), encode_centric=False)
    ref, ref_t = O.nvfp4_quantize(x), O.nvfp4_quantize_transposed(x)
    _same(fp4_row, ref.codes, "row codes")
    _same(sc_row, ref.pages(), "row pages")
    _same(fp4_col, ref_t.codes, "col codes")
    _same(sc_col, ref_t.pages(), "col pages")


def test_nvfp4_with_supplied_amax_and_strided_input():
    x, _ = O.make_quantizer_inputs(256, 512, seed=7)
    big = x.to(DEV)
    view = big[:, 128:384]  # ld = 512, cols = 256
    am = torch.tensor([float(x.float().abs().amax())], device=DEV)
    fp4_row, sc_row, _, _, sg, _ = fa4b.tk_quantize_for_gemm(view, return_transpose=False, amax_in=am, encode_centric=False)
    ref = O.nvfp4_quantize(x[:, 128:384].contiguous(), amax=am.cpu())
    _same(fp4_row, ref.codes, "row codes")
    _same(sc_row, ref.pages(), "row pages")


@pytest.mark.parametrize("shape,seed", [((128, 128), 4), ((256, 384), 5), ((512, 1024), 6)])
def test_nvfp4_weight_tiles_and_dual_transpose_match_oracle(shape, seed):
    w, _ = O.make_quantizer_inputs(*shape, seed=seed)
    w[16:32, 32:48] = 0.0  # an all-zero tile
    fwd, tr = fa4b.prepare_nvfp4_projection_weight_dual(w.to(DEV))
    ref, ref_t = O.nvfp4_quantize_weight(w)
    assert fwd[2].data_ptr() == tr[2].data_ptr() and float(fwd[2]) == float(ref.global_scale)
    _same(fwd[0], ref.codes, "weight codes")
    _same(fwd[1], ref.pages(), "weight scale pages")
    _same(tr[0], ref_t.codes, "transposed weight codes")
    _same(tr[1], ref_t.pages(), "transposed weight scale pages")
    single = fa4b.prepare_nvfp4_projection_weight(w.to(DEV))
    _same(single[0], ref.codes, "weight codes (single)")
    _same(single[1], ref.pages(), "weight scale pages (single)")


def test_nvfp4_weight_dual_is_a_transpose_at_projection_size():
    # 4096 x 4096 (a Llama-3-8B projection): the two operands decode to transposes of each other, and every
    # 16 x 16 tile carries one scale
    g = torch.Generator(device=DEV).manual_seed(11)
    w = (torch.randn(4096, 4096, device=DEV, generator=g) * 0.02).bfloat16()
    fwd, tr = fa4b.prepare_nvfp4_projection_weight_dual(w)
    a = fa4b.dequant_nvfp4(*fwd)
    b = fa4b.dequant_nvfp4(*tr)
    assert torch.equal(a, b.t())
    assert O.rel_l2(w.float().cpu(), a.cpu()) < 0.12
    ref, _ = O.nvfp4_quantize_weight(w[:256].cpu())  # a slab against the oracle (same tensor-wide amax needed)
    slab = O.nvfp4_quantize_weight(w.cpu())[0]
    _same(fwd[0], slab.codes, "codes at 4096 x 4096")
    _same(fwd[1], slab.pages(), "scale pages at 4096 x 4096")


@pytest.mark.parametrize("M,N,K,seed", [(128, 256, 256, 1), (256, 512, 1024, 2), (384, 768, 4096, 3), (384, 1280, 768, 4),
                                        (1152, 768, 1792, 5), (128, 4096, 256, 6)])
def test_project_nvfp4_matches_oracle_on_represented_operands(M, N, K, seed):
    x, _ = O.make_quantizer_inputs(M, K, seed=seed)
    w, _ = O.make_quantizer_inputs(N, K, seed=seed + 100)
    w = (w * 0.05).bfloat16()
    fp4, sc, _, _, sg, _ = fa4b.tk_quantize_for_gemm(x.to(DEV), return_transpose=False, encode_centric=False)
    weight = fa4b.prepare_nvfp4_projection_weight(w.to(DEV))
    y = fa4b.project_nvfp4((fp4, sc, sg), weight)
    assert y.shape == (M, N) and y.dtype == torch.bfloat16
    ref = O.project_nvfp4_reference(O.nvfp4_quantize(x), O.nvfp4_quantize_weight(w)[0])
    # FP32 sums on the tensor core against float64 sums: the same bf16 value except where the exact result sits
    # within an FP32 rounding of a bf16 boundary (tolerance: rel-L2 1e-4, no element off by more than one bf16 step)
    assert O.rel_l2(ref.float(), y.float().cpu()) < 1e-4
    step = torch.maximum(ref.float().abs(), torch.tensor(1e-3)) * 2.0 ** -7
    assert bool(((ref.float() - y.float().cpu()).abs() <= step).all())


def test_project_nvfp4_with_the_transposed_weight_gives_the_input_gradient_product():
    # dX = dY . W uses the [K, N] operand of the dual publication: same represented weight, transposed
    g = torch.Generator().manual_seed(9)
    w = (torch.randn(512, 256, generator=g) * 0.05).bfloat16()   # [N, K]
    dy = torch.randn(128, 512, generator=g).bfloat16()           # [M, N]
    fwd, tr = fa4b.prepare_nvfp4_projection_weight_dual(w.to(DEV))
    fp4, sc, _, _, sg, _ = fa4b.tk_quantize_for_gemm(dy.to(DEV), return_transpose=False, encode_centric=False)
    dx = fa4b.project_nvfp4((fp4, sc, sg), tr)                   # [M, K]
    ref = (O.nvfp4_quantize(dy).dequant().double() @ O.nvfp4_quantize_weight(w)[0].dequant().double()).to(torch.bfloat16)
    assert O.rel_l2(ref.float(), dx.float().cpu()) < 1e-4


def test_project_nvfp4_rejects_bad_shapes():
    a = (torch.zeros(128, 128, dtype=torch.uint8, device=DEV), torch.zeros(1, 4, 512, dtype=torch.uint8, device=DEV),
         torch.ones(1, device=DEV))
    w = (torch.zeros(128, 128, dtype=torch.uint8, device=DEV), torch.zeros(1, 4, 512, dtype=torch.uint8, device=DEV),
         torch.ones(1, device=DEV))
    with pytest.raises(ValueError):  # N = 128 is not a multiple of 256
        fa4b.project_nvfp4(a, w)
    with pytest.raises(ValueError):
        fa4b.project_nvfp4(a, (w[0][:, :64], w[1], w[2]))


@pytest.mark.parametrize("inverse", [False, True])
def test_rope_pair_matches_packed_bf16_oracle_bit_for_bit(inverse):
    g = torch.Generator().manual_seed(3)
    B, S, H, D = 2, 96, 5, 128
    big = torch.randn(B, S, H + 2, D + 64, generator=g).bfloat16()
    x = big[:, :, 1:H + 1, 32:32 + D]  # a strided view, as the q columns of a fused QKV projection are
    cos, sin = O.rope_tables(S, D)
    ref = O.rope_pair_reference(x, cos, sin, inverse=inverse)
    dev = big.to(DEV)
    xd = dev[:, :, 1:H + 1, 32:32 + D]
    fa4b.rope_pair_(xd, cos.to(DEV), sin.to(DEV), inverse=inverse)
    _same(xd.contiguous().view(torch.int16), ref.contiguous().view(torch.int16), "rotated values")
    # nothing outside the view moved
    keep = torch.ones_like(big, dtype=torch.bool)
    keep[:, :, 1:H + 1, 32:32 + D] = False
    assert torch.equal(dev.cpu()[keep], big[keep])


def test_rope_pair_inverse_undoes_the_rotation_within_bf16_rounding():
    g = torch.Generator(device=DEV).manual_seed(4)
    x = torch.randn(1, 4096, 8, 128, device=DEV, generator=g).bfloat16()
    cos, sin = (t.to(DEV) for t in O.rope_tables(4096, 128))
    y = fa4b.rope_pair_(x.clone(), cos, sin)
    z = fa4b.rope_pair_(y.clone(), cos, sin, inverse=True)
    assert O.rel_l2(x.float().cpu(), z.float().cpu()) < 1e-2   # two roundings to bf16 each way
    # the rotation keeps each pair's length (to bf16 rounding)
    n0 = x.float().reshape(-1, 2).norm(dim=1)
    n1 = y.float().reshape(-1, 2).norm(dim=1)
    assert float(((n0 - n1).abs() / n0.clamp_min(1e-3)).max()) < 2e-2


@pytest.mark.parametrize("B,S,Hq,Hkv,D,encode_centric", [(2, 256, 4, 2, 128, False), (1, 384, 8, 2, 128, True), (2, 128, 6, 2, 64, False),
                                                          (1, 256, 2, 1, 64, True)])
def test_pack_qkv_grads_is_the_oracle_of_rotation_then_quantisation_and_the_separate_passes(B, S, Hq, Hkv, D, encode_centric):
    """[dQ | dK | dV] -> inverse rotation -> NVFP4 rows and transposed, in one pass: equal byte for byte to the oracle's
    rotation followed by its quantiser, and to the three separate device passes; from three tensors and from the
    column ranges of one buffer; with the amax computed and supplied."""
    g = torch.Generator().manual_seed(100 + S + Hq)
    N = (Hq + 2 * Hkv) * D
    buf = (torch.randn(B * S, N, generator=g) * torch.logspace(-3, 0, N)[None, :]).bfloat16()   # dynamic range across the heads
    dq = buf[:, :Hq * D].view(B, S, Hq, D)
    dk = buf[:, Hq * D:(Hq + Hkv) * D].view(B, S, Hkv, D)
    dv = buf[:, (Hq + Hkv) * D:].view(B, S, Hkv, D)
    cos, sin = O.rope_tables(S, D)
    rotated = torch.cat([O.rope_pair_reference(dq, cos, sin, inverse=True).reshape(B * S, -1),
                         O.rope_pair_reference(dk, cos, sin, inverse=True).reshape(B * S, -1), dv.reshape(B * S, -1)], dim=1)
    quantise = O.nvfp4_quantize_encode_centric if encode_centric else O.nvfp4_quantize
    ref, ref_t = quantise(rotated), quantise(rotated.t().contiguous())
    cd, sd = cos.to(DEV), sin.to(DEV)
    dbuf = buf.to(DEV)
    views = (dbuf[:, :Hq * D].view(B, S, Hq, D), dbuf[:, Hq * D:(Hq + Hkv) * D].view(B, S, Hkv, D), dbuf[:, (Hq + Hkv) * D:].view(B, S, Hkv, D))
    separate = tuple(t.contiguous() for t in views)
    for name, (a, b, c) in (("views of one buffer", views), ("three tensors", separate)):
        out = fa4b.pack_qkv_grads(a, b, c, cd, sd, return_transpose=True, encode_centric=encode_centric)
        assert float(out[5]) == float(rotated.float().abs().amax()), name
        assert float(out[4]) == float(ref.global_scale), name
        _same(out[0], ref.codes, f"{name}: row codes")
        _same(out[1], ref.pages(), f"{name}: row scale pages")
        _same(out[2], ref_t.codes, f"{name}: transposed codes")
        _same(out[3], ref_t.pages(), f"{name}: transposed scale pages")
    assert torch.equal(dbuf.cpu(), buf)  # the gradients themselves are left alone
    # the passes it replaces
    two = dbuf.clone()
    fa4b.rope_pair_(two[:, :Hq * D].view(B, S, Hq, D), cd, sd, inverse=True)
    fa4b.rope_pair_(two[:, Hq * D:(Hq + Hkv) * D].view(B, S, Hkv, D), cd, sd, inverse=True)
    sep = fa4b.tk_quantize_for_gemm(two, return_transpose=True, encode_centric=encode_centric)
    # a supplied amax (the reference's delayed global scale) and a row-only call
    am = sep[5].clone()
    given = fa4b.pack_qkv_grads(*views, cd, sd, return_transpose=False, encode_centric=encode_centric, amax_in=am)
    assert given[2] is None and given[3] is None
    for i, what in ((0, "row codes"), (1, "row scale pages")):
        _same(given[i], sep[i], f"supplied amax: {what}")
    for i, what in ((0, "row codes"), (1, "row scale pages"), (2, "transposed codes"), (3, "transposed scale pages")):
        _same(out[i], sep[i], f"separate passes: {what}")


def test_quantizer_wait_status_is_clear_after_every_kind_of_call():
    """The tile kernels wait for their TMA load with a cycle limit and record a wait that ran out; after ordinary
    calls of every staging kind the record is clear."""
    from fa4b import quantizers as Q

    x, gamma = O.make_quantizer_inputs(256, 512, seed=9)
    xd, gd = x.to(DEV), gamma.to(DEV)
    fa4b.tk_quantize_for_gemm(xd, True, True)
    fa4b.tk_quantize_for_gemm(xd, False, False)
    fa4b.tk_fused_norm_quantize(xd, gd, 1e-6)
    fa4b.prepare_nvfp4_projection_weight_dual(xd)
    Q.check_status()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs in one process")
def test_quantizer_and_projection_on_a_second_device_of_the_same_process():
    """Per-device kernel attributes (shared-memory opt-in) and per-device caches: the same process quantises and
    projects on cuda:0 and then on cuda:1, with identical bytes."""
    x, _ = O.make_quantizer_inputs(256, 512, seed=21)
    w = (torch.randn(256, 512, generator=torch.Generator().manual_seed(22)) * 0.05).bfloat16()
    outs = []
    for dev in ("cuda:0", "cuda:1"):
        with torch.cuda.device(dev):
            a = fa4b.tk_quantize_for_gemm(x.to(dev), return_transpose=True, encode_centric=False)
            wq = fa4b.prepare_nvfp4_projection_weight(w.to(dev))
            y = fa4b.project_nvfp4((a[0], a[1], a[4]), wq)
            torch.cuda.synchronize(dev)
            outs.append([t.cpu() for t in a[:4]] + [y.cpu()])
    for t0, t1 in zip(*outs):
        assert torch.equal(t0, t1)


def test_pack_qkv_grads_at_the_layer_shape_equals_the_separate_passes():
    """Llama-3-8B layer shape (B2, S8192, Hq32, Hkv8, D128: a [16384, 6144] gradient matrix): the one-pass packer and
    the rotation + quantiser passes it replaces write the same bytes; the transposed plane is the row plane of the
    transposed matrix (checked on a slab through the decode utility)."""
    from fa4b import quantizers as Q

    B, S, Hq, Hkv, D = 2, 8192, 32, 8, 128
    g = torch.Generator(device=DEV).manual_seed(77)
    N = (Hq + 2 * Hkv) * D
    buf = (torch.randn(B * S, N, device=DEV, generator=g) * 0.02).bfloat16()
    views = (buf[:, :Hq * D].view(B, S, Hq, D), buf[:, Hq * D:(Hq + Hkv) * D].view(B, S, Hkv, D), buf[:, (Hq + Hkv) * D:].view(B, S, Hkv, D))
    cos, sin = (t.to(DEV) for t in O.rope_tables(S, D))
    fused = fa4b.pack_qkv_grads(*views, cos, sin, return_transpose=True, encode_centric=False)
    two = buf.clone()
    fa4b.rope_pair_(two[:, :Hq * D].view(B, S, Hq, D), cos, sin, inverse=True)
    fa4b.rope_pair_(two[:, Hq * D:(Hq + Hkv) * D].view(B, S, Hkv, D), cos, sin, inverse=True)
    sep = fa4b.tk_quantize_for_gemm(two, return_transpose=True, encode_centric=False)
    Q.check_status()
    assert float(fused[5]) == float(sep[5]) and float(fused[4]) == float(sep[4])
    for i, what in ((0, "row codes"), (1, "row scale pages"), (2, "transposed codes"), (3, "transposed scale pages")):
        assert torch.equal(fused[i], sep[i]), what
    # a slab of the transposed plane decodes to the transpose of the same slab of the row plane's source, block for block
    rows = fa4b.dequant_nvfp4(fused[0][:256].contiguous(), fused[1][:2].contiguous(), fused[4])          # [256, N]
    cols = fa4b.dequant_nvfp4(fused[2][:, :128].contiguous(), fused[3][:, :4].contiguous(), fused[4])    # [N, 256]
    ref = two[:256].float()
    assert O.rel_l2(ref.cpu(), rows.float().cpu()) < 0.12 and O.rel_l2(ref.t().cpu(), cols.float().cpu()) < 0.12


def test_pack_qkv_grads_rejects_bad_layouts():
    cos, sin = (t.to(DEV) for t in O.rope_tables(128, 128))
    dq = torch.zeros(1, 128, 2, 128, dtype=torch.bfloat16, device=DEV)
    dkv = torch.zeros(1, 128, 1, 128, dtype=torch.bfloat16, device=DEV)
    with pytest.raises(ValueError):
        fa4b.pack_qkv_grads(dq.permute(0, 2, 1, 3), dkv, dkv, cos, sin)            # head-major view
    with pytest.raises(ValueError):
        fa4b.pack_qkv_grads(dq, dkv, dkv, cos[:64].contiguous(), sin)                # table of another length
    with pytest.raises(ValueError):
        fa4b.pack_qkv_grads(dq[:, :64], dkv[:, :64], dkv[:, :64], cos[:64].contiguous(), sin[:64].contiguous())  # 64 tokens


@pytest.mark.parametrize("shape,seed", [((128, 128), 11), ((256, 512), 12)])
def test_nvfp4_encode_centric_recipe_matches_its_restatement(shape, seed):
    # the TK quantiser's default recipe; its oracle is pinned by hand-worked known answers (tests/test_oracle_pins.py)
    x, gamma = O.make_quantizer_inputs(*shape, seed=seed)
    x[3, 16:32] = 0.0            # an all-zero block: multiplier 448, stored scale E4M3(1/448)
    x[7, :16] *= 1.0e-4          # a tiny block: the multiplier saturates at 448
    fp4_row, sc_row, fp4_col, sc_col, sg, am = fa4b.tk_quantize_for_gemm(x.to(DEV), return_transpose=True, encode_centric=True)
    ref, ref_t = O.nvfp4_quantize_encode_centric(x), O.nvfp4_quantize_encode_centric(x.t().contiguous())
    assert float(sg) == float(ref.global_scale)
    _same(fp4_row, ref.codes, "row codes")
    _same(sc_row, ref.pages(), "row scale pages")
    _same(fp4_col, ref_t.codes, "transposed codes")
    _same(sc_col, ref_t.pages(), "transposed scale pages")
    # fused with the RMSNorm
    out = fa4b.tk_fused_norm_quantize(x.to(DEV), gamma.to(DEV), 1e-6, return_transpose=False, return_normalized=True, encode_centric=True)
    y = out[-1].cpu()
    ref_y = O.nvfp4_quantize_encode_centric(y)
    _same(out[0], ref_y.codes, "fused row codes")
    _same(out[1], ref_y.pages(), "fused row scale pages")
    # a zero tensor keeps the recipe's E4M3(1/448) scale bytes and zero codes
    z = fa4b.tk_quantize_for_gemm(torch.zeros(128, 128, dtype=torch.bfloat16, device=DEV), return_transpose=False, encode_centric=True)
    assert int(z[0].max()) == 0 and z[1].unique().tolist() == [1] and float(z[4]) == 0.0


def test_nvfp4_encode_centric_kernel_on_the_blocks_worked_by_hand():
    """The known-answer blocks of tests/test_oracle_pins.py (worked from core.cuh:47-60, 103-113 and
    fused_amax_quantize.cuh:235-256 of the reference) through the kernel: scale bytes and codes as computed by hand,
    row-wise and in the transposed output."""
    x = torch.zeros(128, 128)
    x[0, :16] = torch.tensor([6, -3, 1.5, 0.75, 0.25, 1.25, 1.75, 2.5, 3.5, 5, -0.75, -5, 0, 0.5, 2, 4])
    x[0, 16:32] = torch.tensor([2688, 1024, 512, -2688] + [0] * 12)
    x[0, 48:64] = torch.tensor([2.0 ** -10, -(2.0 ** -10), 2.0 ** -12] + [0] * 13)
    x[1, :16] = torch.tensor([3, 0.375, 0.125, -0.375] + [0] * 12)
    x[1, 16:32] = torch.tensor([5, 4, 1, 2, -4] + [0] * 11)
    xb = x.bfloat16()
    fp4_row, sc_row, fp4_col, sc_col, sg, am = fa4b.tk_quantize_for_gemm(xb.to(DEV), True, True)  # the reference's positional call
    assert float(am) == 2688.0 and float(sg) == 1.0
    codes = O.unpack_nibbles(fp4_row.cpu())
    assert codes[0, :16].tolist() == [7, 13, 3, 2, 0, 2, 4, 4, 6, 6, 10, 14, 0, 1, 4, 6]
    assert codes[0, 16:32].tolist() == [7, 4, 2, 15] + [0] * 12 and codes[0, 48:64].tolist() == [1, 9, 0] + [0] * 13
    assert codes[1, :16].tolist() == [7, 2, 0, 10] + [0] * 12 and codes[1, 16:32].tolist() == [7, 6, 2, 4, 14] + [0] * 11
    scales = O.pages_to_scales(sc_row.cpu())
    assert scales[0, :4].tolist() == [0x38, 0x7E, 0x01, 0x01] and scales[1, :4].tolist() == [0x30, 0x35, 0x01, 0x01]
    assert scales[2:].unique().tolist() == [0x01]  # all-zero blocks: E4M3(1 / 448)
    ref_t = O.nvfp4_quantize_encode_centric(xb.t().contiguous())
    _same(fp4_col, ref_t.codes, "transposed codes")
    _same(sc_col, ref_t.pages(), "transposed scale pages")


def _wide_range(M, K, seed, lo=-20, hi=20):
    """rows of very different magnitude: small rows get scale byte 0 (step clamped to FLT_MIN), where x / step
    overflows and only the sign and saturation survive; mid rows land in the subnormal E4M3 scale range"""
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(M, K, generator=g) * torch.exp2(torch.randint(lo, hi, (M, 1), generator=g).float())
    return x.bfloat16()


@pytest.mark.parametrize("seed,lo,hi", [(31, -20, 20), (32, -40, 0), (33, -4, 12)])
def test_nvfp4_wide_dynamic_range_matches_oracle(seed, lo, hi):
    x = _wide_range(512, 512, seed, lo, hi)
    fp4_row, sc_row, fp4_col, sc_col, sg, _ = fa4b.tk_quantize_for_gemm(x.to(DEV), return_transpose=True, encode_centric=False)
    ref, ref_t = O.nvfp4_quantize(x), O.nvfp4_quantize_transposed(x)
    assert float(sg) == float(ref.global_scale)
    _same(fp4_row, ref.codes, "row codes")
    _same(sc_row, ref.pages(), "row scale pages")
    _same(fp4_col, ref_t.codes, "transposed codes")
    _same(sc_col, ref_t.pages(), "transposed scale pages")


def test_nvfp4_supplied_amax_far_below_the_data_saturates_like_the_oracle():
    x = _wide_range(256, 256, 34, 0, 10)
    tiny = torch.tensor([2.0 ** -20], dtype=torch.float32)
    fp4_row, sc_row, _, _, sg, _ = fa4b.tk_quantize_for_gemm(x.to(DEV), return_transpose=False, amax_in=tiny.to(DEV), encode_centric=False)
    ref = O.nvfp4_quantize(x, amax=tiny)
    assert float(sg) == float(ref.global_scale)
    _same(fp4_row, ref.codes, "row codes")
    _same(sc_row, ref.pages(), "row scale pages")


def test_mxfp4_wide_dynamic_range_matches_oracle():
    x = _wide_range(256, 512, 35, -60, 60)
    for mode in ("ceil", "rte_mantissa", "floor"):
        fp4, sc = fa4b.mxfp4_quantize_for_gemm(x.to(DEV), mode=mode)
        ref = O.mxfp4_quantize(x, mode=mode)
        _same(fp4, ref.codes, f"codes ({mode})")
        _same(sc, ref.pages(), f"scale pages ({mode})")


@pytest.mark.parametrize("mode", ["ceil", "rte_mantissa", "floor"])
def test_mxfp4_matches_oracle(mode):
    x, _ = O.make_quantizer_inputs(256, 512, seed=11)
    x[5, 64:96] = 0
    x[6, :32] = torch.full((32,), 2.0 ** -100).bfloat16()
    fp4, sc = fa4b.mxfp4_quantize_for_gemm(x.to(DEV), mode)
    ref = O.mxfp4_quantize(x, mode)
    _same(fp4, ref.codes, "codes")
    _same(sc, ref.pages(), "E8M0 pages")
    assert torch.equal(fa4b.dequant_mxfp4(fp4, sc).cpu(), ref.dequant())


def test_fused_rmsnorm_nvfp4_matches_oracle():
    x, gamma = O.make_quantizer_inputs(256, 1024, seed=13)
    fp4_row, sc_row, fp4_col, sc_col, sg, inv_rms, am, y = fa4b.tk_fused_norm_quantize(
        x.to(DEV), gamma.to(DEV), 1e-6, return_transpose=True, return_normalized=True, encode_centric=False)
    _, inv_ref = O.rmsnorm_reference(x, gamma, 1e-6)
    # FP32 tree sum vs the oracle's FP64 mean: at most 2 ulp on inv_rms
    ulp = (inv_rms.cpu().view(torch.int32) - inv_ref.view(torch.int32)).abs().max().item()
    assert ulp <= 2, ulp
    ref = O.rmsnorm_nvfp4(x, gamma, 1e-6, inv_rms=inv_rms.cpu())
    _same(y.view(torch.int16), ref.y.view(torch.int16), "normalised bf16")
    assert float(am) == float(ref.amax) and float(sg) == float(ref.row.global_scale)
    _same(fp4_row, ref.row.codes, "row codes")
    _same(sc_row, ref.row.pages(), "row pages")
    _same(fp4_col, ref.col.codes, "col codes")
    _same(sc_col, ref.col.pages(), "col pages")


def test_full_size_quantizers_by_slabs_and_transpose_property():
    """16384 x 4096 (the benchmark shape): oracle on sampled 128-row slabs, and the
    transposed output must equal the row-wise output of the transposed input."""
    M, K = 16384, 4096
    x, gamma = O.make_quantizer_inputs(M, K, seed=20260825)
    xd = x.to(DEV)
    fp4_row, sc_row, fp4_col, sc_col, sg, am = fa4b.tk_quantize_for_gemm(xd, encode_centric=False)
    amax = am.cpu()
    for r0 in (0, 4096 + 128, M - 128):
        ref = O.nvfp4_quantize(x[r0:r0 + 128], amax=amax)
        _same(fp4_row[r0:r0 + 128], ref.codes, f"row codes slab {r0}")
        _same(sc_row[r0 // 128], ref.pages()[0], f"row pages slab {r0}")
    t_row, t_sc, _, _, _, _ = fa4b.tk_quantize_for_gemm(xd.t().contiguous(), return_transpose=False, encode_centric=False)
    _same(fp4_col, t_row, "transposed codes vs row-wise of x^T")
    _same(sc_col, t_sc, "transposed pages vs row-wise of x^T")
    fp4, sc = fa4b.mxfp4_quantize_for_gemm(xd)
    for r0 in (0, M - 128):
        ref = O.mxfp4_quantize(x[r0:r0 + 128])
        _same(fp4[r0:r0 + 128], ref.codes, f"mx codes slab {r0}")
        _same(sc[r0 // 128], ref.pages()[0], f"mx pages slab {r0}")
    out = fa4b.tk_fused_norm_quantize(xd, gamma.to(DEV), 1e-6, encode_centric=False)
    inv = out[5].cpu()
    r0 = 8192
    y = O.rmsnorm_apply(x[r0:r0 + 128], gamma, inv[r0:r0 + 128])
    ref = O.nvfp4_quantize(y, amax=out[6].cpu())
    _same(out[0][r0:r0 + 128], ref.codes, "fused row codes slab")
    _same(out[1][r0 // 128], ref.pages()[0], "fused row pages slab")
    assert fa4b.amax(xd).item() == float(x.float().abs().amax())


@pytest.mark.parametrize("M,K", [(256, 1024), (384, 2048), (128, 4096)])
def test_rmsnorm_backward_matches_fp32_reference(M, K):
    """dx and dgamma of the fused RMSNorm (FP32 arithmetic, bf16 results): agreement to bf16 rounding with the
    CPU restatement; the forward's inv_rms is the saved statistic."""
    x, gamma = O.make_quantizer_inputs(M, K, seed=40 + M)
    g = torch.Generator().manual_seed(M + K)
    dy = (torch.randn(M, K, generator=g) * 0.1).bfloat16()
    out = fa4b.tk_fused_norm_quantize(x.to(DEV), gamma.to(DEV), 1e-6, return_transpose=False, encode_centric=False)
    inv_rms = out[5]
    want_dx, want_dg = O.rmsnorm_backward_reference(x, gamma, inv_rms.cpu(), dy)
    dx, dgamma = fa4b.rmsnorm_backward_bf16(x.to(DEV), gamma.to(DEV), inv_rms, dy.to(DEV))
    assert O.rel_l2(want_dx, dx.cpu()) < 3e-3      # one bf16 rounding each side: 2^-9 / sqrt(3) per element at most
    assert (want_dx.float() - dx.cpu().float()).abs().max() <= 2.0 ** -7 * want_dx.float().abs().max()
    assert O.rel_l2(want_dg, dgamma.cpu()) < 3e-3
    with pytest.raises(Exception):
        fa4b.rmsnorm_backward_bf16(x.to(DEV), gamma.to(DEV)[:-8], inv_rms, dy.to(DEV))

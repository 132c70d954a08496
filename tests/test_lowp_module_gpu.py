"""Module-level forward (hidden states in, hidden states out) against the oracle's composition of the same steps."""

import pytest
import torch

import fa4b
import fa4b_oracle as O
from fa4b.lowp_module import LowpFA4Attention, LowpFA4AttentionBlock, pair_interleave_qk_rows, replace_attention_modules

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _block_inputs(B, S, hidden, Hq, Hkv, D, seed):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(B, S, hidden, generator=g).bfloat16()
    mk = lambda r, c: (torch.randn(r, c, generator=g) / c ** 0.5).bfloat16()
    wq, wk, wv, wo = mk(Hq * D, hidden), mk(Hkv * D, hidden), mk(Hkv * D, hidden), mk(hidden, Hq * D)
    cos, sin = O.rope_tables(S, D)
    return x, wq, wk, wv, wo, cos, sin


def test_module_forward_matches_oracle_composition():
    B, S, hidden, Hq, Hkv, D = 1, 256, 512, 4, 2, 128
    x, wq, wk, wv, wo, cos, sin = _block_inputs(B, S, hidden, Hq, Hkv, D, seed=21)
    blk = LowpFA4AttentionBlock(wq.to(DEV), wk.to(DEV), wv.to(DEV), wo.to(DEV), Hq, Hkv, D)
    y, mid = blk.forward(x.to(DEV), cos.to(DEV), sin.to(DEV), return_intermediates=True)
    ref_y, ref_qkv, ref_o = O.lowp_attention_block_reference(x, wq, wk, wv, wo, cos, sin, Hq, Hkv, D)
    assert y.shape == (B, S, hidden) and y.dtype == torch.bfloat16
    # projections: FP32 sums on the tensor core against float64 sums (rel-L2 1e-4); a bf16 value that lands on
    # the other side of a rounding boundary can move an FP4 code downstream, hence the wider bounds after it
    v_cols = slice((Hq + Hkv) * D, (Hq + 2 * Hkv) * D)  # the q and k columns of the buffer have been rotated in place
    assert O.rel_l2(ref_qkv[:, v_cols].float(), mid["qkv"][:, v_cols].float().cpu()) < 1e-4
    assert O.rel_l2(ref_o.float(), mid["o"].float().cpu()) < 1e-2
    assert O.rel_l2(ref_y.float(), y.float().cpu()) < 2e-2


def test_module_forward_tracks_a_bf16_attention_block():
    # against plain bf16 / fp32 math the low-precision block stays within the error of its formats
    B, S, hidden, Hq, Hkv, D = 2, 256, 1024, 8, 2, 128
    x, wq, wk, wv, wo, cos, sin = _block_inputs(B, S, hidden, Hq, Hkv, D, seed=22)
    blk = LowpFA4AttentionBlock(wq.to(DEV), wk.to(DEV), wv.to(DEV), wo.to(DEV), Hq, Hkv, D)
    y = blk(x.to(DEV), cos.to(DEV), sin.to(DEV))
    rows = x.float().reshape(B * S, hidden)
    q = (rows @ wq.float().t()).bfloat16().reshape(B, S, Hq, D)
    k = (rows @ wk.float().t()).bfloat16().reshape(B, S, Hkv, D)
    v = (rows @ wv.float().t()).bfloat16().reshape(B, S, Hkv, D)
    q, k = O.rope_pair_reference(q, cos, sin), O.rope_pair_reference(k, cos, sin)
    o, _ = O.attn_reference_fp32(q.permute(0, 2, 1, 3), k.permute(0, 2, 1, 3), v.permute(0, 2, 1, 3))
    ref = (o.permute(0, 2, 1, 3).reshape(B * S, Hq * D).float() @ wo.float().t()).reshape(B, S, hidden)
    # two NVFP4 x NVFP4 projections and an FP4 score matmul on Gaussian data: the CPU oracle of the same block sits
    # at 0.29 from this reference
    assert O.rel_l2(ref, y.float().cpu()) < 0.4


def test_module_backward_matches_oracle_composition():
    B, S, hidden, Hq, Hkv, D = 1, 256, 512, 4, 2, 128
    x, wq, wk, wv, wo, cos, sin = _block_inputs(B, S, hidden, Hq, Hkv, D, seed=31)
    dy = (torch.randn(B, S, hidden, generator=torch.Generator().manual_seed(32)) * 0.05).bfloat16()
    blk = LowpFA4AttentionBlock(wq.to(DEV), wk.to(DEV), wv.to(DEV), wo.to(DEV), Hq, Hkv, D)
    y, saved = blk.forward(x.to(DEV), cos.to(DEV), sin.to(DEV), return_intermediates=True)
    got = blk.backward(dy.to(DEV), saved, cos.to(DEV), sin.to(DEV))
    blk.check_status(saved["workspace"])  # the one host synchronisation of the step: six projection slots + attention
    want = O.lowp_attention_block_backward_reference(dy, x, wq, wk, wv, wo, cos, sin, Hq, Hkv, D)
    # Five chained low-precision GEMMs and the attention backward: a bf16 value on the other side of a rounding
    # boundary in one stage moves FP4 / FP8 codes in the next, so the bound is wider than a single kernel's
    # (tolerance: rel-L2 5e-2 per gradient; the single kernels are tested at 1e-4 / 2e-2 on their own)
    for name, g, w in zip(("dx", "dwq", "dwk", "dwv", "dwo"), got, want):
        assert g.shape == w.shape, name
        assert O.rel_l2(w.float(), g.float().cpu()) < 5e-2, name


def test_module_gradients_point_along_fp32_gradients():
    # cosine similarity against autograd through the same block in FP32 math
    B, S, hidden, Hq, Hkv, D = 1, 256, 512, 4, 2, 128
    x, wq, wk, wv, wo, cos, sin = _block_inputs(B, S, hidden, Hq, Hkv, D, seed=33)
    dy = (torch.randn(B, S, hidden, generator=torch.Generator().manual_seed(34)) * 0.05).bfloat16()
    blk = LowpFA4AttentionBlock(wq.to(DEV), wk.to(DEV), wv.to(DEV), wo.to(DEV), Hq, Hkv, D)
    y, saved = blk.forward(x.to(DEV), cos.to(DEV), sin.to(DEV), return_intermediates=True)
    got = blk.backward(dy.to(DEV), saved, cos.to(DEV), sin.to(DEV))
    xf, ws = x.float().requires_grad_(), [w.float().requires_grad_() for w in (wq, wk, wv, wo)]
    rows = xf.reshape(B * S, hidden)
    fc = torch.complex(cos.float(), sin.float())[None, :, None, :]
    rot = lambda t: torch.view_as_real(torch.view_as_complex(t.reshape(*t.shape[:-1], -1, 2)) * fc).flatten(3)
    q = rot((rows @ ws[0].t()).reshape(B, S, Hq, D)).permute(0, 2, 1, 3)
    k = rot((rows @ ws[1].t()).reshape(B, S, Hkv, D)).permute(0, 2, 1, 3).repeat_interleave(Hq // Hkv, dim=1)
    v = (rows @ ws[2].t()).reshape(B, S, Hkv, D).permute(0, 2, 1, 3).repeat_interleave(Hq // Hkv, dim=1)
    sc = (q @ k.transpose(-1, -2)) * D ** -0.5
    sc = sc.masked_fill(torch.ones(S, S, dtype=torch.bool).triu(1), float("-inf"))
    o = (torch.softmax(sc, -1) @ v).permute(0, 2, 1, 3).reshape(B * S, Hq * D)
    (o @ ws[3].t()).reshape(B, S, hidden).backward(dy.float())
    for name, g, w in zip(("dx", "dwq", "dwk", "dwv", "dwo"), got, (xf.grad, ws[0].grad, ws[1].grad, ws[2].grad, ws[3].grad)):
        cosine = torch.nn.functional.cosine_similarity(g.float().cpu().flatten(), w.flatten(), dim=0)
        assert float(cosine) > 0.85, (name, float(cosine))


def test_trainable_module_routes_autograd_through_the_block_and_requantises_after_an_update():
    B, S, hidden, Hq, Hkv, D = 1, 256, 512, 4, 2, 128
    x, wq, wk, wv, wo, cos, sin = _block_inputs(B, S, hidden, Hq, Hkv, D, seed=41)
    mod = LowpFA4Attention(hidden, Hq, Hkv, D, device=DEV)
    with torch.no_grad():
        for lin, w in ((mod.wq, wq), (mod.wk, wk), (mod.wv, wv), (mod.wo, wo)):
            lin.weight.copy_(w.to(DEV))
    xd = x.to(DEV).requires_grad_()
    freqs = (cos.to(DEV), sin.to(DEV))
    y = mod(xd, freqs)
    dy = (torch.randn(B, S, hidden, generator=torch.Generator().manual_seed(42)) * 0.05).bfloat16().to(DEV)
    y.backward(dy)
    blk = LowpFA4AttentionBlock(wq.to(DEV), wk.to(DEV), wv.to(DEV), wo.to(DEV), Hq, Hkv, D)
    y2, saved = blk.forward(x.to(DEV), *freqs, return_intermediates=True)
    want = blk.backward(dy, saved, *freqs)
    assert torch.equal(y, y2)
    for g, w in zip((xd.grad, mod.wq.weight.grad, mod.wk.weight.grad, mod.wv.weight.grad, mod.wo.weight.grad), want):
        assert torch.equal(g, w)
    # an in-place update of a weight invalidates the cached quantised operands
    first = mod._block
    with torch.no_grad():
        mod.wo.weight.mul_(0.5)
    y3 = mod(x.to(DEV), freqs)
    assert mod._block is not first
    assert O.rel_l2(0.5 * y.detach().float().cpu(), y3.detach().float().cpu()) < 2e-2
    with pytest.raises(ValueError):
        mod(x.to(DEV), freqs, attention_masks=object())


def test_fused_qkv_publication_writes_the_same_operands_as_the_three_passes():
    from fa4b import attention

    B, S, hidden, Hq, Hkv, D = 2, 256, 512, 4, 2, 128
    x, wq, wk, wv, wo, cos, sin = _block_inputs(B, S, hidden, Hq, Hkv, D, seed=61)
    cos, sin = cos.to(DEV), sin.to(DEV)
    rows = x.to(DEV).reshape(B * S, hidden)
    a_codes, a_pages, _, _, a_g, _ = fa4b.tk_quantize_for_gemm(rows, return_transpose=False, encode_centric=False)
    weight = fa4b.prepare_nvfp4_projection_weight(torch.cat((wq, wk, wv), 0).contiguous().to(DEV))
    # three passes: projection, rotation, publication at a unit global scale
    qkv = fa4b.project_nvfp4((a_codes, a_pages, a_g), weight)
    q = qkv[:, :Hq * D].view(B, S, Hq, D)
    k = qkv[:, Hq * D:(Hq + Hkv) * D].view(B, S, Hkv, D)
    v = qkv[:, (Hq + Hkv) * D:].view(B, S, Hkv, D)
    fa4b.rope_pair_(q, cos, sin)
    fa4b.rope_pair_(k, cos, sin)
    qh, kh, vh = (t.permute(0, 2, 1, 3) for t in (q, k, v))
    o_ref, lse_ref, ws_ref = attention.attn_forward(qh, kh, vh, global_scale="one")
    # one pass
    ws = attention.alloc_workspace(attention.make_dims(qh, kh, None, "e4m3_fp8", global_scale="one"), DEV)
    ws.buf.zero_()
    fa4b.project_qkv_publish((a_codes, a_pages, a_g), weight, cos, sin, ws)
    got, want = ws.operands(), ws_ref.operands()
    for name in ("q_codes", "q_scales", "q_global", "k_codes", "k_scales", "k_global", "v_fp8", "q_fp8", "k_fp8"):
        if name in want:
            assert torch.equal(got[name].view(torch.uint8), want[name].view(torch.uint8)), name
    o, lse = attention.attn_forward_prepared(ws)
    assert torch.equal(o, o_ref) and torch.equal(lse, lse_ref)


def test_fused_dout_publication_writes_the_same_statistics_as_the_two_passes():
    from fa4b import attention

    B, S, hidden, Hq, Hkv, D = 2, 256, 512, 4, 2, 128
    x, wq, wk, wv, wo, cos, sin = _block_inputs(B, S, hidden, Hq, Hkv, D, seed=81)
    blk = LowpFA4AttentionBlock(wq.to(DEV), wk.to(DEV), wv.to(DEV), wo.to(DEV), Hq, Hkv, D)
    y, saved = blk.forward(x.to(DEV), cos.to(DEV), sin.to(DEV), return_intermediates=True)
    dy = (torch.randn(B * S, hidden, generator=torch.Generator().manual_seed(82)) * 0.05).bfloat16().to(DEV)
    g_r, g_p, _, _, g_g, _ = fa4b.tk_quantize_for_gemm(dy, return_transpose=False, encode_centric=False)
    o_rows, lse, ws = saved["o"], saved["lse"], saved["workspace"]
    # two passes
    do_rows = fa4b.project_nvfp4((g_r, g_p, g_g), blk.w_o_t)
    attention.attn_bwd_preprocess(o_rows.view(B, S, Hq, D).permute(0, 2, 1, 3), lse, do_rows.view(B, S, Hq, D).permute(0, 2, 1, 3), ws)
    want = {k: v.clone() for k, v in ws.operands().items() if k in ("do_fp8", "dstat", "lstat")}
    for k in want:
        ws.operands()[k].view(torch.uint8).zero_()
    # one pass
    fa4b.project_dout_publish((g_r, g_p, g_g), blk.w_o_t, o_rows, lse, ws)
    got = ws.operands()
    for k in want:
        assert torch.equal(got[k].view(torch.uint8), want[k].view(torch.uint8)), k


def test_module_with_fused_publication_matches_the_unfused_module_and_the_oracle():
    B, S, hidden, Hq, Hkv, D = 1, 256, 512, 4, 2, 128
    x, wq, wk, wv, wo, cos, sin = _block_inputs(B, S, hidden, Hq, Hkv, D, seed=71)
    dy = (torch.randn(B, S, hidden, generator=torch.Generator().manual_seed(72)) * 0.05).bfloat16()
    w = [t.to(DEV) for t in (wq, wk, wv, wo)]
    fused = LowpFA4AttentionBlock(*w, Hq, Hkv, D, fused_publish=True)
    plain = LowpFA4AttentionBlock(*w, Hq, Hkv, D, global_scale="one")
    yf, sf = fused.forward(x.to(DEV), cos.to(DEV), sin.to(DEV), return_intermediates=True)
    yp, sp = plain.forward(x.to(DEV), cos.to(DEV), sin.to(DEV), return_intermediates=True)
    assert torch.equal(yf, yp) and torch.equal(sf["lse"], sp["lse"]) and sf["qkv"] is None
    gf = fused.backward(dy.to(DEV), sf, cos.to(DEV), sin.to(DEV))
    gp = plain.backward(dy.to(DEV), sp, cos.to(DEV), sin.to(DEV))
    for a, b in zip(gf, gp):
        assert torch.equal(a, b)
    ref_y, _, _ = O.lowp_attention_block_reference(x, wq, wk, wv, wo, cos, sin, Hq, Hkv, D, global_scale="one")
    assert O.rel_l2(ref_y.float(), yf.float().cpu()) < 2e-2
    want = O.lowp_attention_block_backward_reference(dy, x, wq, wk, wv, wo, cos, sin, Hq, Hkv, D, global_scale="one")
    for name, g, r in zip(("dx", "dwq", "dwk", "dwv", "dwo"), gf, want):
        assert O.rel_l2(r.float(), g.float().cpu()) < 5e-2, name
    with pytest.raises(ValueError):
        LowpFA4AttentionBlock(*w, Hq, Hkv, D, fused_publish=True, global_scale="amax_per_bh")


class _TitanAttention(torch.nn.Module):
    """TorchTitan's Llama attention in a few lines: complex-pair rotation, repeated KV, causal softmax attention."""

    def __init__(self, hidden, n_heads, n_kv_heads, head_dim):
        super().__init__()
        self.n_heads, self.n_kv_heads, self.head_dim = n_heads, n_kv_heads, head_dim
        mk = lambda i, o: torch.nn.Linear(i, o, bias=False, device=DEV, dtype=torch.bfloat16)
        self.wq, self.wk, self.wv = mk(hidden, n_heads * head_dim), mk(hidden, n_kv_heads * head_dim), mk(hidden, n_kv_heads * head_dim)
        self.wo = mk(n_heads * head_dim, hidden)

    def forward(self, x, freqs_cis, attention_masks=None):
        B, S, _ = x.shape
        q = self.wq(x).view(B, S, self.n_heads, self.head_dim)
        k = self.wk(x).view(B, S, self.n_kv_heads, self.head_dim)
        v = self.wv(x).view(B, S, self.n_kv_heads, self.head_dim)
        rot = lambda t: torch.view_as_real(torch.view_as_complex(t.float().reshape(*t.shape[:-1], -1, 2)) * freqs_cis[None, :S, None, :]).flatten(3).type_as(t)
        q, k = rot(q), rot(k)
        rep = self.n_heads // self.n_kv_heads
        o = torch.nn.functional.scaled_dot_product_attention(q.transpose(1, 2), k.transpose(1, 2).repeat_interleave(rep, 1),
                                                             v.transpose(1, 2).repeat_interleave(rep, 1), is_causal=True)
        return self.wo(o.transpose(1, 2).reshape(B, S, -1))


def test_replaced_module_follows_the_bf16_module_it_replaces_and_trains():
    torch.manual_seed(51)
    hidden, Hq, Hkv, D, B, S = 512, 4, 2, 128, 2, 256
    model = torch.nn.ModuleDict({"attention": _TitanAttention(hidden, Hq, Hkv, D)})
    inv = 1.0 / (500000.0 ** (torch.arange(0, D, 2, device=DEV, dtype=torch.float32) / D))
    ang = torch.arange(2 * S, device=DEV, dtype=torch.float32)[:, None] * inv[None, :]
    freqs_cis = torch.polar(torch.ones_like(ang), ang)  # longer than the sequence, as TorchTitan's table is
    x = torch.randn(B, S, hidden, device=DEV).bfloat16()
    want = model["attention"](x, freqs_cis)
    assert replace_attention_modules(model) == 1
    got = model["attention"](x, freqs_cis, None)
    cosine = torch.nn.functional.cosine_similarity(got.float().flatten(), want.float().flatten(), dim=0)
    assert float(cosine) > 0.93, float(cosine)
    # one SGD step through the low-precision backward lowers a regression loss on this batch
    target = torch.randn_like(want)
    opt = torch.optim.SGD(model.parameters(), lr=0.05)
    losses = []
    for _ in range(3):
        opt.zero_grad()
        loss = (model["attention"](x, freqs_cis, None).float() - target.float()).pow(2).mean()
        loss.backward()
        opt.step()
        losses.append(float(loss))
    assert losses[2] < losses[0], losses


def test_pair_interleave_keeps_scores():
    Hq, D, hidden = 2, 8, 16
    g = torch.Generator().manual_seed(5)
    w = torch.randn(Hq * D, hidden, generator=g)
    wi = pair_interleave_qk_rows(w, Hq, D)
    assert torch.equal(wi[0], w[0]) and torch.equal(wi[1], w[D // 2]) and torch.equal(wi[2], w[1])
    a, b = torch.randn(3, hidden, generator=g), torch.randn(3, hidden, generator=g)
    s0 = (a @ w.t()).reshape(3, Hq, D) @ (b @ w.t()).reshape(3, Hq, D).transpose(1, 2)
    s1 = (a @ wi.t()).reshape(3, Hq, D) @ (b @ wi.t()).reshape(3, Hq, D).transpose(1, 2)
    assert torch.allclose(s0, s1, atol=1e-4)


def test_module_rejects_masks_and_bad_shapes():
    B, S, hidden, Hq, Hkv, D = 1, 128, 512, 4, 2, 128
    x, wq, wk, wv, wo, cos, sin = _block_inputs(B, S, hidden, Hq, Hkv, D, seed=23)
    blk = LowpFA4AttentionBlock(wq.to(DEV), wk.to(DEV), wv.to(DEV), wo.to(DEV), Hq, Hkv, D)
    with pytest.raises(ValueError):
        blk.forward(x.to(DEV), cos.to(DEV), sin.to(DEV), attention_masks=object())
    with pytest.raises(ValueError):
        blk.forward(x.to(DEV)[:, :100], cos.to(DEV), sin.to(DEV))
    with pytest.raises(ValueError):
        LowpFA4AttentionBlock(wq.to(DEV), wk.to(DEV), wv.to(DEV), wo.to(DEV), Hq, 3, D)

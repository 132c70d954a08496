"""Generate the golden fixtures in this folder from the reference's own Python.

Run in a container that has the reference checkout (it is imported, never
copied):

    python tests/golden/make_golden.py /path/to/reference

Outputs (small, committed): ``quantizers.npz`` and ``backward_s128.npz``.
The parity tests only read the ``.npz`` files; they never import the
reference.  BF16 / FP8 tensors are stored as raw integer bit patterns.
"""

from __future__ import annotations

import pathlib
import os
import sys

import numpy as np
import torch


def bits16(t):
    return t.contiguous().view(torch.int16).numpy()


def bits8(t):
    return t.contiguous().view(torch.uint8).numpy()


def main(ref_root: str) -> None:
    sys.path.insert(0, ref_root)
    sys.dont_write_bytecode = True
    import tk_fa4.lowp_fa4_bwd.projection_quantization_reference as R
    import tk_fa4.lowp_fa4_bwd.validate_native_tk_d128_backward as V

    out = pathlib.Path(__file__).resolve().parent
    g = torch.Generator().manual_seed(20260825)
    x = torch.randn(128, 256, generator=g)
    x[:, 7] *= 20.0  # an outlier channel
    x[5, 32:64] = 0.0  # all-zero blocks
    x[9, :16] = torch.tensor([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0, 6.0] * 2) * 0.5
    x = x.bfloat16()

    fx = {"x": bits16(x)}
    stock = R.fake_quantize_nvfp4(x, block_shape=(1, 16))
    fx["nvfp4_stock_values"] = bits16(stock.values)
    # every reference CUDA producer rounds payloads nearest-even; the
    # reference's own RNE routine replaces the bucketize step for that variant
    saved = R._quantize_e2m1
    R._quantize_e2m1 = R._quantize_e2m1_rne
    try:
        rne = R.fake_quantize_nvfp4(x, block_shape=(1, 16))
        rne_t = R.fake_quantize_nvfp4(x.t().contiguous(), block_shape=(1, 16))
        mx = {m: R.fake_quantize_mxfp4(x, block_shape=(1, 32), scale_mode=m) for m in ("ceil", "rte")}
        w2d = R.fake_quantize_nvfp4(x, block_shape=(16, 16))
    finally:
        R._quantize_e2m1 = saved
    fx["nvfp4_values"] = bits16(rne.values)
    fx["nvfp4_block_scales"] = rne.block_scales.reshape(128, 16).numpy()
    fx["nvfp4_global_decode"] = np.float32(rne.diagnostics["global_decode"])
    fx["nvfp4_t_values"] = bits16(rne_t.values)
    fx["nvfp4_t_block_scales"] = rne_t.block_scales.reshape(256, 8).numpy()
    # learned-weight recipe: one scale per 16x16 tile; and the reference's byte-level transposition of a
    # prepared operand (built here from the represented values and scales the reference itself returned)
    fx["nvfp4_w2d_values"] = bits16(w2d.values)
    fx["nvfp4_w2d_block_scales"] = w2d.block_scales.reshape(8, 16).numpy()
    gd = torch.tensor(w2d.diagnostics["global_decode"], dtype=torch.float32)
    sc = w2d.block_scales.reshape(8, 16).to(torch.float8_e4m3fn)  # exact: the values are E4M3 numbers
    dec = sc.float().repeat_interleave(16, 0).repeat_interleave(16, 1) * gd
    mag = (w2d.values.float().abs() / dec.clamp_min(1e-30))
    lv = torch.tensor(R.E2M1_LEVELS)
    code = (mag[..., None] - lv).abs().argmin(-1).to(torch.uint8) | (torch.signbit(w2d.values).to(torch.uint8) << 3)
    payload = (code[:, 0::2] | (code[:, 1::2] << 4)).contiguous()
    rows, cols = x.shape
    rr = torch.arange(rows)[:, None]
    gg = torch.arange(cols // 16)[None, :]
    pages = torch.zeros(rows // 128, cols // 64, 512, dtype=torch.uint8)
    pages[rr // 128, gg // 4, (rr % 32) * 16 + ((rr % 128) // 32) * 4 + gg % 4] = sc.view(torch.uint8).repeat_interleave(16, 0)
    tp, ts, _ = R.transpose_prepared_nvfp4_weight_reference((payload, pages, gd.reshape(1)))
    fx["nvfp4_w2d_payload"] = payload.numpy()
    fx["nvfp4_w2d_pages"] = pages.numpy()
    fx["nvfp4_w2d_t_payload"] = tp.numpy()
    fx["nvfp4_w2d_t_pages"] = ts.numpy()
    for m, r in mx.items():
        fx[f"mxfp4_{m}_values"] = bits16(r.values)
        fx[f"mxfp4_{m}_block_scales"] = r.block_scales.reshape(128, 8).numpy()
    v = torch.randn(1, 64, 2, 32, generator=g).bfloat16()  # [B,S,H,D]
    rv = R.fake_quantize_mxfp4_v_1d(v)
    fx["v"] = bits16(v)
    fx["v_values"] = bits16(rv.values)
    fx["v_block_scales"] = rv.block_scales.numpy()
    mid = torch.tensor((0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0))
    fx["e2m1_midpoints"] = mid.numpy()
    fx["e2m1_midpoints_rne"] = R._quantize_e2m1_rne(mid).numpy()
    np.savez_compressed(out / "quantizers.npz", **fx)

    # represented-operand FP32 backward at S=128 (one kv head, its 4 query heads)
    st = V.make_represented_state(V.Shape(batch=1, sequence=128), device="cpu", seed=20260829)
    gr = V.represented_e4m3_causal_reference(st)
    np.savez_compressed(
        out / "backward_s128.npz",
        q=bits8(st.q[:, :, :4]), k=bits8(st.k[:, :, :1]), v=bits8(st.v[:, :, :1]),
        dout=bits8(st.dout[:, :, :4]),
        lstat=st.lstat[:, :4].numpy(), dstat=st.dstat[:, :4].numpy(),
        dq=gr.dq[:, :, :4].numpy().astype(np.float32),
        dk=gr.dk[:, :, :1].numpy().astype(np.float32),
        dv=gr.dv[:, :, :1].numpy().astype(np.float32),
        softmax_scale=np.float32(V.SOFTMAX_SCALE),
    )
    print("wrote", sorted(p.name for p in out.glob("*.npz")))


if __name__ == "__main__":
    main(sys.argv[1] if len(sys.argv) > 1 else os.environ.get("FA4_REFERENCE_ROOT", "reference"))

"""fa4b: B200 (sm_100a) low-precision attention path -- NVFP4 Q.K^T with
FP8-E4M3 P.V (MXFP4 P/V as a diagnostic route), forward and backward, and the
NVFP4 / MXFP4 block quantizers that feed it.  Host side of the C ABI in
include/fa4b.h; every operator runs hand-written CUDA and raises if the
library is missing."""

from . import _lib, parallel  # noqa: F401
from .quantizers import (  # noqa: F401
    amax,
    dequant_mxfp4,
    dequant_nvfp4,
    mxfp4_quantize_for_gemm,
    prepare_nvfp4_projection_weight,
    project_nvfp4,
    project_qkv_publish,
    project_dout_publish,
    rope_pair_,
    pack_qkv_grads,
    prepare_nvfp4_projection_weight_dual,
    rmsnorm_backward_bf16,
    tk_fused_norm_quantize,
    tk_quantize_for_gemm,
)

__all__ = [
    "amax", "dequant_mxfp4", "dequant_nvfp4", "mxfp4_quantize_for_gemm", "prepare_nvfp4_projection_weight", "project_nvfp4", "project_qkv_publish", "project_dout_publish", "rope_pair_", "pack_qkv_grads", "prepare_nvfp4_projection_weight_dual", "rmsnorm_backward_bf16", "tk_fused_norm_quantize",
    "tk_quantize_for_gemm",
]

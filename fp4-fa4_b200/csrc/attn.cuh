// Declarations shared by the attention sources: dimension checks, the layout of the
// operand cache (workspace), kernel launchers.
#pragma once
#include "common.cuh"
#include "tc_sm100.cuh"

namespace fa4b {

constexpr int kTileQ = 128;
constexpr int kTileKV = 128;
constexpr float kLog2e = 1.4426950408889634f;
constexpr float kLn2 = 0.6931471805599453f;
constexpr float kPLift = 8.0f;  // probabilities are represented times 2^8

inline size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

inline int check_dims(const fa4b_attn_dims& d) {
  FA4B_REQUIRE(d.B > 0 && d.Hq > 0 && d.Hkv > 0 && d.S > 0, FA4B_BAD_SHAPE, "B, Hq, Hkv and S must be positive");
  FA4B_REQUIRE(d.D == 64 || d.D == 128, FA4B_BAD_SHAPE, "head dim %d: only 64 and 128 are built", d.D);
  FA4B_REQUIRE(d.S % 128 == 0, FA4B_BAD_SHAPE, "S=%d must be a multiple of 128", d.S);
  FA4B_REQUIRE(d.Hq % d.Hkv == 0, FA4B_BAD_SHAPE, "Hq=%d must be a multiple of Hkv=%d", d.Hq, d.Hkv);
  FA4B_REQUIRE(d.pv_format == FA4B_PV_FP8_E4M3 || d.pv_format == FA4B_PV_MXFP4_E8M0, FA4B_UNSUPPORTED, "unknown pv_format %d",
               d.pv_format);
  FA4B_REQUIRE(d.mask == FA4B_MASK_CAUSAL || d.mask == FA4B_MASK_NONE, FA4B_UNSUPPORTED, "unknown mask %d", d.mask);
  FA4B_REQUIRE(d.global_scale_mode == FA4B_GLOBAL_AMAX_PER_BH || d.global_scale_mode == FA4B_GLOBAL_ONE, FA4B_UNSUPPORTED,
               "unknown global_scale_mode %d", d.global_scale_mode);
  return FA4B_OK;
}

inline fa4b_attn_ws_layout make_ws_layout(const fa4b_attn_dims& d) {
  fa4b_attn_ws_layout l{};
  const size_t nq = (size_t)d.B * d.Hq, nk = (size_t)d.B * d.Hkv, S = d.S, D = d.D;
  size_t off = 0;
  auto take = [&](size_t bytes) {
    const size_t at = off;
    off = align_up(off + bytes, 1024);
    return at;
  };
  l.q_codes = take(nq * S * D / 2);
  l.q_scales = take(nq * (S / 128) * (D / 64) * 512);
  l.q_global = take(nq * 4);
  l.k_codes = take(nk * S * D / 2);
  l.k_scales = take(nk * (S / 128) * (D / 64) * 512);
  l.k_global = take(nk * 4);
  l.v_fp8 = take(nk * S * D);
  l.k_fp8 = take(nk * S * D);  // k_codes .. k_fp8 are one contiguous range: what a sequence-sharded run sends on
  l.q_fp8 = take(nq * S * D);
  l.do_fp8 = take(nq * S * D);
  l.dstat = take(nq * S * 4);
  l.lstat = take(nq * S * 4);
  l.dq_accum = take(nq * S * D * 4);
  l.amax_bits = take((nq + nk) * 4);
  l.status = take(64);
  l.total = off;
  return l;
}

// MXFP4 P.V route: the V section holds codes [B*Hkv, D, S/2] and then the E8M0 pages [B*Hkv, S/128, 512]
inline size_t v_mx_pages_offset(const fa4b_attn_dims& d) { return align_up((size_t)d.B * d.Hkv * d.D * d.S / 2, 1024); }

inline float resolve_scale(const fa4b_attn_dims& d) { return d.softmax_scale > 0.f ? d.softmax_scale : 1.0f / sqrtf((float)d.D); }

void fill_kernel_info(fa4b_info* out);
void fill_bwd_info(fa4b_info* out);

int launch_attn_prepare(const fa4b_attn_prepare_args& a, cudaStream_t st);
int launch_attn_fwd(const fa4b_attn_fwd_args& a, cudaStream_t st);
int launch_attn_bwd_preprocess(const fa4b_attn_bwd_args& a, cudaStream_t st);
int launch_attn_bwd(const fa4b_attn_bwd_args& a, cudaStream_t st);
int launch_attn_accumulate(float* acc, const void* part, int64_t n, void* out, cudaStream_t st);
int launch_attn_merge(float* o_acc, float* lse_acc, const void* o_part, const float* lse_part, int64_t n_rows, int D, void* o_out,
                      cudaStream_t st);

}  // namespace fa4b

// Declarations shared by the attention sources: dimension checks, the layout of the
// operand cache (workspace), kernel launchers.
#pragma once
#include "common.cuh"
#include <algorithm>

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

// The operand cache in two sections.  Saved: what the forward publishes and the backward replays (Q/K codes, scale
// pages and global scales, the E4M3 operands, the amax and status words) -- the bytes a training step keeps from
// forward to backward.  Transient: what only lives inside one backward call (E5M2 dO, the row statistics, the FP32
// accumulators); it may be a second buffer shared by every layer (fa4b_attn_bwd_args.scratch).
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
  l.amax_bits = take((nq + nk) * 4);
  l.status = take(64);
  l.saved_total = off;
  l.do_fp8 = take(nq * S * D);
  l.dstat = take(nq * S * 4);
  l.lstat = take(nq * S * 4);
  l.dq_accum = take(nq * S * D * 4);
  l.dkv_accum = take(2 * nk * S * D * 4);  // dK sums, then dV sums
  l.total = off;
  return l;
}

// ---- work list of the backward ------------------------------------------------------------------------------
// Per (batch, kv head): the key tiles in order, each one's L query tiles (L = n - kt under the causal mask, n
// otherwise) cut into ceil(L / chunk) parts of nearly equal length.
struct BwdItem {
  int kt, qt_lo, qt_hi, parts;
};
// sum over L = 1..m of ceil(L / chunk)
__host__ __device__ inline int bwd_items_upto(int m, int chunk) {
  const int a = m / chunk, r = m % chunk;
  return chunk * a * (a + 1) / 2 + r * (a + 1);
}
__host__ __device__ inline int bwd_items_per_head(int n_tiles, int chunk, bool causal) {
  return causal ? bwd_items_upto(n_tiles, chunk) : n_tiles * ((n_tiles + chunk - 1) / chunk);
}
__host__ __device__ inline BwdItem bwd_item_of(int idx, int n_tiles, int chunk, bool causal) {
  BwdItem it;
  int L, part, first;
  if (causal) {
    const int total = bwd_items_upto(n_tiles, chunk);
    int lo = 0, hi = n_tiles - 1;  // largest kt whose first item is at or before idx
    while (lo < hi) {
      const int mid = (lo + hi + 1) >> 1;
      if (total - bwd_items_upto(n_tiles - mid, chunk) <= idx) lo = mid; else hi = mid - 1;
    }
    it.kt = lo;
    part = idx - (total - bwd_items_upto(n_tiles - lo, chunk));
    L = n_tiles - lo;
    first = lo;
  } else {
    const int per_tile = (n_tiles + chunk - 1) / chunk;
    it.kt = idx / per_tile;
    part = idx % per_tile;
    L = n_tiles;
    first = 0;
  }
  it.parts = (L + chunk - 1) / chunk;
  it.qt_lo = first + (int)((long long)L * part / it.parts);
  it.qt_hi = first + (int)((long long)L * (part + 1) / it.parts);
  return it;
}
// Query tiles per work item.  A launch of many (batch, kv head) units needs no cut: in key-tile-major order the long
// key tiles start first and the short ones fill the tail (cutting costs 2 % there: more CTA set-ups, dK / dV through
// FP32 sums).  With fewer than about six CTAs per SM the tiles are cut so that the launch has about four items per
// SM (measured best of 3, 4, 6, 8 and 12 on launches of 2, 4 and 8 units at S = 8192), at least two query tiles each
// (a shorter item is mostly set-up).
inline int bwd_chunk(const fa4b_attn_dims& d, int n_sm) {
  const long long n = d.S / 128;
  const long long heads = (long long)d.B * d.Hkv;
  if (heads * n >= 6ll * n_sm) return (int)n;
  const long long units = heads * (d.mask == FA4B_MASK_CAUSAL ? n * (n + 1) / 2 : n * n);
  const long long want = (units + 4ll * n_sm - 1) / (4ll * n_sm);
  return (int)std::min<long long>(std::max<long long>(want, 2), n);
}

// (batch, kv head) units per launch group: as many as keep the group's FP32 dQ rows (Hq / Hkv query heads of S x D
// floats per unit) within 72 MB, a little over half of the 126 MB L2 -- four units at S = 8192, D = 128, four query
// heads per kv head.  The same count serves the f16 sums (half the bytes): eight units per group measured slower.
inline int bwd_head_group(const fa4b_attn_dims& d) {
  const long long per_unit = (long long)(d.Hq / d.Hkv) * d.S * d.D * 4;
  const long long fit = (72ll << 20) / per_unit;
  return (int)std::min<long long>(std::max<long long>(fit, 1), (long long)d.B * d.Hkv);
}

// Whether a backward call keeps its dQ sums as f16 (see BwdParams::dq_half) instead of FP32: when this one call forms
// the whole sum (no FA4B_BWD_KEEP_DQ_ACCUM / FA4B_BWD_SKIP_DQ_OUT) and the caller has not asked for FP32 sums.
inline bool bwd_dq_half(const fa4b_attn_dims&, int flags) {
  return !(flags & (FA4B_BWD_KEEP_DQ_ACCUM | FA4B_BWD_SKIP_DQ_OUT | FA4B_BWD_DQ_SUMS_FP32));
}

// base to which the layout's transient offsets apply: the caller's separate scratch buffer, or the workspace itself
inline uint8_t* transient_base(const fa4b_attn_bwd_args& a, const fa4b_attn_ws_layout& l) {
  return a.scratch ? static_cast<uint8_t*>(a.scratch) - l.saved_total : static_cast<uint8_t*>(a.ws);
}

// MXFP4 P.V route: the V section holds codes [B*Hkv, D, S/2] and then the E8M0 pages [B*Hkv, S/128, 512]
inline size_t v_mx_pages_offset(const fa4b_attn_dims& d) { return align_up((size_t)d.B * d.Hkv * d.D * d.S / 2, 1024); }

inline float resolve_scale(const fa4b_attn_dims& d) { return d.softmax_scale > 0.f ? d.softmax_scale : 1.0f / sqrtf((float)d.D); }

// device address of the library's built-in operand cache (fa4b_attn_fwd_static) on the current device
int static_ws_pointer(void** out);

void fill_kernel_info(fa4b_info* out);
void fill_bwd_info(fa4b_info* out);

// skip_q: publish K and V only (the forward kernel quantises Q itself); the amax words of Q are still taken
int launch_attn_prepare(const fa4b_attn_prepare_args& a, cudaStream_t st, bool skip_q = false);
int launch_attn_fwd(const fa4b_attn_fwd_args& a, cudaStream_t st);
// zero_dq: the launch also clears the dQ accumulator of the backward call it belongs to
int launch_attn_bwd_preprocess(const fa4b_attn_bwd_args& a, cudaStream_t st, bool zero_dq = false);
int launch_attn_bwd(const fa4b_attn_bwd_args& a, cudaStream_t st);
int launch_attn_accumulate(float* acc, const void* part, int64_t n, void* out, cudaStream_t st);
int launch_attn_merge(float* o_acc, float* lse_acc, const void* o_part, const float* lse_part, int64_t n_rows, int D, void* o_out,
                      cudaStream_t st);

}  // namespace fa4b

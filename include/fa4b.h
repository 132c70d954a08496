/*
 * fa4b -- C ABI of the B200 (sm_100a) low-precision attention path.
 *
 * Plain pointers and sizes only: every buffer is a CUDA device pointer owned
 * by the caller unless a comment says "host".  `stream` is a cudaStream_t
 * passed as void* (NULL = the legacy default stream).  Every entry point
 * returns an fa4b_status; on failure fa4b_last_error() (thread local) holds a
 * one-line reason.  Nothing here allocates device memory: scratch space is
 * passed in and sized by the *_workspace_bytes queries.
 *
 * Each entry point names the reference interface it stands in for
 * (paths are relative to the reference project's root).
 */
#ifndef FA4B_H_
#define FA4B_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define FA4B_ABI_VERSION 2

typedef enum fa4b_status {
  FA4B_OK = 0,
  FA4B_BAD_SHAPE = 1,   /* a dimension the kernels do not cover               */
  FA4B_BAD_ALIGN = 2,   /* pointer or stride not aligned as documented        */
  FA4B_UNSUPPORTED = 3, /* format / mode / device not supported               */
  FA4B_CUDA_ERROR = 4,  /* a CUDA runtime or driver call failed               */
  FA4B_TIMEOUT = 5,     /* a bounded device-side wait ran out                 */
  FA4B_BAD_ARG = 6      /* NULL where a buffer is required, overlap, ...      */
} fa4b_status;

const char* fa4b_status_string(int status);
const char* fa4b_last_error(void);

/* ---- formats and modes ------------------------------------------------- */
enum { FA4B_PV_FP8_E4M3 = 0, FA4B_PV_MXFP4_E8M0 = 1 };  /* fa4.exact_pv_format */
enum { FA4B_MASK_CAUSAL = 0, FA4B_MASK_NONE = 1 };
/* global (per batch and head) decode scale of the NVFP4 Q / K operands: amax / 2688 (the recipe of
 * fake_quantize_nvfp4, a statistics pass over Q and K first), or 1 (the reference's attention route,
 * projection_fp4_epilogue.cuh:1922,1942: block scale E4M3(block amax / 6), no statistics pass) */
enum { FA4B_GLOBAL_AMAX_PER_BH = 0, FA4B_GLOBAL_ONE = 1 };
enum { FA4B_MX_CEIL = 0, FA4B_MX_RTE_MANTISSA = 1, FA4B_MX_FLOOR = 2 };
/* NVFP4 block-scale recipe: decode-centric (the stored scale E4M3(bamax / 6 / g) is what is rounded; the
 * arithmetic of fake_quantize_nvfp4) or encode-centric (the multiplier E4M3(6 / (bamax * 2688 / amax)) is
 * rounded and the stored scale is E4M3 of its reciprocal: the default of tk_quantize_for_gemm,
 * TK_quantisation/nvfp4_v6/fused_amax_quantize.cuh:235-256) */
enum { FA4B_RECIPE_DECODE_CENTRIC = 0, FA4B_RECIPE_ENCODE_CENTRIC = 1 };
/* fa4b_attn_bwd flags: a sequence-sharded run folds several key shards into one query shard's dQ */
enum {
  FA4B_BWD_KEEP_DQ_ACCUM = 1 /* do not zero the accumulator first */,
  FA4B_BWD_SKIP_DQ_OUT = 2 /* do not convert it into dq */,
  FA4B_BWD_DQ_SUMS_FP32 = 4 /* keep the partial dQ sums in FP32 where the call would keep them as f16 pairs */
};
enum { FA4B_PREPARE_ALL = 0, FA4B_PREPARE_AMAX = 1, FA4B_PREPARE_QUANTIZE = 2 };
enum { FA4B_LAYOUT_BHSD = 0, FA4B_LAYOUT_BSHD = 1 };

/* ---- fa4b_query --------------------------------------------------------
 * Host only.  Replaces read_hao_direct_topology()
 * (tk_fa4/fp4_fa4_fwd/hao_direct_host.inc:149-261) and
 * native_tk_d128_backward_metadata()
 * (tk_fa4/native_gqa_tk_bwd/v509_*bshd.cu:446-522). */
typedef struct fa4b_info {
  int abi_version;
  int build_sm;            /* 100 (compiled for sm_100a)                      */
  int fwd_threads, fwd_smem_bytes, fwd_tmem_columns, fwd_kv_stages;
  int bwd_threads, bwd_smem_bytes, bwd_tmem_columns;
  int tile_q, tile_kv;     /* 128, 128                                        */
  int wait_limit;          /* wall-clock cap of every device-side wait, ms    */
} fa4b_info;
int fa4b_query(fa4b_info* out);

/* ---- fa4b_amax ----------------------------------------------------------
 * max |x| of n bf16 values -> amax[0] (f32).  Replaces
 * fused_amax_pipelined_kernel (TK_quantisation/nvfp4_v6/amax_pipelined.cuh:142). */
int fa4b_amax(const void* x_bf16, int64_t n, float* amax, void* stream);

/* ---- fa4b_quant_nvfp4 ---------------------------------------------------
 * Row-wise (1x16) and optionally transposed (16x1) NVFP4 of x[rows, cols]
 * bf16 (row stride ld elements).  Replaces tk_quantize_for_gemm /
 * tk_quantize_transpose (TK_quantisation/nvfp4_v6/tk_quantize.cu:3172-3177)
 * and quantize_nvfp4_projection_operand (tk_fa4/interface.py:991), with the
 * decode-centric arithmetic of projection_quantization_reference.py:456-470.
 *   amax         [1] f32: written unless amax_is_input != 0
 *   global_scale [1] f32: amax / 2688
 *   codes_row  [rows, cols/2] u8 (even column in the low nibble)
 *   scales_row [rows/128, cols/64, 512] E4M3 bytes; byte
 *              (r%32)*16 + ((r%128)/32)*4 + (kblock%4) of page (r/128, kblock/4)
 *   codes_col  [cols, rows/2], scales_col [cols/128, rows/64, 512]: optional
 * rows and cols must be multiples of 128. */
typedef struct fa4b_quant_nvfp4_args {
  const void* x;
  int64_t rows, cols, ld;
  float* amax;
  int amax_is_input;
  float* global_scale;
  uint8_t* codes_row;
  uint8_t* scales_row;
  uint8_t* codes_col;  /* NULL = no transposed output */
  uint8_t* scales_col;
  int recipe;          /* FA4B_RECIPE_* */
} fa4b_quant_nvfp4_args;
int fa4b_quant_nvfp4(const fa4b_quant_nvfp4_args* a, void* stream);

/* ---- fa4b_quant_check_status ----------------------------------------------
 * The NVFP4 quantizer kernels (fa4b_quant_nvfp4, fa4b_quant_nvfp4_weight,
 * fa4b_rmsnorm_quant_nvfp4, fa4b_pack_qkv_grads) wait for the TMA load of
 * their tile with a cycle limit; a wait that runs out is recorded in a status
 * word on the device instead of spinning.  This call synchronises the stream,
 * reads that word, clears it and returns FA4B_TIMEOUT if it was set (the
 * outputs of the affected call are then incomplete), FA4B_OK otherwise.  No
 * reference counterpart: the reference's quantizers spin without a limit
 * (TK_quantisation/nvfp4_v6/fused_amax_quantize.cuh:130-179). */
int fa4b_quant_check_status(void* stream);

/* ---- fa4b_quant_nvfp4_weight --------------------------------------------
 * The same outputs for a learned projection weight: one scale per 16 x 16
 * tile (the E4M3 byte of the tile's amax), stored once per 1 x 16 group of
 * the tile in either orientation, so that the transposed operand is the
 * byte-for-byte transpose of the row-wise one and both share global_scale.
 * Replaces quantize_nvfp4_projection_weight and
 * quantize_nvfp4_projection_weight_dual (tk_fa4/interface.py:1221-1313);
 * arithmetic of fake_quantize_nvfp4(block_shape=(16, 16)), layout of
 * transpose_prepared_nvfp4_weight_reference
 * (projection_quantization_reference.py:473-590, 200-290). */
int fa4b_quant_nvfp4_weight(const fa4b_quant_nvfp4_args* a, void* stream);

/* ---- fa4b_project_nvfp4 --------------------------------------------------
 * y[M, N] bf16 = A[M, K] . W[N, K]^T for two prepared NVFP4 operands (the
 * outputs of fa4b_quant_nvfp4 / fa4b_rmsnorm_quant_nvfp4 for the activation,
 * fa4b_quant_nvfp4_weight for the weight): block-scaled FP4 tensor-core MMAs,
 * FP32 accumulation, the product of the two global scales applied once at
 * the end.  Replaces project_nvfp4_generic behind b300_project_nvfp4
 * (tk_fa4/interface.py:1619-1640).  M % 128 == 0, N % 256 == 0, K % 128 == 0.
 *   status [4] u32 (device): zeroed by the call; status[0] != 0 afterwards
 *   means a device-side wait gave up (status[1] = site). */
typedef struct fa4b_project_nvfp4_args {
  const uint8_t* a_codes;   /* [M, K/2] */
  const uint8_t* a_scales;  /* [M/128, K/64, 512] */
  const float* a_global;    /* [1] */
  const uint8_t* w_codes;   /* [N, K/2] */
  const uint8_t* w_scales;  /* [N/128, K/64, 512] */
  const float* w_global;    /* [1] */
  int64_t M, N, K;
  void* y;                  /* bf16 [M, ldy] */
  int64_t ldy;
  uint32_t* status;
} fa4b_project_nvfp4_args;
int fa4b_project_nvfp4(const fa4b_project_nvfp4_args* a, void* stream);

/* ---- fa4b_project_qkv_publish --------------------------------------------
 * The QKV projection of an attention block with the publication of the
 * attention operands fused into its epilogue: y = x . Wqkv^T is never written;
 * per head of 128 features the epilogue rounds to bf16, rotates Q and K
 * (pair-native, tables bf16 [S, 64]) and writes into the attention workspace
 * `ws` (layout of fa4b_attn_ws_layout_query for `d`) the NVFP4 codes and scale
 * pages of Q and K at a unit global scale, and E4M3(4x) of Q, K and V --
 * what fa4b_project_nvfp4 + fa4b_rope_pair + fa4b_attn_prepare produce in
 * three passes.  The columns of Wqkv are Hq query heads, Hkv key heads, Hkv
 * value heads; rows of x are tokens (batch-major).  a->y is ignored.
 * Requires d->D == 128, FA4B_PV_FP8_E4M3, FA4B_GLOBAL_ONE.  Replaces the
 * epilogue of b300_project_qkv_gqa_d128_unified_lowp_nvfp4
 * (tk_fa4/interface.py:5238; projection_fp4_epilogue.cuh:1453-1579, 873-983).
 * Declared after fa4b_attn_dims below. */

/* ---- fa4b_rope_pair -------------------------------------------------------
 * In-place rotary embedding of x[B, S, H, D] bf16 (element strides given; the
 * last dimension contiguous) in the pair-native order: (x[2i], x[2i+1]) turns
 * by the angle of (rope_cos[s, i], rope_sin[s, i]), tables bf16 [S, D/2].
 * Packed BF16 arithmetic, out = fma(perp, sin, mul(pair, cos)): the numbers of
 * rope_pair_qk_inplace behind b300_rope_pair_qk_ (tk_fa4/interface.py:6584-6599;
 * apply_rope_pair, projection_fp4_epilogue.cuh:447-479).  inverse != 0 turns
 * the other way (the gradient's rotation, b300_inverse_rope_interleaved_qkv_grad_,
 * tk_fa4/interface.py:6564). */
typedef struct fa4b_rope_pair_args {
  void* x;
  int64_t B, S, H, D;
  int64_t stride_b, stride_s, stride_h;
  const void* rope_cos;
  const void* rope_sin;
  int inverse;
} fa4b_rope_pair_args;
int fa4b_rope_pair(const fa4b_rope_pair_args* a, void* stream);

/* ---- fa4b_pack_qkv_grads --------------------------------------------------
 * The operand of the QKV projection's backward GEMMs from the attention
 * gradients in one pass: the token-major matrix [dQ | dK | dV] of
 * [B*S, (Hq + 2 Hkv) D] bf16 is gathered from the three gradient tensors
 * (rows are tokens, batch-major; row strides in elements, so the three may be
 * column ranges of one buffer), dQ and dK turn back through the pair-native
 * rotation of their token (the arithmetic of fa4b_rope_pair with inverse != 0),
 * and the result is written as NVFP4 rows and, optionally, transposed NVFP4
 * (outputs as in fa4b_quant_nvfp4 with rows = B*S, cols = (Hq + 2 Hkv) D).
 * Byte for byte what fa4b_rope_pair on dQ and dK followed by fa4b_quant_nvfp4
 * of the concatenation produce; the rotated bf16 matrix is never written.
 * amax: written (one extra read of the gradients) unless amax_is_input != 0 --
 * the reference's producer always takes a global scale decided beforehand.
 * Replaces the producer kernel of
 * tk_fa4/lowp_fa4_bwd/gqa_d128_hierarchical_qkv_nvfp4_quantize.cuh:1-140 behind
 * b300_pack_gqa_d128_hierarchical_qkv_gradient_nvfp4_tiles
 * (tk_fa4/interface.py:4864-4912) for row-major dQ, and its D = 64 sibling
 * b300_project_gqa_d64_paired_qkv_gradient_nvfp4 (tk_fa4/interface.py:4712).
 * B*S and (Hq + 2 Hkv) D must be multiples of 128; D is 64 or 128. */
typedef struct fa4b_pack_qkv_grads_args {
  const void* dq;          /* bf16, token row t at dq + t * ld_q: Hq heads of D   */
  const void* dk;          /* bf16, Hkv heads of D per token                      */
  const void* dv;
  int64_t ld_q, ld_k, ld_v;
  int64_t B, S, Hq, Hkv, D;
  const void* rope_cos;    /* bf16 [S, D/2] */
  const void* rope_sin;
  float* amax;
  int amax_is_input;
  float* global_scale;
  uint8_t* codes_row;
  uint8_t* scales_row;
  uint8_t* codes_col;      /* NULL = no transposed output */
  uint8_t* scales_col;
  int recipe;              /* FA4B_RECIPE_* */
} fa4b_pack_qkv_grads_args;
int fa4b_pack_qkv_grads(const fa4b_pack_qkv_grads_args* a, void* stream);

/* ---- fa4b_rmsnorm_quant_nvfp4 -------------------------------------------
 * y = bf16((x * inv_rms[row]) * gamma[col]), inv_rms = 1/sqrt(mean x^2 + eps);
 * then fa4b_quant_nvfp4 of y with amax over the bf16 y.  Replaces
 * tk_fused_norm_quantize (TK_quantisation/nvfp4_v6/tk_quantize.cu:2353-2366)
 * and quantize_nvfp4_projection_operand_rmsnorm (tk_fa4/interface.py:1056).
 *   inv_rms [rows] f32 out;  y_out [rows, cols] bf16 optional (NULL = skip). */
typedef struct fa4b_rmsnorm_quant_nvfp4_args {
  const void* x;
  const void* gamma;
  int64_t rows, cols, ld;
  float eps;
  float* inv_rms;
  void* y_out;
  float* amax;
  float* global_scale;
  uint8_t* codes_row;
  uint8_t* scales_row;
  uint8_t* codes_col;
  uint8_t* scales_col;
  int recipe;          /* FA4B_RECIPE_* */
} fa4b_rmsnorm_quant_nvfp4_args;
int fa4b_rmsnorm_quant_nvfp4(const fa4b_rmsnorm_quant_nvfp4_args* a, void* stream);

/* ---- fa4b_rmsnorm_bwd ---------------------------------------------------
 * Backward of y = (x * inv_rms[row]) * gamma[col] given dy:
 *   proj[row] = mean_col(dy * gamma * x);  dx = bf16(inv_rms * (dy * gamma - x * inv_rms^2 * proj));
 *   dgamma[col] = bf16(sum_row dy * (x * inv_rms)), accumulated in FP32.
 * Replaces rmsnorm_backward_bf16 (tk_fa4/interface.py:1144-1150; kernel
 * tk_fa4/lowp_fa4_bwd/rmsnorm_nvfp4_quantize.cuh:321-462), for any cols % 8 == 0 up to 8192 instead of
 * the reference's fixed 2048.  `partials` is caller-owned FP32 scratch of
 * fa4b_rmsnorm_bwd_workspace_bytes(cols) bytes (per-CTA column sums before the final reduction). */
typedef struct fa4b_rmsnorm_bwd_args {
  const void* x;      /* [rows, cols] bf16, row stride ld */
  const void* gamma;  /* [cols] bf16 */
  const float* inv_rms; /* [rows] */
  const void* dy;     /* [rows, cols] bf16, row stride ld_dy */
  int64_t rows, cols, ld, ld_dy;
  void* dx;           /* [rows, cols] bf16, dense */
  void* dgamma;       /* [cols] bf16 */
  float* partials;
} fa4b_rmsnorm_bwd_args;
size_t fa4b_rmsnorm_bwd_workspace_bytes(int64_t cols);
int fa4b_rmsnorm_bwd(const fa4b_rmsnorm_bwd_args* a, void* stream);

/* ---- fa4b_quant_mxfp4 ---------------------------------------------------
 * Row-wise 1x32 MXFP4 with E8M0 scales.  Replaces mxfp4_quantize_for_gemm
 * (TK_quantisation/mxfp4_v3/tk_quantize.cu:2052-2054).
 *   codes [rows, cols/2]; scales [rows/128, cols/128, 512] E8M0 bytes, same
 *   page byte order as above with kblock = col/32; byte 0 = all-zero block. */
typedef struct fa4b_quant_mxfp4_args {
  const void* x;
  int64_t rows, cols, ld;
  int mode; /* FA4B_MX_* */
  uint8_t* codes;
  uint8_t* scales;
} fa4b_quant_mxfp4_args;
int fa4b_quant_mxfp4(const fa4b_quant_mxfp4_args* a, void* stream);

/* ---- fa4b_dequant_* (test utilities) --------------------------------------
 * Replace tk_reconstruct_row (TK_quantisation/nvfp4_v6/tk_quantize.cu:3225-3234)
 * and decode_prepared_nvfp4_matrix (projection_quantization_reference.py:293-329). */
int fa4b_dequant_nvfp4(const uint8_t* codes, const uint8_t* scale_pages, const float* global_scale,
                       int64_t rows, int64_t cols, float* out_f32, void* stream);
int fa4b_dequant_mxfp4(const uint8_t* codes, const uint8_t* scale_pages,
                       int64_t rows, int64_t cols, float* out_f32, void* stream);

/* ---- attention ------------------------------------------------------------
 * Causal grouped-query attention, NVFP4 Q.K^T and FP8-E4M3 (or MXFP4) P.V.
 * q/o/do/dq are [B,Hq,S,D], k/v/dk/dv [B,Hkv,S,D] bf16, addressed through
 * element strides (batch, head, seq); the last dim is contiguous.  S must be a
 * multiple of 128, D is 64 or 128, Hq a multiple of Hkv.
 *
 * The operand cache `ws` (fa4b_attn_workspace_bytes) receives, in this order:
 *   q NVFP4 codes [B,Hq,S,D/2], scale pages [B,Hq,S/128,D/64,512], global [B,Hq];
 *   the same for k; v as E4M3(4v) [B,Hkv,S,D]; q and k as E4M3(4x) (backward);
 * the optional out-pointers of fa4b_attn_fwd_args expose them for parity checks. */
typedef struct fa4b_attn_dims {
  int32_t B, Hq, Hkv, S, D;
  float softmax_scale; /* <= 0: 1/sqrt(D) */
  int32_t pv_format;   /* FA4B_PV_* */
  int32_t mask;        /* FA4B_MASK_*; forward only.  FA4B_MASK_NONE serves the off-diagonal blocks of a
                          sequence-sharded (context-parallel) run, where every key precedes every query */
  int32_t global_scale_mode; /* FA4B_GLOBAL_*; read by fa4b_attn_prepare (and fa4b_attn_fwd when it prepares) */
} fa4b_attn_dims;

typedef struct fa4b_strides {
  int64_t batch, head, seq; /* in elements */
} fa4b_strides;

size_t fa4b_attn_workspace_bytes(const fa4b_attn_dims* d);
int fa4b_project_qkv_publish(const fa4b_project_nvfp4_args* a, const fa4b_attn_dims* d, const void* rope_cos, const void* rope_sin, void* ws,
                             void* stream);
/* The output projection's input-gradient GEMM dO = dY . Wo with the backward's publication fused into its epilogue:
 * dO is never written as bf16; per head the epilogue writes E5M2(4 dO), dstat and lstat into `ws` -- what
 * fa4b_project_nvfp4 + fa4b_attn_bwd_preprocess produce in two passes (fa4b_attn_bwd then runs with
 * preprocessed = 1).  o_rows: the forward's output, bf16 [B*S, Hq*128]; lse f32 [B, Hq, S].  Replaces the epilogue of
 * b300_project_dout_unified_lowp_nvfp4_v509_e5m2 (tk_fa4/interface.py:5824-5942; projection_fp4_epilogue.cuh:4049-4127). */
int fa4b_project_dout_publish(const fa4b_project_nvfp4_args* a, const fa4b_attn_dims* d, const void* o_rows, const float* lse, void* ws,
                              void* stream);

/* Offsets (bytes) of the cached operands inside the workspace.  With pv_format = FA4B_PV_MXFP4_E8M0 the
 * `v_fp8` section holds V as sequence-grouped MXFP4 instead (the operand of forward_hao_direct_fp4pv,
 * hao_direct_fp4pv_host.inc:1141-1237): codes [B*Hkv, D, S/2] (two keys per byte, feature-major), then at the
 * next multiple of 1024 bytes the E8M0 scale pages [B*Hkv, S/128, 512] (row = feature, k-block = 32 keys). */
typedef struct fa4b_attn_ws_layout {
  /* saved section [0, saved_total): published by the forward, replayed by the backward -- the only bytes a
   * training step has to keep between the two (the reference keeps the same operands, release/routes.json:443-447) */
  size_t q_codes, q_scales, q_global, k_codes, k_scales, k_global;
  size_t v_fp8, k_fp8, q_fp8, amax_bits, status, saved_total;
  /* transient section [saved_total, total): lives inside one backward call -- E5M2 dO, dstat, lstat, the dQ
   * accumulator (FP32-sized; a call that forms the whole sum keeps f16 values in its first half, see fa4b_attn_bwd)
   * and the FP32 dK / dV accumulators of key tiles whose query range is split over several CTAs.
   * Either the tail of `ws`, or a separate buffer of total - saved_total bytes passed as
   * fa4b_attn_bwd_args.scratch and shared by every layer */
  size_t do_fp8, dstat, lstat, dq_accum, dkv_accum, total;
} fa4b_attn_ws_layout;
int fa4b_attn_ws_layout_query(const fa4b_attn_dims* d, fa4b_attn_ws_layout* out);

/* fa4b_attn_prepare: per-(batch, head) amax, NVFP4 Q/K and E4M3 V/Q/K
 * publication into `ws`.  Replaces the quantise/publish half of the QKV
 * projection epilogue (tk_fa4/lowp_fa4_bwd/projection_fp4_epilogue.cuh:
 * 1453-1579 stage_codes_perblock_qk, 1861-1945 publish_forward_qk_perblock_scales,
 * 873-983 publish_v_fp8). */
typedef struct fa4b_attn_prepare_args {
  fa4b_attn_dims dims;
  const void* q; fa4b_strides q_strides;
  const void* k; fa4b_strides k_strides;
  const void* v; fa4b_strides v_strides;
  void* ws;
  int32_t phase; /* 0: everything.  FA4B_PREPARE_AMAX: only the per-(batch, head) amax words of q and k
                    (fa4b_attn_ws_layout.amax_bits: B*Hq then B*Hkv f32).  FA4B_PREPARE_QUANTIZE: publish with
                    the amax words already in `ws` -- a caller that shards the sequence across GPUs takes the
                    maximum of the words over its shards and ranks between the two phases, so that every
                    shard is quantised with the scale of the whole sequence */
} fa4b_attn_prepare_args;
int fa4b_attn_prepare(const fa4b_attn_prepare_args* a, void* stream);

/* fa4b_attn_fwd: O and LSE (natural log, [B,Hq,S] f32).  Replaces
 * forward_hao_direct_fp8pv / forward_hao_direct_fp4pv
 * (tk_fa4/fp4_fa4_fwd/hao_direct_host.inc:263-275, 511-521;
 * hao_direct_fp4pv_host.inc:1141-1237).  Unless `prepared` is non-zero the call
 * publishes the operands itself: one statistics launch for the per-head amax of Q and K (none at the unit global
 * scale), one launch that publishes K and V, and the forward kernel quantises its own query rows to NVFP4 (16-element
 * blocks, E4M3 block scales, the head's FP32 global scale) before its first Q.K^T, leaving codes, scale pages and
 * E4M3(4q) in `ws` for the backward -- byte for byte what fa4b_attn_prepare writes.  The MXFP4 P.V route quantises P to MXFP4 in 32-key groups (E8M0, ceil) inside the
 * kernel, takes the row sum over the represented P, and is forward only (fa4b_attn_bwd returns FA4B_UNSUPPORTED). */
typedef struct fa4b_attn_fwd_args {
  fa4b_attn_dims dims;
  const void* q; fa4b_strides q_strides;
  const void* k; fa4b_strides k_strides;
  const void* v; fa4b_strides v_strides;
  void* o; fa4b_strides o_strides;
  float* lse;
  void* ws;
  int32_t prepared;
  void* ev_before; /* optional cudaEvent_t recorded just before / after the */
  void* ev_after;  /* attention kernel itself (per-kernel timing)           */
  const void* kv_ws; /* optional: a second operand cache of the same dims whose K and V sections (k_codes up to
                        q_fp8 of the layout, one contiguous range) are used instead of `ws`'s; with prepared != 0
                        this is how a block of queries meets the keys of another sequence shard */
} fa4b_attn_fwd_args;
int fa4b_attn_fwd(const fa4b_attn_fwd_args* a, void* stream);

/* fa4b_attn_merge: fold one partial result into a running one, row by row (n_rows = B*Hq*S rows of D values):
 * lse' = log(exp(lse_acc) + exp(lse_part)), o_acc' = o_acc exp(lse_acc - lse') + o_part exp(lse_part - lse').
 * o_acc f32 [n_rows, D] and lse_acc f32 [n_rows] are updated in place (start from o_acc = 0, lse_acc = -inf);
 * o_part is the bf16 [n_rows, D] output of fa4b_attn_fwd on one key shard, lse_part its LSE.  With o_out != NULL
 * the merged rows are also written as bf16 (the last fold).  The reference has no counterpart (it runs
 * data-parallel replicas only, torchtitan/experiments/fa4/exact_lowp_attention.py:4123-4136). */
int fa4b_attn_merge(float* o_acc, float* lse_acc, const void* o_part, const float* lse_part, int64_t n_rows, int32_t D,
                    void* o_out, void* stream);

/* fa4b_attn_fwd_static: fa4b_attn_fwd for hosts that cannot allocate device
 * memory where attention runs (an execute hook that must not allocate, a
 * serving loop with a frozen memory budget).  No counterpart in the reference,
 * whose callers always pre-allocate.  `ws` and `prepared` of the args are
 * ignored: the operand cache is a fixed array inside the library, held by every
 * GPU that loads it until the process exits.  Shapes whose forward operands
 * (fa4b_attn_ws_layout.saved_total) exceed FA4B_STATIC_WS_BYTES are rejected with
 * FA4B_BAD_SHAPE.  Calls no cudaMalloc/cudaFree or any allocating routine.
 * fa4b_attn_check_status(dims, NULL, stream) reports a device-side wait that ran
 * out during the last such call on the current device.
 * The first call on a device looks the array's address up (once per device,
 * with that device current); make that first call before any stream capture.
 * All calls share the array: calls that overlap on the GPU race. */
#define FA4B_STATIC_WS_BYTES (8u << 20)
int fa4b_attn_fwd_static(const fa4b_attn_fwd_args* a, void* stream);

/* fa4b_attn_bwd_preprocess: dO5 = E5M2(4 dO), dstat = -4 sum_d O*dO5,
 * lstat = 8 - LSE*log2e, into `ws`.  Replaces the dO/statistics publisher
 * project_dout_unified_fp4_nvfp4_v509_e5m2
 * (tk_fa4/lowp_fa4_bwd/projection_fp4_epilogue.cuh:840-871, 4049-4127). */
typedef struct fa4b_attn_bwd_args {
  fa4b_attn_dims dims;
  const void* o; fa4b_strides o_strides;
  const void* dout; fa4b_strides do_strides;
  const float* lse;
  void* dq; fa4b_strides dq_strides;
  void* dk; fa4b_strides dk_strides;
  void* dv; fa4b_strides dv_strides;
  void* ws; /* the workspace the forward filled (operands are replayed from it) */
  int32_t preprocessed; /* non-zero: fa4b_attn_bwd_preprocess already ran on ws */
  void* ev_before;      /* optional cudaEvent_t around the main backward kernel */
  void* ev_after;
  const void* kv_ws;    /* optional: a second operand cache of the same dims whose K and V sections are used instead
                           of `ws`'s (the keys of another sequence shard); the queries, dO and statistics stay `ws`'s */
  int32_t flags;        /* FA4B_BWD_*: how this call treats the dQ accumulator */
  void* scratch;        /* optional, 1024-byte aligned: the transient section of the layout (total - saved_total
                           bytes) as a buffer of its own; `ws` then only needs its first saved_total bytes.  NULL:
                           the transient section is the tail of `ws` */
} fa4b_attn_bwd_args;
int fa4b_attn_bwd_preprocess(const fa4b_attn_bwd_args* a, void* stream);

/* fa4b_attn_bwd: dQ, dK, dV (bf16, written, not accumulated).  Replaces
 * backward_nvfp4_score_e4m3_qkv_e5m2_dout_bshd_precleared_dq_out
 * (tk_fa4/native_gqa_tk_bwd/v509_*bshd.cu:406-444) and the D64 kernel v416.
 * Runs the preprocess step itself unless `preprocessed` is set.  Uses the
 * transient section's accumulators as scratch (dQ zeroed here unless FA4B_BWD_KEEP_DQ_ACCUM).  The partial dQ sums of
 * the key tiles meet in the dQ accumulator as f16 pairs (32 dQ per value: half the reduction traffic of FP32 sums, the
 * reference's v420 adds them as bf16; dQ of two runs then differs by the order of those roundings, about 1e-3
 * relative) when one call forms the whole sum; FA4B_BWD_DQ_SUMS_FP32 asks for FP32 sums, and a sum carried across
 * calls (FA4B_BWD_KEEP_DQ_ACCUM, FA4B_BWD_SKIP_DQ_OUT) is always FP32: such a sum starts with a call that carries
 * FA4B_BWD_SKIP_DQ_OUT, never with a call that wrote dq (the accumulator would hold f16 words).  One CTA per
 * (key tile, part of the tile's query range, batch and kv head), key-tile-major; in a launch of few heads a key
 * tile that sees more query tiles than the launch's chunk length is cut into parts whose dK / dV meet as FP32
 * sums (fa4b_attn_bwd_plan).  With
 * dims.mask = FA4B_MASK_NONE every key is visible to every query (a key shard that precedes the query shard);
 * the statistics must then come from the LSE and O of the whole sequence. */
int fa4b_attn_bwd(const fa4b_attn_bwd_args* a, void* stream);

/* fa4b_attn_bwd_plan / _plan_item: host only.  The work list fa4b_attn_bwd launches for `d` on a device of n_sm
 * multiprocessors (n_sm <= 0: the current device): one CTA per item; items_per_head items per (batch, kv head):
 * the key tiles in order, each tile's query range in `parts` nearly equal pieces of at most `chunk` query tiles
 * (chunk = S / 128, i.e. no cut, when the launch has about six CTAs per SM without one).  Launch order: the heads
 * in groups of head_group (as many as keep the group's FP32 dQ rows within about half of L2); inside a group
 * key-tile-major: item i of every head of the group, then item i + 1.  split_rows: leading key rows of every kv
 * head whose dK / dV pass through the FP32 accumulators.  Stands in for the grid half of
 * native_tk_d128_backward_metadata() (tk_fa4/native_gqa_tk_bwd/v509_*bshd.cu:446-522; grid at
 * v509_*bshd.cuh:1561-1565).  _plan_item writes {batch * Hkv + kv head, key tile, first query tile, end query
 * tile, parts} of the CTA with block index `index`. */
typedef struct fa4b_bwd_plan {
  int32_t chunk, items_per_head, split_rows, head_group;
  int64_t grid;
} fa4b_bwd_plan;
int fa4b_attn_bwd_plan(const fa4b_attn_dims* d, int32_t n_sm, fa4b_bwd_plan* out);
int fa4b_attn_bwd_plan_item(const fa4b_attn_dims* d, int32_t n_sm, int64_t index, int32_t out[5]);

/* fa4b_attn_accumulate: acc[i] += part[i] (FP32 += bf16) over n values, n % 8 == 0; with out != NULL the sums are
 * also written as bf16.  Folds the dK / dV of one block call into a running FP32 sum (no reference counterpart). */
int fa4b_attn_accumulate(float* acc, const void* part, int64_t n, void* out, void* stream);

/* fa4b_attn_check_status: synchronises `stream`, then reports FA4B_TIMEOUT if a
 * bounded wait inside the last attention kernel on this workspace gave up
 * (the reference's waits are unbounded, hao_direct_kernel.inc:17-23; this
 * query has no counterpart there).  ws == NULL: the built-in operand cache of
 * fa4b_attn_fwd_static on the current device. */
int fa4b_attn_check_status(const fa4b_attn_dims* d, const void* ws, void* stream);

/* ---- tensor-core self tests ("microgates") -------------------------------
 * One 128x128xK product per launch through the same tcgen05 instruction
 * forms, shared-memory descriptors and TMEM layouts the attention kernels
 * use; out is [128,128] f32.  The reference proves each primitive the same
 * way (tk_fa4/native_gqa_tk_bwd/e5m2_dout_mixed_mma_microgate_20260831.cuh:213-316).
 *   kind 0: NVFP4 x NVFP4 block-scaled (a,b packed codes [128,K/2], sfa/sfb pages)
 *   kind 1: E4M3 x E4M3, both K-major        kind 2: E4M3 x E5M2, both K-major
 *   kind 3: E4M3 A K-major, B MN-major ([K,128] row-major)
 *   kind 4: A MN-major ([K,128]), B MN-major  kind 5: A from TMEM (TS form), B MN-major
 *   kind 6: MXFP4 x MXFP4 block-scaled (E8M0 scale pages)
 * status_out [4] u32 device: [0] = 0 ok / 1 wait ran out. */
int fa4b_microgate(int kind, int K, const void* a, const void* b, const void* sfa, const void* sfb,
                   float* out, uint32_t* status_out, void* stream);

/* Tensor-core peak of this GPU for the two MMA kinds the attention kernels use: one CTA per SM issues
 * `iters` back-to-back MMAs (M128 N256; kind 0: kind::f8f6f4 E4M3, K32; kind 1: kind::mxf4nvf4 block-scaled
 * E2M1, K64) on operands resident in shared memory.  The caller times the launch; FLOPs = SMs * iters *
 * 2*128*256*K.  Gives the roofline denominators that the reference reads off data sheets
 * (results/fp4_fa4_technical_report_v2_20260819/sections/07_profile.tex:183-184 quotes nominal peaks).
 * status_out [4] u32 device: [0] = 0 ok / 1 wait ran out. */
int fa4b_tensor_peak(int kind, int iters, uint32_t* status_out, void* stream);

/* fa4b_wait_selftest: the give-up path of the kernels' bounded waits, run on purpose and harmlessly: one small
 * kernel waits, with a budget of limit_cycles SM clocks (1..1e8), on barriers that nothing arms -- no copy or
 * tensor-core operation in flight -- records the site as the attention kernels do and returns.  The expected
 * result is FA4B_TIMEOUT with the site in fa4b_last_error(); the context stays usable.  status_out [8] u32 device:
 * [0..3] the give-up record, [4..6] what the two waits saw.  (The reference's waits are unbounded,
 * hao_direct_kernel.inc:17-23, and have no such test.) */
int fa4b_wait_selftest(int64_t limit_cycles, uint32_t* status_out, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* FA4B_H_ */

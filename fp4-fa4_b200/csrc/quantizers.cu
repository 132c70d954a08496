// Memory-bound block quantizers: amax, NVFP4 (row-wise + transposed), fused
// RMSNorm + NVFP4, MXFP4, and the decode utilities.  All are HBM-bound byte
// work: 128-bit loads, warp-shuffle reductions, packed e2m1 stores, one
// 128x128 tile per CTA staged in shared memory so that the transposed
// quantisation reads the input once.
#include <cstdarg>
#include <mutex>

#include "common.cuh"
#include "tc_sm100.cuh"

namespace fa4b {

static thread_local char g_error[512] = "";
void set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_error, sizeof(g_error), fmt, ap);
  va_end(ap);
}
const char* last_error() { return g_error; }

// multiprocessors of the current device (148 on a B200); 0 when the query fails
int sm_count() {
  static std::mutex mu;
  static int cached[64] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return 0;
  std::lock_guard<std::mutex> lock(mu);
  if (dev >= 0 && dev < 64 && cached[dev] > 0) return cached[dev];
  int n = 0;
  if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return 0;
  if (dev >= 0 && dev < 64) cached[dev] = n;
  return n;
}

// ------------------------------------------------------------------ amax
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

__device__ __forceinline__ __nv_bfloat162 absmax2(__nv_bfloat162 acc, uint32_t w) {
  return __hmax2(acc, __habs2(*reinterpret_cast<__nv_bfloat162*>(&w)));
}

__global__ void __launch_bounds__(256) amax_kernel(const uint4* __restrict__ x, int64_t n_vec, const __nv_bfloat16* tail,
                                                   int n_tail, float* __restrict__ amax) {
  __nv_bfloat162 acc = __float2bfloat162_rn(0.f);
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
  for (; i + 3 * stride < n_vec; i += 4 * stride) {  // four independent loads in flight per thread
    const uint4 v0 = __ldg(x + i), v1 = __ldg(x + i + stride), v2 = __ldg(x + i + 2 * stride), v3 = __ldg(x + i + 3 * stride);
    acc = absmax2(absmax2(absmax2(absmax2(acc, v0.x), v0.y), v0.z), v0.w);
    acc = absmax2(absmax2(absmax2(absmax2(acc, v1.x), v1.y), v1.z), v1.w);
    acc = absmax2(absmax2(absmax2(absmax2(acc, v2.x), v2.y), v2.z), v2.w);
    acc = absmax2(absmax2(absmax2(absmax2(acc, v3.x), v3.y), v3.z), v3.w);
  }
  for (; i < n_vec; i += stride) {
    const uint4 v = __ldg(x + i);
    acc = absmax2(absmax2(absmax2(absmax2(acc, v.x), v.y), v.z), v.w);
  }
  float m = fmaxf(__bfloat162float(acc.x), __bfloat162float(acc.y));
  if (blockIdx.x == 0 && threadIdx.x < n_tail) m = fmaxf(m, fabsf(__bfloat162float(tail[threadIdx.x])));
  m = warp_max(m);
  __shared__ float wm[8];
  if ((threadIdx.x & 31) == 0) wm[threadIdx.x >> 5] = m;
  __syncthreads();
  if (threadIdx.x < 32) {
    m = warp_max(threadIdx.x < 8 ? wm[threadIdx.x] : 0.f);
    if (threadIdx.x == 0) atomicMax(reinterpret_cast<int*>(amax), __float_as_int(m));  // non-negative floats order as ints
  }
}

// ------------------------------------------------------------------ RMSNorm statistics
// One CTA per row: inv_rms, and the amax of y = bf16((x*inv_rms)*gamma).  The row stays in
// registers between the two reductions, so x is read once here.
template <int VEC_PER_THREAD>
__global__ void __launch_bounds__(256) rmsnorm_stats_kernel(const __nv_bfloat16* __restrict__ x, int64_t ld, int cols,
                                                            const __nv_bfloat16* __restrict__ gamma, float eps,
                                                            float* __restrict__ inv_rms, float* __restrict__ amax) {
  const int64_t row = blockIdx.x;
  const uint4* xr = reinterpret_cast<const uint4*>(x + row * ld);
  const uint4* gr = reinterpret_cast<const uint4*>(gamma);
  const int n_vec = cols / 8;
  uint4 v[VEC_PER_THREAD];
  float ss = 0.f;
#pragma unroll
  for (int j = 0; j < VEC_PER_THREAD; ++j) {
    const int i = threadIdx.x + j * 256;
    v[j] = (i < n_vec) ? __ldg(xr + i) : make_uint4(0, 0, 0, 0);
    const uint32_t w[4] = {v[j].x, v[j].y, v[j].z, v[j].w};
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const float a = bf16_bits_to_f32(w[k] & 0xffffu), b = bf16_bits_to_f32(w[k] >> 16);
      ss = fmaf(a, a, ss);
      ss = fmaf(b, b, ss);
    }
  }
  __shared__ float red[8];
  __shared__ float s_inv;
  ss = warp_sum(ss);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
  __syncthreads();
  if (threadIdx.x == 0) {
    float t = 0.f;
#pragma unroll
    for (int k = 0; k < 8; ++k) t += red[k];
    const float inv = 1.0f / sqrtf(t / (float)cols + eps);
    s_inv = inv;
    inv_rms[row] = inv;
  }
  __syncthreads();
  const float inv = s_inv;
  float m = 0.f;
#pragma unroll
  for (int j = 0; j < VEC_PER_THREAD; ++j) {
    const int i = threadIdx.x + j * 256;
    if (i < n_vec) {
      const uint4 gv = __ldg(gr + i);
      const uint32_t w[4] = {v[j].x, v[j].y, v[j].z, v[j].w};
      const uint32_t gw[4] = {gv.x, gv.y, gv.z, gv.w};
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const float a = (bf16_bits_to_f32(w[k] & 0xffffu) * inv) * bf16_bits_to_f32(gw[k] & 0xffffu);
        const float b = (bf16_bits_to_f32(w[k] >> 16) * inv) * bf16_bits_to_f32(gw[k] >> 16);
        m = fmaxf(m, fmaxf(fabsf(__bfloat162float(__float2bfloat16_rn(a))), fabsf(__bfloat162float(__float2bfloat16_rn(b)))));
      }
    }
  }
  m = warp_max(m);
  __syncthreads();
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = m;
  __syncthreads();
  if (threadIdx.x == 0) {
    float t = 0.f;
#pragma unroll
    for (int k = 0; k < 8; ++k) t = fmaxf(t, red[k]);
    atomicMax(reinterpret_cast<int*>(amax), __float_as_int(t));
  }
}

// ------------------------------------------------------------------ RMSNorm backward
// One CTA walks rows blockIdx.x, blockIdx.x + gridDim.x, ...; a thread owns VEC chunks of 8 columns, keeps gamma
// and its column sums of dy * (x * inv_rms) in registers, and leaves the sums as one FP32 row of `partials`.
constexpr int kRmsBwdParts = 512;  // upper bound of the partial rows (sizes the workspace, whatever the device); a launch uses two CTAs per SM
template <int VEC>
__global__ void __launch_bounds__(256) rmsnorm_bwd_kernel(const __nv_bfloat16* __restrict__ x, int64_t ld, const __nv_bfloat16* __restrict__ gamma,
                                                          const float* __restrict__ inv_rms, const __nv_bfloat16* __restrict__ dy, int64_t ld_dy,
                                                          int64_t rows, int cols, __nv_bfloat16* __restrict__ dx, float* __restrict__ partials) {
  const int n_vec = cols / 8;
  float gv[VEC][8], acc[VEC][8];
#pragma unroll
  for (int j = 0; j < VEC; ++j) {
    const int i = threadIdx.x + j * 256;
    uint4 g4 = make_uint4(0, 0, 0, 0);
    if (i < n_vec) g4 = __ldg(reinterpret_cast<const uint4*>(gamma) + i);
    const uint32_t w[4] = {g4.x, g4.y, g4.z, g4.w};
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      gv[j][2 * k] = bf16_bits_to_f32(w[k] & 0xffffu);
      gv[j][2 * k + 1] = bf16_bits_to_f32(w[k] >> 16);
      acc[j][2 * k] = acc[j][2 * k + 1] = 0.f;
    }
  }
  __shared__ float red[8];
  __shared__ float s_proj;
  for (int64_t row = blockIdx.x; row < rows; row += gridDim.x) {
    float xv[VEC][8], dv[VEC][8];
    float local = 0.f;
#pragma unroll
    for (int j = 0; j < VEC; ++j) {
      const int i = threadIdx.x + j * 256;
      uint4 x4 = make_uint4(0, 0, 0, 0), d4 = make_uint4(0, 0, 0, 0);
      if (i < n_vec) {
        x4 = __ldg(reinterpret_cast<const uint4*>(x + row * ld) + i);
        d4 = __ldg(reinterpret_cast<const uint4*>(dy + row * ld_dy) + i);
      }
      const uint32_t xw[4] = {x4.x, x4.y, x4.z, x4.w}, dw[4] = {d4.x, d4.y, d4.z, d4.w};
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        xv[j][2 * k] = bf16_bits_to_f32(xw[k] & 0xffffu);
        xv[j][2 * k + 1] = bf16_bits_to_f32(xw[k] >> 16);
        dv[j][2 * k] = bf16_bits_to_f32(dw[k] & 0xffffu);
        dv[j][2 * k + 1] = bf16_bits_to_f32(dw[k] >> 16);
      }
#pragma unroll
      for (int e = 0; e < 8; ++e) local = fmaf(dv[j][e] * gv[j][e], xv[j][e], local);
    }
    local = warp_sum(local);
    __syncthreads();  // the previous row's s_proj has been read by everyone
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = local;
    __syncthreads();
    if (threadIdx.x == 0) {
      float tsum = 0.f;
#pragma unroll
      for (int k = 0; k < 8; ++k) tsum += red[k];
      s_proj = tsum / (float)cols;
    }
    __syncthreads();
    const float inv = __ldg(inv_rms + row);
    const float corr = inv * inv * s_proj;
#pragma unroll
    for (int j = 0; j < VEC; ++j) {
      const int i = threadIdx.x + j * 256;
      uint32_t o[4];
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const float a = inv * (dv[j][2 * k] * gv[j][2 * k] - xv[j][2 * k] * corr);
        const float b = inv * (dv[j][2 * k + 1] * gv[j][2 * k + 1] - xv[j][2 * k + 1] * corr);
        const __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
        o[k] = *reinterpret_cast<const uint32_t*>(&h);
      }
      if (i < n_vec) *reinterpret_cast<uint4*>(dx + row * (int64_t)cols + (int64_t)i * 8) = make_uint4(o[0], o[1], o[2], o[3]);
#pragma unroll
      for (int e = 0; e < 8; ++e) acc[j][e] = fmaf(dv[j][e], xv[j][e] * inv, acc[j][e]);
    }
  }
#pragma unroll
  for (int j = 0; j < VEC; ++j) {
    const int i = threadIdx.x + j * 256;
    if (i < n_vec) {
      float* dst = partials + (int64_t)blockIdx.x * cols + (int64_t)i * 8;
      *reinterpret_cast<float4*>(dst) = make_float4(acc[j][0], acc[j][1], acc[j][2], acc[j][3]);
      *reinterpret_cast<float4*>(dst + 4) = make_float4(acc[j][4], acc[j][5], acc[j][6], acc[j][7]);
    }
  }
}
__global__ void __launch_bounds__(256) rmsnorm_bwd_reduce_kernel(const float* __restrict__ partials, int n_parts, int cols,
                                                                 __nv_bfloat16* __restrict__ dgamma) {
  const int c = blockIdx.x * 256 + threadIdx.x;
  if (c >= cols) return;
  float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;
  int p = 0;
  for (; p + 4 <= n_parts; p += 4) {
    a0 += partials[(int64_t)p * cols + c];
    a1 += partials[(int64_t)(p + 1) * cols + c];
    a2 += partials[(int64_t)(p + 2) * cols + c];
    a3 += partials[(int64_t)(p + 3) * cols + c];
  }
  for (; p < n_parts; ++p) a0 += partials[(int64_t)p * cols + c];
  dgamma[c] = __float2bfloat16_rn((a0 + a1) + (a2 + a3));
}

// ------------------------------------------------------------------ NVFP4 tile kernel
constexpr int kTile = 128;

struct Nvfp4Params {
  const __nv_bfloat16* x;
  int64_t ld;
  int64_t rows, cols;
  const __nv_bfloat16* gamma;  // NORM only
  const float* inv_rms;        // NORM only
  __nv_bfloat16* y_out;        // NORM only, optional
  const float* amax;
  float* global_scale;
  uint8_t* codes_row;
  uint8_t* scales_row;
  uint8_t* codes_col;
  uint8_t* scales_col;
  int recipe;  // FA4B_RECIPE_*
  // GRADS staging: columns [0, n0) come from x, [n0, n1) from x1, [n1, cols) from x2 (each with its own row stride); the
  // first two ranges are heads of D features that turn back through the rotation of row % S
  const __nv_bfloat16* x1;
  const __nv_bfloat16* x2;
  int64_t ld1, ld2, n0, n1;
  const __nv_bfloat16* rope_cos;
  const __nv_bfloat16* rope_sin;
  int S, D;
};

// One bf16 pair (x, y) turned by the angle of (cos, sin) in packed bf16 arithmetic, out = fma(perp, sin, mul(pair, cos))
// with perp = (-y, x): the numbers of apply_rope_pair (tk_fa4/lowp_fa4_bwd/projection_fp4_epilogue.cuh:447-479).
__device__ __forceinline__ uint32_t rope_word(uint32_t w, uint32_t c16, uint32_t s16) {
  const uint32_t cc = c16 * 0x00010001u, s2 = s16 * 0x00010001u;
  const uint32_t perp = ((w << 16) | (w >> 16)) ^ 0x00008000u;
  const __nv_bfloat162 r = __hfma2(*reinterpret_cast<const __nv_bfloat162*>(&perp), *reinterpret_cast<const __nv_bfloat162*>(&s2),
                                   __hmul2(*reinterpret_cast<const __nv_bfloat162*>(&w), *reinterpret_cast<const __nv_bfloat162*>(&cc)));
  return *reinterpret_cast<const uint32_t*>(&r);
}
// Eight gradient features of (row, col) of the [dQ | dK | dV] matrix, dQ and dK turned back through the rotation.
__device__ __forceinline__ uint4 load_grad_chunk(const Nvfp4Params& p, int64_t row, int64_t col) {
  const __nv_bfloat16* src = col < p.n0 ? p.x + row * p.ld + col : (col < p.n1 ? p.x1 + row * p.ld1 + (col - p.n0) : p.x2 + row * p.ld2 + (col - p.n1));
  uint4 v = __ldg(reinterpret_cast<const uint4*>(src));
  if (col < p.n1) {
    const int s = (int)(row % p.S), d8 = (int)((col < p.n0 ? col : col - p.n0) % p.D) >> 3;
    const uint2 cv = __ldg(reinterpret_cast<const uint2*>(p.rope_cos + (int64_t)s * (p.D / 2) + d8 * 4));
    const uint2 sv = __ldg(reinterpret_cast<const uint2*>(p.rope_sin + (int64_t)s * (p.D / 2) + d8 * 4));
    v.x = rope_word(v.x, cv.x & 0xffffu, (sv.x & 0xffffu) ^ 0x8000u);
    v.y = rope_word(v.y, cv.x >> 16, (sv.x >> 16) ^ 0x8000u);
    v.z = rope_word(v.z, cv.y & 0xffffu, (sv.y & 0xffffu) ^ 0x8000u);
    v.w = rope_word(v.w, cv.y >> 16, (sv.y >> 16) ^ 0x8000u);
  }
  return v;
}

// amax of the rotated gradient matrix (the values the tile kernel will stage), eight features per thread and step
__global__ void __launch_bounds__(256) grads_amax_kernel(const Nvfp4Params p, float* __restrict__ amax) {
  const int64_t per_row = p.cols / 8, n_chunks = p.rows * per_row;
  __nv_bfloat162 acc = __float2bfloat162_rn(0.f);
  for (int64_t c = (int64_t)blockIdx.x * 256 + threadIdx.x; c < n_chunks; c += (int64_t)gridDim.x * 256) {
    const uint4 v = load_grad_chunk(p, c / per_row, (c % per_row) * 8);
    acc = absmax2(absmax2(absmax2(absmax2(acc, v.x), v.y), v.z), v.w);
  }
  float m = warp_max(fmaxf(__bfloat162float(acc.x), __bfloat162float(acc.y)));
  __shared__ float wm[8];
  if ((threadIdx.x & 31) == 0) wm[threadIdx.x >> 5] = m;
  __syncthreads();
  if (threadIdx.x < 32) {
    m = warp_max(threadIdx.x < 8 ? wm[threadIdx.x] : 0.f);
    if (threadIdx.x == 0) atomicMax(reinterpret_cast<int*>(amax), __float_as_int(m));
  }
}

// W2D: one scale per 16 x 16 tile (learned projection weights): every 1 x 16 group of the tile, in either
// orientation, carries the scale of the tile's amax, so the transposed output is the byte-for-byte transpose of
// the row-wise one.
// STAGE: what the tile is as it lands in shared memory -- the matrix itself (a TMA load), the RMSNorm of it, or the
// [dQ | dK | dV] gradient matrix gathered from three tensors with the inverse rotation applied (both through
// registers).
enum { kStagePlain = 0, kStageNorm = 1, kStageGrads = 2 };

// Shared memory of one 128 x 128 tile.  Every buffer that a TMA copy touches carries the swizzle of its tensor map,
// and the thread mappings below are chosen so that each warp-wide access meets every bank at most once (twice for
// the 8-byte writes of transposed codes).
struct TileSmem {
  alignas(1024) uint8_t tile[2][128 * 128];  // bf16 columns [0, 64) and [64, 128): 128-byte rows, 128B swizzle
  alignas(1024) uint8_t out_row[128 * 64];   // row-wise codes: a 64-byte row per tile row, 64B swizzle
  alignas(1024) uint8_t out_col[128 * 64];   // transposed codes: a 64-byte row per tile column, 64B swizzle
  alignas(16) uint8_t sc_row[2 * 512];
  alignas(16) uint8_t sc_col[2 * 512];
  union {
    StepTable steps;        // decode-centric recipes: division table of this tensor's global scale
    EncodeTable enc_steps;  // encode-centric recipe: multiplier table
  };
  float tile_amax[64];
  alignas(8) uint64_t bar;
  volatile uint32_t abort_flag;
};
constexpr int kTileSmemBytes = (int)sizeof(TileSmem) + 1024;

// status of the quantizer kernels' waits (word 0 != 0: a tile load did not arrive; words 1-3 as in the attention kernels)
__device__ uint32_t g_quant_status[4];

// The buffers one tile is worked in.
struct TileBuffers {
  const uint8_t* tile0;    // bf16 columns [0, 64): 128-byte rows, 128B swizzle
  const uint8_t* tile1;    // bf16 columns [64, 128)
  uint8_t* out_row;        // row-wise codes: a 64-byte row per tile row, 64B swizzle
  uint8_t* out_col;        // transposed codes: a 64-byte row per tile column, 64B swizzle
  uint8_t* sc_row;         // two scale pages of the row-wise codes
  uint8_t* sc_col;         // two scale pages of the transposed codes
  const StepTable* steps;
  const EncodeTable* enc_steps;
  float* tile_amax;        // W2D: amax of the 64 16 x 16 tiles
};

// W2D: amax of every 16 x 16 tile of the staged tile, four threads per tile, four rows each (ends with a block-wide barrier)
__device__ __forceinline__ void tile_amax_pass(const TileBuffers& tb, int t) {
  const int id = t >> 2, r0 = (id >> 3) * 16 + (t & 3) * 4, c0 = (id & 7) * 16;
  uint32_t m2 = 0;
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    const uint8_t* half = ((c0 >> 6) ? tb.tile1 : tb.tile0);
    const uint4 a = *reinterpret_cast<const uint4*>(half + swizzled_offset((uint32_t)(r0 + k), (uint32_t)(c0 & 63) * 2u, 128));
    const uint4 b = *reinterpret_cast<const uint4*>(half + swizzled_offset((uint32_t)(r0 + k), (uint32_t)(c0 & 63) * 2u + 16u, 128));
    m2 = absmax_bf16x2(absmax_bf16x2(absmax_bf16x2(absmax_bf16x2(m2, a.x), a.y), a.z), a.w);
    m2 = absmax_bf16x2(absmax_bf16x2(absmax_bf16x2(absmax_bf16x2(m2, b.x), b.y), b.z), b.w);
  }
  float m = fmaxf(bf16_bits_to_f32(m2 & 0xffffu), bf16_bits_to_f32(m2 >> 16));
  m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 1));
  m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 2));
  if ((t & 3) == 0) tb.tile_amax[id] = m;
  __syncthreads();
}

// Row pass and column pass of one staged tile: codes and scale pages into the shared-memory buffers.
template <bool COL, bool W2D, bool ENC>
__device__ __forceinline__ void tile_passes(const TileBuffers& tb, int t, float g, float inv6g, float s_enc) {
  // ---- row-wise 1x16 blocks: a thread takes half a row (four blocks of one 128-byte swizzled row).  The 32 lanes of a
  // warp are 32 consecutive rows, so the eight lanes of a quarter warp read eight different 16-byte chunks.
  {
    const int r = t & 127, half = t >> 7;
    const uint8_t* src = ((half) ? tb.tile1 : tb.tile0) + r * 128;
    uint32_t sword = 0;
#pragma unroll
    for (int i = 0; i < 2; ++i) {  // 32 columns (two blocks) at a time
      uint32_t w[16];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const uint4 v = *reinterpret_cast<const uint4*>(src + (((4 * i + j) ^ (r & 7)) << 4));
        w[4 * j] = v.x; w[4 * j + 1] = v.y; w[4 * j + 2] = v.z; w[4 * j + 3] = v.w;
      }
      uint32_t codes[4];
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        float m = 0.f;
        uint64_t x[8];
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          x[k] = bf16x2_to_f32x2(w[8 * h + k]);
          if (!W2D) m = absmax3(m, x[k]);  // on the unpacked values: one three-input maximum per pair
        }
        const int kb = half * 4 + 2 * i + h;
        const float bamax = W2D ? tb.tile_amax[(r >> 4) * 8 + kb] : m;
        uint32_t sbyte;
        if (ENC) {
          nvfp4_codes16_encode(x, bamax, s_enc, (*tb.enc_steps), sbyte, codes[2 * h], codes[2 * h + 1]);
        } else {
          sbyte = nvfp4_scale_byte(bamax, g, inv6g);
          nvfp4_codes16(x, bamax, (*tb.steps), sbyte, codes[2 * h], codes[2 * h + 1]);
        }
        sword |= sbyte << (8 * (2 * i + h));
      }
      *reinterpret_cast<uint4*>(&tb.out_row[swizzled_offset((uint32_t)r, (uint32_t)(half * 32 + i * 16), 64)]) =
          make_uint4(codes[0], codes[1], codes[2], codes[3]);
    }
    // the four scale bytes of this half row are one aligned word of page `half`
    *reinterpret_cast<uint32_t*>(&tb.sc_row[half * 512 + page_offset(r, 0)]) = sword;
  }
  // ---- column-wise 16x1 blocks (transposed output): a thread takes two adjacent columns (one 32-bit word per tile
  // row) and two consecutive blocks of 16 rows; the 32 lanes of a warp read 32 consecutive words of a row
  if (COL) {
    const int cp = t & 63, rb0 = (t >> 6) * 2;
    const uint8_t* src = ((cp >> 5) ? tb.tile1 : tb.tile0) + (cp & 3) * 4;
    uint32_t xoff[8];  // the 16-byte chunk of this column pair in a row with (row & 7) == j
#pragma unroll
    for (int j = 0; j < 8; ++j) xoff[j] = (uint32_t)((((cp & 31) >> 2) ^ j) << 4);
    uint32_t spair[2] = {0, 0};
    uint32_t ccodes[2][4];  // per column: the 32 rows of this thread's two blocks, 16 bytes
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const int rb = rb0 + i;
      uint32_t w[16];
#pragma unroll
      for (int k = 0; k < 16; ++k) w[k] = *reinterpret_cast<const uint32_t*>(src + (rb * 16 + k) * 128 + xoff[k & 7]);
#pragma unroll
      for (int h = 0; h < 2; ++h) {  // low halves: column 2cp, high halves: column 2cp + 1
        const int c = 2 * cp + h;
        uint64_t x[8];
        float m = 0.f;
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          x[k] = h ? pack2u(w[2 * k] & 0xFFFF0000u, w[2 * k + 1] & 0xFFFF0000u) : pack2u(w[2 * k] << 16, w[2 * k + 1] << 16);
          if (!W2D) m = absmax3(m, x[k]);
        }
        const float bamax = W2D ? tb.tile_amax[rb * 8 + (c >> 4)] : m;
        uint32_t lo, hi, sbyte;
        if (ENC) {
          nvfp4_codes16_encode(x, bamax, s_enc, (*tb.enc_steps), sbyte, lo, hi);
        } else {
          sbyte = nvfp4_scale_byte(bamax, g, inv6g);
          nvfp4_codes16(x, bamax, (*tb.steps), sbyte, lo, hi);
        }
        ccodes[h][2 * i] = lo;
        ccodes[h][2 * i + 1] = hi;
        spair[h] |= sbyte << (8 * i);
      }
    }
    // transposed tensor: row = c (within this tile's 128 columns), kblock = rb (within 8); two consecutive blocks
    // are two adjacent bytes of a page
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      *reinterpret_cast<uint4*>(&tb.out_col[swizzled_offset((uint32_t)(2 * cp + h), (uint32_t)rb0 * 8u, 64)]) =
          make_uint4(ccodes[h][0], ccodes[h][1], ccodes[h][2], ccodes[h][3]);
      *reinterpret_cast<uint16_t*>(&tb.sc_col[(rb0 >> 2) * 512 + page_offset(2 * cp + h, rb0)]) = (uint16_t)spair[h];
    }
  }}

template <int STAGE, bool COL, bool W2D = false, bool ENC = false>
__global__ void __launch_bounds__(256, 4) nvfp4_tile_kernel(const Nvfp4Params p, const __grid_constant__ CUtensorMap map_x,
                                                         const __grid_constant__ CUtensorMap map_row, const __grid_constant__ CUtensorMap map_col) {
  extern __shared__ uint8_t tile_smem_raw[];
  TileSmem& s = *reinterpret_cast<TileSmem*>(tile_smem_raw + ((1024u - (smem_u32(tile_smem_raw) & 1023u)) & 1023u));

  const int t = threadIdx.x;
  // tiles run from the end of the matrix to its start: the statistics pass that precedes this kernel
  // read the matrix front to back, so its last part is the part still in L2
  const int64_t row0 = (int64_t)(gridDim.y - 1 - blockIdx.y) * kTile, col0 = (int64_t)(gridDim.x - 1 - blockIdx.x) * kTile;
  if (STAGE == kStagePlain && t == 0) {
    s.abort_flag = 0u;
    mbar_init(&s.bar, 1);
    fence_barrier_init();
    mbar_expect_tx(&s.bar, 2 * 128 * 128);
    tma_load_2d(s.tile[0], &map_x, (int)col0, (int)row0, &s.bar);
    tma_load_2d(s.tile[1], &map_x, (int)col0 + 64, (int)row0, &s.bar);
  }
  const float amax = *p.amax;
  const float g = amax / kNvfp4GlobalDiv;
  const bool all_zero = !(amax > 0.f);
  const float inv6g = all_zero ? 0.f : 1.0f / (6.0f * g);  // an all-zero tensor: every scale byte and code 0
  // encode-centric recipe: S_enc = 2688 / amax, 1 for an all-zero tensor (core.cuh:103-113)
  float s_enc = fminf(kNvfp4GlobalDiv / amax, 3.4028235e38f);
  if (amax == 0.f || s_enc == 0.f) s_enc = 1.0f;
  if (blockIdx.x == 0 && blockIdx.y == 0 && t == 0) *p.global_scale = g;
  if (ENC) fill_encode_table(s.enc_steps, s_enc, t);
  else fill_step_table(s.steps, g, t);

  // ---- stage the tile -----------------------------------------------------------
  if (STAGE != kStagePlain) {
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int chunk = t + i * 256;  // 2048 chunks of 8 bf16
      const int r = chunk >> 4, c8 = (chunk & 15) * 8;
      uint4 v;
      if (STAGE == kStageGrads) {
        v = load_grad_chunk(p, row0 + r, col0 + c8);
      } else {
        v = __ldg(reinterpret_cast<const uint4*>(p.x + (row0 + r) * p.ld + col0 + c8));
        const float inv = __ldg(p.inv_rms + row0 + r);
        const uint4 gv = __ldg(reinterpret_cast<const uint4*>(p.gamma + col0 + c8));
        uint32_t w[4] = {v.x, v.y, v.z, v.w};
        const uint32_t gw[4] = {gv.x, gv.y, gv.z, gv.w};
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          const float a = (bf16_bits_to_f32(w[k] & 0xffffu) * inv) * bf16_bits_to_f32(gw[k] & 0xffffu);
          const float b = (bf16_bits_to_f32(w[k] >> 16) * inv) * bf16_bits_to_f32(gw[k] >> 16);
          const __nv_bfloat162 y = __floats2bfloat162_rn(a, b);
          w[k] = *reinterpret_cast<const uint32_t*>(&y);
        }
        v = make_uint4(w[0], w[1], w[2], w[3]);
        if (p.y_out) *reinterpret_cast<uint4*>(p.y_out + (row0 + r) * p.cols + col0 + c8) = v;
      }
      *reinterpret_cast<uint4*>(&s.tile[c8 >> 6][swizzled_offset((uint32_t)r, (uint32_t)(c8 & 63) * 2u, 128)]) = v;
    }
  }
  __syncthreads();  // tables (and the staged tile, or the barrier's initialisation) visible
  if (STAGE == kStagePlain) {
    if (!mbar_wait(&s.bar, 0, &s.abort_flag, g_quant_status, 1, (uint32_t)blockIdx.y)) {
      if (t == 0) mbar_wait_teardown(&s.bar, 0);  // the copies may still be on their way into this CTA's memory
      __syncthreads();
      return;
    }
  }
  TileBuffers tb;
  tb.tile0 = s.tile[0]; tb.tile1 = s.tile[1];
  tb.out_row = s.out_row; tb.out_col = s.out_col; tb.sc_row = s.sc_row; tb.sc_col = s.sc_col;
  tb.steps = &s.steps; tb.enc_steps = &s.enc_steps; tb.tile_amax = s.tile_amax;
  if (W2D) tile_amax_pass(tb, t);
  tile_passes<COL, W2D, ENC>(tb, t, g, inv6g, s_enc);
  fence_async_smem();  // the code planes are read by TMA stores
  __syncthreads();
  // ---- codes leave as TMA stores, the scale pages as 16-byte words ------------------------------
  if (t == 0) {
    tma_store_2d(&map_row, s.out_row, (int)(col0 / 2), (int)row0);
    if (COL) tma_store_2d(&map_col, s.out_col, (int)(row0 / 2), (int)col0);
    tma_store_commit();
  } else if (t >= 64 && t < 128) {
    const int u = t - 64;
    const int page = u >> 5, off = (u & 31) * 16;
    uint8_t* dst = p.scales_row + ((row0 / 128) * (p.cols / 64) + col0 / 64 + page) * 512 + off;
    *reinterpret_cast<uint4*>(dst) = *reinterpret_cast<const uint4*>(&s.sc_row[page * 512 + off]);
  } else if (COL && t >= 128 && t < 192) {
    const int u = t - 128;
    const int page = u >> 5, off = (u & 31) * 16;
    uint8_t* dst = p.scales_col + ((col0 / 128) * (p.rows / 64) + row0 / 64 + page) * 512 + off;
    *reinterpret_cast<uint4*>(dst) = *reinterpret_cast<const uint4*>(&s.sc_col[page * 512 + off]);
  }
  if (t == 0) tma_store_wait_read();  // shared memory stays allocated until the stores have read it
}

// ------------------------------------------------------------------ MXFP4
__device__ __forceinline__ int mx_exponent(float bamax, int mode) {
  // bamax > 0 is a bf16 value; returns the unbiased power-of-two exponent of the block scale
  const uint32_t bits = __float_as_uint(fmaxf(bamax, kFltMin));
  const int e = (int)(bits >> 23) - 127;
  const uint32_t man = bits & 0x7fffffu;
  if (mode == FA4B_MX_CEIL) return e + (man != 0);
  if (mode == FA4B_MX_FLOOR) return e;
  // mantissa round-to-nearest, a tie keeps an even biased exponent
  const bool up = man > 0x400000u || (man == 0x400000u && ((e + 127) & 1));
  return e + up;
}

__global__ void __launch_bounds__(256) mxfp4_kernel(const __nv_bfloat16* __restrict__ x, int64_t ld, int64_t rows, int64_t cols,
                                                    int mode, uint8_t* __restrict__ codes, uint8_t* __restrict__ scales) {
  const int64_t kblocks = cols / 32;
  const int64_t idx = (int64_t)blockIdx.x * 256 + threadIdx.x;
  const bool live = idx < rows * kblocks;
  const int64_t row = live ? idx / kblocks : 0, kb = live ? idx % kblocks : 0;
  uint32_t w[16];
  uint32_t m2 = 0;
  const uint4* src = reinterpret_cast<const uint4*>(x + row * ld + kb * 32);
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const uint4 v = live ? __ldg(src + j) : make_uint4(0, 0, 0, 0);
    w[4 * j] = v.x; w[4 * j + 1] = v.y; w[4 * j + 2] = v.z; w[4 * j + 3] = v.w;
  }
#pragma unroll
  for (int k = 0; k < 16; ++k) m2 = absmax_bf16x2(m2, w[k]);
  const float bamax = fmaxf(bf16_bits_to_f32(m2 & 0xffffu), bf16_bits_to_f32(m2 >> 16));
  uint32_t packed[4] = {0, 0, 0, 0};
  uint32_t ebyte = 0;
  if (bamax > 0.f) {
    const int e = max(mx_exponent(bamax, mode), -126);
    ebyte = (uint32_t)min(e + 127, 254);
    // step d = RN(2^e / 6) (significand 0x2AAAAB, never all ones); q = RN(x / d) through r = RN(1 / d)
    const float d = fmaxf(__uint_as_float((uint32_t)(e + 127) << 23) / 6.0f, kFltMin);
    const float r = __frcp_rn(d);
    const uint64_t r2 = pack2(r, r), nd2 = pack2(-d, -d);
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      uint64_t q[8];
#pragma unroll
      for (int k = 0; k < 8; ++k) q[k] = div2_exact(bf16x2_to_f32x2(w[8 * h + k]), r2, nd2);
      e2m1_pack16(q, packed[2 * h], packed[2 * h + 1]);
    }
  }
  if (live) *reinterpret_cast<uint4*>(codes + row * (cols / 2) + kb * 16) = make_uint4(packed[0], packed[1], packed[2], packed[3]);
  // the four blocks of a 128-column page row are held by four adjacent lanes
  uint32_t quad = ebyte << (8 * (threadIdx.x & 3));
  quad |= __shfl_xor_sync(0xffffffffu, quad, 1);
  quad |= __shfl_xor_sync(0xffffffffu, quad, 2);
  if (live && (threadIdx.x & 3) == 0) {
    uint8_t* page = scales + ((row / 128) * (cols / 128) + kb / 4) * 512;
    *reinterpret_cast<uint32_t*>(page + page_offset((uint32_t)row, 0)) = quad;
  }
}

// ------------------------------------------------------------------ decode utilities
__global__ void dequant_kernel(const uint8_t* __restrict__ codes, const uint8_t* __restrict__ pages, const float* g,
                               int64_t rows, int64_t cols, int block, float* __restrict__ out) {
  const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= rows * cols) return;
  const int64_t r = idx / cols, c = idx % cols;
  const uint32_t byte = codes[r * (cols / 2) + c / 2];
  const uint32_t code = (c & 1) ? (byte >> 4) : (byte & 15u);
  const int64_t kb = c / block;
  const uint32_t s = pages[((r / 128) * (cols / (4 * block)) + kb / 4) * 512 + page_offset((uint32_t)r, (uint32_t)kb)];
  float d;
  if (block == 16) d = e4m3_to_f32(s) * *g;
  else d = s ? __uint_as_float(s << 23) / 6.0f : 0.f;
  out[idx] = e2m1_to_f32(code) * d;
}

static int check_matrix(const void* x, int64_t rows, int64_t cols, int64_t ld) {
  FA4B_REQUIRE(x != nullptr, FA4B_BAD_ARG, "input pointer is NULL");
  FA4B_REQUIRE(rows > 0 && cols > 0 && rows % 128 == 0 && cols % 128 == 0, FA4B_BAD_SHAPE,
               "rows=%lld cols=%lld must be positive multiples of 128", (long long)rows, (long long)cols);
  FA4B_REQUIRE(ld >= cols && ld % 8 == 0, FA4B_BAD_ALIGN, "row stride %lld must be >= cols and a multiple of 8 elements", (long long)ld);
  FA4B_REQUIRE((reinterpret_cast<uintptr_t>(x) & 15) == 0, FA4B_BAD_ALIGN, "input must be 16-byte aligned");
  return FA4B_OK;
}

}  // namespace fa4b

using namespace fa4b;

struct TileMaps {
  CUtensorMap x, row, col;
};
template <int STAGE, bool COL, bool W2D, bool ENC>
static int launch_nvfp4_kernel(const Nvfp4Params& p, const TileMaps& m, dim3 grid, cudaStream_t st) {
  FA4B_CUDA(cudaFuncSetAttribute(nvfp4_tile_kernel<STAGE, COL, W2D, ENC>, cudaFuncAttributeMaxDynamicSharedMemorySize, kTileSmemBytes));
  nvfp4_tile_kernel<STAGE, COL, W2D, ENC><<<grid, 256, kTileSmemBytes, st>>>(p, m.x, m.row, m.col);
  return FA4B_OK;
}
template <int STAGE, bool W2D>
static int launch_nvfp4_stage(const Nvfp4Params& p, const TileMaps& m, dim3 grid, cudaStream_t st) {
  const bool col = p.codes_col != nullptr, enc = !W2D && p.recipe == FA4B_RECIPE_ENCODE_CENTRIC;
  if (col) return enc ? launch_nvfp4_kernel<STAGE, true, W2D, !W2D>(p, m, grid, st) : launch_nvfp4_kernel<STAGE, true, W2D, false>(p, m, grid, st);
  return enc ? launch_nvfp4_kernel<STAGE, false, W2D, !W2D>(p, m, grid, st) : launch_nvfp4_kernel<STAGE, false, W2D, false>(p, m, grid, st);
}
// The tensor maps of one call: the bf16 matrix in boxes of 64 columns x 128 rows (plain staging only), the two code
// planes in boxes of 64 bytes x 128 rows.
static int launch_nvfp4(const Nvfp4Params& p, int stage, cudaStream_t st, bool weight_tiles = false) {
  dim3 grid((unsigned)(p.cols / 128), (unsigned)(p.rows / 128));
  TileMaps m;
  if (int s = make_tensor_map(&m.row, p.codes_row, 1, (uint64_t)p.cols / 2, (uint64_t)p.rows, 0, (uint64_t)p.cols / 2, 0, 64, 128)) return s;
  m.col = m.row;
  m.x = m.row;
  if (p.codes_col)
    if (int s = make_tensor_map(&m.col, p.codes_col, 1, (uint64_t)p.rows / 2, (uint64_t)p.cols, 0, (uint64_t)p.rows / 2, 0, 64, 128)) return s;
  if (stage == kStagePlain)
    if (int s = make_tensor_map(&m.x, p.x, 2, (uint64_t)p.cols, (uint64_t)p.rows, 0, (uint64_t)p.ld * 2, 0, 64, 128)) return s;
  int r;
  if (weight_tiles) r = launch_nvfp4_stage<kStagePlain, true>(p, m, grid, st);
  else if (stage == kStageNorm) r = launch_nvfp4_stage<kStageNorm, false>(p, m, grid, st);
  else if (stage == kStageGrads) r = launch_nvfp4_stage<kStageGrads, false>(p, m, grid, st);
  else r = launch_nvfp4_stage<kStagePlain, false>(p, m, grid, st);
  if (r) return r;
  FA4B_CUDA(cudaGetLastError());
  return FA4B_OK;
}

extern "C" {

const char* fa4b_last_error(void) { return fa4b::last_error(); }

const char* fa4b_status_string(int s) {
  switch (s) {
    case FA4B_OK: return "ok";
    case FA4B_BAD_SHAPE: return "bad shape";
    case FA4B_BAD_ALIGN: return "bad alignment";
    case FA4B_UNSUPPORTED: return "unsupported";
    case FA4B_CUDA_ERROR: return "CUDA error";
    case FA4B_TIMEOUT: return "device wait timed out";
    case FA4B_BAD_ARG: return "bad argument";
    default: return "unknown status";
  }
}

int fa4b_amax(const void* x, int64_t n, float* amax, void* stream) {
  FA4B_REQUIRE(x && amax && n > 0, FA4B_BAD_ARG, "fa4b_amax: NULL pointer or n <= 0");
  FA4B_REQUIRE((reinterpret_cast<uintptr_t>(x) & 15) == 0, FA4B_BAD_ALIGN, "fa4b_amax: input must be 16-byte aligned");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  FA4B_CUDA(cudaMemsetAsync(amax, 0, sizeof(float), st));
  const int64_t n_vec = n / 8;
  const int n_tail = (int)(n % 8);
  const int grid = (int)std::min<int64_t>((int64_t)std::max(sm_count(), 1) * 8, std::max<int64_t>(1, (n_vec + 255) / 256));
  amax_kernel<<<grid, 256, 0, st>>>(static_cast<const uint4*>(x), n_vec, static_cast<const __nv_bfloat16*>(x) + n_vec * 8, n_tail, amax);
  FA4B_CUDA(cudaGetLastError());
  return FA4B_OK;
}

static int quant_nvfp4_impl(const fa4b_quant_nvfp4_args* a, void* stream, bool weight_tiles) {
  FA4B_REQUIRE(a != nullptr, FA4B_BAD_ARG, "args is NULL");
  if (int s = check_matrix(a->x, a->rows, a->cols, a->ld)) return s;
  FA4B_REQUIRE(a->amax && a->global_scale && a->codes_row && a->scales_row, FA4B_BAD_ARG, "fa4b_quant_nvfp4: an output pointer is NULL");
  FA4B_REQUIRE((a->codes_col == nullptr) == (a->scales_col == nullptr), FA4B_BAD_ARG, "codes_col and scales_col go together");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (!a->amax_is_input) {
    FA4B_REQUIRE(a->ld == a->cols, FA4B_UNSUPPORTED, "computing amax needs a dense matrix (ld == cols); pass amax_is_input");
    if (int s = fa4b_amax(a->x, a->rows * a->cols, a->amax, stream)) return s;
  }
  Nvfp4Params p{};
  p.x = static_cast<const __nv_bfloat16*>(a->x);
  p.ld = a->ld; p.rows = a->rows; p.cols = a->cols;
  p.amax = a->amax; p.global_scale = a->global_scale;
  p.codes_row = a->codes_row; p.scales_row = a->scales_row;
  p.codes_col = a->codes_col; p.scales_col = a->scales_col;
  FA4B_REQUIRE(a->recipe == FA4B_RECIPE_DECODE_CENTRIC || (a->recipe == FA4B_RECIPE_ENCODE_CENTRIC && !weight_tiles), FA4B_UNSUPPORTED,
               "recipe %d (the 16 x 16 weight recipe is decode-centric only)", a->recipe);
  p.recipe = a->recipe;
  return launch_nvfp4(p, kStagePlain, st, weight_tiles);
}

int fa4b_quant_nvfp4(const fa4b_quant_nvfp4_args* a, void* stream) { return quant_nvfp4_impl(a, stream, false); }

int fa4b_quant_check_status(void* stream) {
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  uint32_t host[4] = {0, 0, 0, 0};
  FA4B_CUDA(cudaMemcpyFromSymbolAsync(host, g_quant_status, sizeof(host), 0, cudaMemcpyDeviceToHost, st));
  FA4B_CUDA(cudaStreamSynchronize(st));
  if (host[0] == 0) return FA4B_OK;
  const uint32_t zero[4] = {0, 0, 0, 0};
  FA4B_CUDA(cudaMemcpyToSymbolAsync(g_quant_status, zero, sizeof(zero), 0, cudaMemcpyHostToDevice, st));
  FA4B_CUDA(cudaStreamSynchronize(st));
  set_error("a quantizer tile load did not arrive within the wait limit (site %u, block %u, tile row %u)", host[1], host[2], host[3]);
  return FA4B_TIMEOUT;
}

int fa4b_quant_nvfp4_weight(const fa4b_quant_nvfp4_args* a, void* stream) { return quant_nvfp4_impl(a, stream, true); }

int fa4b_pack_qkv_grads(const fa4b_pack_qkv_grads_args* a, void* stream) {
  FA4B_REQUIRE(a != nullptr, FA4B_BAD_ARG, "args is NULL");
  FA4B_REQUIRE(a->dq && a->dk && a->dv && a->rope_cos && a->rope_sin, FA4B_BAD_ARG, "fa4b_pack_qkv_grads: an input pointer is NULL");
  FA4B_REQUIRE(a->amax && a->global_scale && a->codes_row && a->scales_row, FA4B_BAD_ARG, "fa4b_pack_qkv_grads: an output pointer is NULL");
  FA4B_REQUIRE((a->codes_col == nullptr) == (a->scales_col == nullptr), FA4B_BAD_ARG, "codes_col and scales_col go together");
  FA4B_REQUIRE(a->B > 0 && a->S > 0 && a->Hq > 0 && a->Hkv > 0 && (a->D == 64 || a->D == 128), FA4B_BAD_SHAPE,
               "B, S, Hq, Hkv must be positive and D 64 or 128");
  const int64_t rows = a->B * a->S, n0 = a->Hq * a->D, n1 = n0 + a->Hkv * a->D, cols = n1 + a->Hkv * a->D;
  FA4B_REQUIRE(rows % 128 == 0 && cols % 128 == 0, FA4B_BAD_SHAPE, "B*S=%lld and (Hq+2Hkv)*D=%lld must be multiples of 128", (long long)rows,
               (long long)cols);
  FA4B_REQUIRE(a->ld_q >= n0 && a->ld_k >= n1 - n0 && a->ld_v >= cols - n1 && (a->ld_q | a->ld_k | a->ld_v) % 8 == 0, FA4B_BAD_ALIGN,
               "row strides must cover a token's heads and be multiples of 8 elements");
  FA4B_REQUIRE(((reinterpret_cast<uintptr_t>(a->dq) | reinterpret_cast<uintptr_t>(a->dk) | reinterpret_cast<uintptr_t>(a->dv) |
                 reinterpret_cast<uintptr_t>(a->codes_row) | reinterpret_cast<uintptr_t>(a->scales_row) | reinterpret_cast<uintptr_t>(a->codes_col) |
                 reinterpret_cast<uintptr_t>(a->scales_col)) & 15) == 0 &&
                   ((reinterpret_cast<uintptr_t>(a->rope_cos) | reinterpret_cast<uintptr_t>(a->rope_sin)) & 7) == 0,
               FA4B_BAD_ALIGN, "gradients and outputs must be 16-byte aligned, rope tables 8-byte aligned");
  FA4B_REQUIRE(a->recipe == FA4B_RECIPE_DECODE_CENTRIC || a->recipe == FA4B_RECIPE_ENCODE_CENTRIC, FA4B_UNSUPPORTED, "recipe %d", a->recipe);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  Nvfp4Params p{};
  p.x = static_cast<const __nv_bfloat16*>(a->dq); p.x1 = static_cast<const __nv_bfloat16*>(a->dk); p.x2 = static_cast<const __nv_bfloat16*>(a->dv);
  p.ld = a->ld_q; p.ld1 = a->ld_k; p.ld2 = a->ld_v;
  p.n0 = n0; p.n1 = n1; p.rows = rows; p.cols = cols;
  p.rope_cos = static_cast<const __nv_bfloat16*>(a->rope_cos); p.rope_sin = static_cast<const __nv_bfloat16*>(a->rope_sin);
  p.S = (int)a->S; p.D = (int)a->D;
  p.amax = a->amax; p.global_scale = a->global_scale;
  p.codes_row = a->codes_row; p.scales_row = a->scales_row;
  p.codes_col = a->codes_col; p.scales_col = a->scales_col;
  p.recipe = a->recipe;
  if (!a->amax_is_input) {
    FA4B_CUDA(cudaMemsetAsync(a->amax, 0, sizeof(float), st));
    const int grid = (int)std::min<int64_t>((int64_t)std::max(sm_count(), 1) * 8, (rows * (cols / 8) + 255) / 256);
    grads_amax_kernel<<<grid, 256, 0, st>>>(p, a->amax);
    FA4B_CUDA(cudaGetLastError());
  }
  return launch_nvfp4(p, kStageGrads, st);
}

int fa4b_rmsnorm_quant_nvfp4(const fa4b_rmsnorm_quant_nvfp4_args* a, void* stream) {
  FA4B_REQUIRE(a != nullptr, FA4B_BAD_ARG, "args is NULL");
  if (int s = check_matrix(a->x, a->rows, a->cols, a->ld)) return s;
  FA4B_REQUIRE(a->gamma && a->inv_rms && a->amax && a->global_scale && a->codes_row && a->scales_row, FA4B_BAD_ARG,
               "fa4b_rmsnorm_quant_nvfp4: a required pointer is NULL");
  FA4B_REQUIRE((a->codes_col == nullptr) == (a->scales_col == nullptr), FA4B_BAD_ARG, "codes_col and scales_col go together");
  FA4B_REQUIRE(a->cols <= 8 * 256 * 8, FA4B_BAD_SHAPE, "cols=%lld exceeds the 16384-column limit of the row-statistics kernel", (long long)a->cols);
  FA4B_REQUIRE((reinterpret_cast<uintptr_t>(a->gamma) & 15) == 0, FA4B_BAD_ALIGN, "gamma must be 16-byte aligned");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  FA4B_CUDA(cudaMemsetAsync(a->amax, 0, sizeof(float), st));
  const auto* x = static_cast<const __nv_bfloat16*>(a->x);
  const auto* gm = static_cast<const __nv_bfloat16*>(a->gamma);
  const int vec = (int)((a->cols / 8 + 255) / 256);
  const unsigned rows = (unsigned)a->rows;
  if (vec <= 1) rmsnorm_stats_kernel<1><<<rows, 256, 0, st>>>(x, a->ld, (int)a->cols, gm, a->eps, a->inv_rms, a->amax);
  else if (vec <= 2) rmsnorm_stats_kernel<2><<<rows, 256, 0, st>>>(x, a->ld, (int)a->cols, gm, a->eps, a->inv_rms, a->amax);
  else if (vec <= 4) rmsnorm_stats_kernel<4><<<rows, 256, 0, st>>>(x, a->ld, (int)a->cols, gm, a->eps, a->inv_rms, a->amax);
  else rmsnorm_stats_kernel<8><<<rows, 256, 0, st>>>(x, a->ld, (int)a->cols, gm, a->eps, a->inv_rms, a->amax);
  FA4B_CUDA(cudaGetLastError());
  Nvfp4Params p{};
  p.x = x; p.ld = a->ld; p.rows = a->rows; p.cols = a->cols;
  p.gamma = gm; p.inv_rms = a->inv_rms; p.y_out = static_cast<__nv_bfloat16*>(a->y_out);
  p.amax = a->amax; p.global_scale = a->global_scale;
  p.codes_row = a->codes_row; p.scales_row = a->scales_row;
  p.codes_col = a->codes_col; p.scales_col = a->scales_col;
  FA4B_REQUIRE(a->recipe == FA4B_RECIPE_DECODE_CENTRIC || a->recipe == FA4B_RECIPE_ENCODE_CENTRIC, FA4B_UNSUPPORTED, "recipe %d", a->recipe);
  p.recipe = a->recipe;
  return launch_nvfp4(p, kStageNorm, st);
}

size_t fa4b_rmsnorm_bwd_workspace_bytes(int64_t cols) { return cols > 0 ? (size_t)kRmsBwdParts * (size_t)cols * sizeof(float) : 0; }

int fa4b_rmsnorm_bwd(const fa4b_rmsnorm_bwd_args* a, void* stream) {
  FA4B_REQUIRE(a != nullptr, FA4B_BAD_ARG, "args is NULL");
  FA4B_REQUIRE(a->x && a->gamma && a->inv_rms && a->dy && a->dx && a->dgamma && a->partials, FA4B_BAD_ARG, "fa4b_rmsnorm_bwd: NULL pointer");
  FA4B_REQUIRE(a->rows > 0 && a->cols > 0 && a->cols % 8 == 0 && a->cols <= 8 * 256 * 4, FA4B_BAD_SHAPE,
               "rows=%lld cols=%lld: cols must be a multiple of 8 up to 8192", (long long)a->rows, (long long)a->cols);
  FA4B_REQUIRE(a->ld >= a->cols && a->ld_dy >= a->cols && a->ld % 8 == 0 && a->ld_dy % 8 == 0, FA4B_BAD_ALIGN,
               "row strides must be >= cols and multiples of 8 elements");
  FA4B_REQUIRE(((reinterpret_cast<uintptr_t>(a->x) | reinterpret_cast<uintptr_t>(a->dy) | reinterpret_cast<uintptr_t>(a->gamma) |
                 reinterpret_cast<uintptr_t>(a->dx) | reinterpret_cast<uintptr_t>(a->partials)) & 15) == 0,
               FA4B_BAD_ALIGN, "fa4b_rmsnorm_bwd: 16-byte alignment");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const auto* x = static_cast<const __nv_bfloat16*>(a->x);
  const auto* gm = static_cast<const __nv_bfloat16*>(a->gamma);
  const auto* dy = static_cast<const __nv_bfloat16*>(a->dy);
  auto* dx = static_cast<__nv_bfloat16*>(a->dx);
  const int cols = (int)a->cols;
  const int n_parts = (int)std::min<int64_t>(a->rows, std::min(kRmsBwdParts, 2 * std::max(sm_count(), 1)));
  const int vec = (int)((a->cols / 8 + 255) / 256);
  if (vec <= 1) rmsnorm_bwd_kernel<1><<<n_parts, 256, 0, st>>>(x, a->ld, gm, a->inv_rms, dy, a->ld_dy, a->rows, cols, dx, a->partials);
  else if (vec <= 2) rmsnorm_bwd_kernel<2><<<n_parts, 256, 0, st>>>(x, a->ld, gm, a->inv_rms, dy, a->ld_dy, a->rows, cols, dx, a->partials);
  else rmsnorm_bwd_kernel<4><<<n_parts, 256, 0, st>>>(x, a->ld, gm, a->inv_rms, dy, a->ld_dy, a->rows, cols, dx, a->partials);
  FA4B_CUDA(cudaGetLastError());
  rmsnorm_bwd_reduce_kernel<<<(cols + 255) / 256, 256, 0, st>>>(a->partials, n_parts, cols, static_cast<__nv_bfloat16*>(a->dgamma));
  FA4B_CUDA(cudaGetLastError());
  return FA4B_OK;
}

int fa4b_quant_mxfp4(const fa4b_quant_mxfp4_args* a, void* stream) {
  FA4B_REQUIRE(a != nullptr, FA4B_BAD_ARG, "args is NULL");
  if (int s = check_matrix(a->x, a->rows, a->cols, a->ld)) return s;
  FA4B_REQUIRE(a->codes && a->scales, FA4B_BAD_ARG, "fa4b_quant_mxfp4: an output pointer is NULL");
  FA4B_REQUIRE(a->mode >= FA4B_MX_CEIL && a->mode <= FA4B_MX_FLOOR, FA4B_UNSUPPORTED, "unknown MXFP4 scale mode %d", a->mode);
  const int64_t n = a->rows * (a->cols / 32);
  mxfp4_kernel<<<(unsigned)((n + 255) / 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(a->x), a->ld, a->rows, a->cols, a->mode, a->codes, a->scales);
  FA4B_CUDA(cudaGetLastError());
  return FA4B_OK;
}

int fa4b_dequant_nvfp4(const uint8_t* codes, const uint8_t* pages, const float* g, int64_t rows, int64_t cols, float* out, void* stream) {
  FA4B_REQUIRE(codes && pages && g && out, FA4B_BAD_ARG, "fa4b_dequant_nvfp4: NULL pointer");
  FA4B_REQUIRE(rows > 0 && cols > 0 && rows % 128 == 0 && cols % 64 == 0, FA4B_BAD_SHAPE, "rows %% 128 and cols %% 64 must be 0");
  const int64_t n = rows * cols;
  dequant_kernel<<<(unsigned)((n + 255) / 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(codes, pages, g, rows, cols, 16, out);
  FA4B_CUDA(cudaGetLastError());
  return FA4B_OK;
}

int fa4b_dequant_mxfp4(const uint8_t* codes, const uint8_t* pages, int64_t rows, int64_t cols, float* out, void* stream) {
  FA4B_REQUIRE(codes && pages && out, FA4B_BAD_ARG, "fa4b_dequant_mxfp4: NULL pointer");
  FA4B_REQUIRE(rows > 0 && cols > 0 && rows % 128 == 0 && cols % 128 == 0, FA4B_BAD_SHAPE, "rows and cols must be multiples of 128");
  const int64_t n = rows * cols;
  dequant_kernel<<<(unsigned)((n + 255) / 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(codes, pages, nullptr, rows, cols, 32, out);
  FA4B_CUDA(cudaGetLastError());
  return FA4B_OK;
}

}  // extern "C"

// ------------------------------------------------------------------ pair-native RoPE
// x[b, s, h, 2i], x[b, s, h, 2i+1] rotate by the angle whose cosine and sine are cos[s, i], sin[s, i] (bf16), in
// packed BF16 arithmetic: out = fma(perp, sin, mul(pair, cos)) with perp = (-y, x), one rounding each -- the
// arithmetic of apply_rope_pair (tk_fa4/lowp_fa4_bwd/projection_fp4_epilogue.cuh:447-479).  The inverse
// rotation (gradients) negates the sine.  Eight elements per thread, in place.
namespace fa4b {
__global__ void __launch_bounds__(256) rope_pair_kernel(__nv_bfloat16* __restrict__ x, int64_t sb, int64_t ss, int64_t sh, int S, int H, int D,
                                                        int64_t n_chunks, const __nv_bfloat16* __restrict__ cs, const __nv_bfloat16* __restrict__ sn,
                                                        int inverse) {
  const int per_row = D / 8;
  for (int64_t c = (int64_t)blockIdx.x * 256 + threadIdx.x; c < n_chunks; c += (int64_t)gridDim.x * 256) {
    const int d8 = (int)(c % per_row);
    const int64_t row = c / per_row;
    const int h = (int)(row % H);
    const int64_t bs = row / H;
    const int s = (int)(bs % S);
    const int64_t b = bs / S;
    uint4* px = reinterpret_cast<uint4*>(x + b * sb + (int64_t)s * ss + (int64_t)h * sh + d8 * 8);
    const uint2 cv = __ldg(reinterpret_cast<const uint2*>(cs + (int64_t)s * (D / 2) + d8 * 4));
    const uint2 sv = __ldg(reinterpret_cast<const uint2*>(sn + (int64_t)s * (D / 2) + d8 * 4));
    uint4 v = *px;
    uint32_t w[4] = {v.x, v.y, v.z, v.w};
    const uint32_t cw[2] = {cv.x, cv.y}, sw[2] = {sv.x, sv.y};
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const uint32_t c16 = (cw[k >> 1] >> (16 * (k & 1))) & 0xffffu;
      uint32_t s16 = (sw[k >> 1] >> (16 * (k & 1))) & 0xffffu;
      if (inverse) s16 ^= 0x8000u;
      w[k] = rope_word(w[k], c16, s16);
    }
    *px = make_uint4(w[0], w[1], w[2], w[3]);
  }
}
}  // namespace fa4b

int fa4b_rope_pair(const fa4b_rope_pair_args* a, void* stream) {
  FA4B_REQUIRE(a != nullptr && a->x && a->rope_cos && a->rope_sin, FA4B_BAD_ARG, "fa4b_rope_pair: NULL pointer");
  FA4B_REQUIRE(a->B > 0 && a->S > 0 && a->H > 0 && a->D > 0 && a->D % 8 == 0, FA4B_BAD_SHAPE, "B, S, H must be positive and D a positive multiple of 8");
  FA4B_REQUIRE(a->stride_b % 8 == 0 && a->stride_s % 8 == 0 && a->stride_h % 8 == 0 && (reinterpret_cast<uintptr_t>(a->x) & 15) == 0, FA4B_BAD_ALIGN,
               "x must be 16-byte aligned with strides that are multiples of 8 elements");
  FA4B_REQUIRE(((reinterpret_cast<uintptr_t>(a->rope_cos) | reinterpret_cast<uintptr_t>(a->rope_sin)) & 7) == 0, FA4B_BAD_ALIGN,
               "rope tables must be 8-byte aligned");
  const int64_t n_chunks = a->B * a->S * a->H * (a->D / 8);
  const unsigned grid = (unsigned)std::min<int64_t>((n_chunks + 255) / 256, (int64_t)std::max(sm_count(), 1) * 16);
  fa4b::rope_pair_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<__nv_bfloat16*>(a->x), a->stride_b, a->stride_s, a->stride_h, (int)a->S, (int)a->H, (int)a->D, n_chunks,
      static_cast<const __nv_bfloat16*>(a->rope_cos), static_cast<const __nv_bfloat16*>(a->rope_sin), a->inverse);
  FA4B_CUDA(cudaGetLastError());
  return FA4B_OK;
}

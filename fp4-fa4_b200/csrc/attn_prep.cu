// Memory-bound operand publication for the attention kernels: per-(batch, head)
// amax, NVFP4 codes + scale pages + E4M3 copies of Q and K, E4M3 V, and the
// backward's E5M2 dO with its two row statistics.
#include "attn.cuh"

namespace fa4b {

__device__ __forceinline__ float warp_max_f(float v) {
#pragma unroll
  for (int o = 16; o; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

struct HeadView {
  const __nv_bfloat16* p;
  int64_t sb, sh, ss;  // element strides: batch, head, sequence
  int H;
  __device__ __forceinline__ const __nv_bfloat16* row(int bh, int s) const {
    return p + (int64_t)(bh / H) * sb + (int64_t)(bh % H) * sh + (int64_t)s * ss;
  }
};

// grid (row chunks, B*Hq + B*Hkv): amax over the [S, D] slice of one head of Q (first n_first slices) or K
template <int D>
__global__ void __launch_bounds__(256) head_amax_kernel(HeadView xq, HeadView xk, int n_first, int S, int rows_per_cta,
                                                        int* __restrict__ amax_bits) {
  const bool second = (int)blockIdx.y >= n_first;
  const HeadView& x = second ? xk : xq;
  const int bh = second ? blockIdx.y - n_first : blockIdx.y;
  constexpr int kVec = D / 8;             // 16-byte chunks per row
  constexpr int kRowsPerPass = 256 / kVec;
  const int r0 = blockIdx.x * rows_per_cta;
  const int sub = threadIdx.x / kVec, c = threadIdx.x % kVec;
  __nv_bfloat162 acc = __float2bfloat162_rn(0.f);
  for (int r = r0 + sub; r < min(S, r0 + rows_per_cta); r += kRowsPerPass) {
    const uint4 v = __ldg(reinterpret_cast<const uint4*>(x.row(bh, r)) + c);
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int k = 0; k < 4; ++k) acc = __hmax2(acc, __habs2(*reinterpret_cast<const __nv_bfloat162*>(&w[k])));
  }
  float m = warp_max_f(fmaxf(__bfloat162float(acc.x), __bfloat162float(acc.y)));
  __shared__ float wm[8];
  if ((threadIdx.x & 31) == 0) wm[threadIdx.x >> 5] = m;
  __syncthreads();
  if (threadIdx.x == 0) {
#pragma unroll
    for (int k = 1; k < 8; ++k) m = fmaxf(m, wm[k]);
    atomicMax(amax_bits + blockIdx.y, __float_as_int(m));
  }
}

// One tensor's share of the publication launch
struct PublishSide {
  HeadView x;
  int* amax_bits;   // [heads] f32 bits
  uint8_t* codes;   // NVFP4 codes [heads, S, D/2]; NULL for V
  uint8_t* pages;   // scale pages [heads, S/128, D/64, 512]
  float* gscale;    // [heads]
  uint8_t* fp8;     // E4M3(4x) [heads, S, D]
};

// grid (S/128, B*Hq + 2 B*Hkv): one 128-row tile of one head of Q, K or V per CTA.  Q and K: NVFP4 codes, scale pages,
// global scale and E4M3(4x); V (`with_v`): E4M3(4x) only.  `unit_global`: the global decode scale is exactly one
// (amax word 2688, written here) and no statistics pass has run.
template <int D>
__global__ void __launch_bounds__(256) publish_heads_kernel(PublishSide sq, PublishSide sk, PublishSide sv, int nq, int nk, int S,
                                                            int unit_global) {
  constexpr int kKb = D / 16, kPages = D / 64;
  __shared__ __align__(16) uint8_t sc[kPages * 512];
  __shared__ StepTable steps;
  const int which = (int)blockIdx.y < nq ? 0 : ((int)blockIdx.y < nq + nk ? 1 : 2);
  const PublishSide& side = which == 0 ? sq : (which == 1 ? sk : sv);
  const HeadView& x = side.x;
  const int bh = which == 0 ? blockIdx.y : (which == 1 ? blockIdx.y - nq : blockIdx.y - nq - nk);
  const int tile = blockIdx.x, t = threadIdx.x;
  uint8_t* __restrict__ fp8 = side.fp8;
  if (which == 2) {  // V: E4M3(4v) of the tile's 128 rows
    constexpr int kPerRow = D / 16;
    for (int c = t; c < 128 * kPerRow; c += 256) {
      const int r = c / kPerRow, kb = c % kPerRow;
      const int s = tile * 128 + r;
      const uint4* src = reinterpret_cast<const uint4*>(x.row(bh, s) + kb * 16);
      const uint4 lo = __ldg(src), hi = __ldg(src + 1);
      const uint32_t w[8] = {lo.x, lo.y, lo.z, lo.w, hi.x, hi.y, hi.z, hi.w};
      uint32_t o[4];
#pragma unroll
      for (int k = 0; k < 4; ++k)
        o[k] = cvt_e4m3x4(4.f * bf16_bits_to_f32(w[2 * k] & 0xffffu), 4.f * bf16_bits_to_f32(w[2 * k] >> 16),
                          4.f * bf16_bits_to_f32(w[2 * k + 1] & 0xffffu), 4.f * bf16_bits_to_f32(w[2 * k + 1] >> 16));
      *reinterpret_cast<uint4*>(fp8 + ((size_t)bh * S + s) * D + kb * 16) = make_uint4(o[0], o[1], o[2], o[3]);
    }
    return;
  }
  uint8_t* __restrict__ codes = side.codes;
  uint8_t* __restrict__ pages = side.pages;
  const float amax = unit_global ? kNvfp4GlobalDiv : __int_as_float(side.amax_bits[bh]);
  const float g = amax / kNvfp4GlobalDiv;
  const float inv6g = 1.0f / (6.0f * g);
  if (tile == 0 && t == 0) {
    side.gscale[bh] = g;
    if (unit_global) side.amax_bits[bh] = __float_as_int(kNvfp4GlobalDiv);
  }
  const bool all_zero = !(amax > 0.f);
  fill_step_table(steps, g, t);
  __syncthreads();
#pragma unroll
  for (int i = 0; i < (128 * kKb) / 256; ++i) {
    const int b = t + i * 256;
    const int r = b / kKb, kb = b % kKb;
    const int s = tile * 128 + r;
    const uint4* src = reinterpret_cast<const uint4*>(x.row(bh, s) + kb * 16);
    const uint4 lo = __ldg(src), hi = __ldg(src + 1);
    const uint32_t w[8] = {lo.x, lo.y, lo.z, lo.w, hi.x, hi.y, hi.z, hi.w};
    uint64_t xp[8];
    uint32_t m2 = 0;
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      m2 = absmax_bf16x2(m2, w[k]);
      xp[k] = bf16x2_to_f32x2(w[k]);
    }
    const float bamax = fmaxf(bf16_bits_to_f32(m2 & 0xffffu), bf16_bits_to_f32(m2 >> 16));
    uint32_t packed[2] = {0, 0};
    uint32_t sbyte = 0;
    if (!all_zero) {
      sbyte = nvfp4_scale_byte(bamax, g, inv6g);
      nvfp4_codes16(xp, bamax, steps, sbyte, packed[0], packed[1]);
    }
    const size_t row_index = (size_t)bh * S + s;
    *reinterpret_cast<uint2*>(codes + row_index * (D / 2) + kb * 8) = make_uint2(packed[0], packed[1]);
    sc[(kb >> 2) * 512 + page_offset(r, kb)] = (uint8_t)sbyte;
    if (fp8) {
      uint32_t o[4];
      const uint64_t four = pack2(4.f, 4.f);
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        float a0, a1, b0, b1;
        unpack2(mul2(xp[2 * k], four), a0, a1);
        unpack2(mul2(xp[2 * k + 1], four), b0, b1);
        o[k] = cvt_e4m3x4(a0, a1, b0, b1);
      }
      *reinterpret_cast<uint4*>(fp8 + row_index * D + kb * 16) = make_uint4(o[0], o[1], o[2], o[3]);
    }
  }
  __syncthreads();
  if (t < kPages * 32) {
    uint8_t* dst = pages + (((size_t)bh * (S / 128) + tile) * kPages) * 512 + t * 16;
    *reinterpret_cast<uint4*>(dst) = *reinterpret_cast<const uint4*>(&sc[t * 16]);
  }
}

// V as MXFP4 in 1x32 groups along the sequence, stored feature-major: codes [B*Hkv, D, S/2] (two keys
// per byte) and one 512-byte E8M0 page per 128 keys (row = feature, k-block = 32 keys).  Scale exponent:
// floor(log2 amax) plus one when amax / 2^floor >= 1.203125 (the reference's V cut-off,
// projection_quantization_reference.py:695-704); step d = 2^e / 6.  grid (S/128, B*Hkv).
template <int D>
__global__ void __launch_bounds__(256) v_to_mx_kernel(HeadView x, int S, uint8_t* __restrict__ codes, uint8_t* __restrict__ pages) {
  constexpr int kPitch = D + 8;
  __shared__ __align__(16) __nv_bfloat16 tile[128 * kPitch];
  __shared__ __align__(16) uint8_t page[512];
  const int bh = blockIdx.y, kt = blockIdx.x, t = threadIdx.x;
  constexpr int kVec = D / 8;
  for (int c = t; c < 128 * kVec; c += 256) {
    const int r = c / kVec, c8 = (c % kVec) * 8;
    *reinterpret_cast<uint4*>(&tile[r * kPitch + c8]) = __ldg(reinterpret_cast<const uint4*>(x.row(bh, kt * 128 + r) + c8));
  }
  for (int i = t; i < 128; i += 256) reinterpret_cast<uint32_t*>(page)[i] = 0;
  __syncthreads();
  for (int item = t; item < D * 4; item += 256) {
    const int d = item % D, kb = item / D;  // adjacent lanes take adjacent features: conflict-free column reads
    float v[32];
    float amax = 0.f;
#pragma unroll
    for (int k = 0; k < 32; ++k) {
      v[k] = __bfloat162float(tile[(kb * 32 + k) * kPitch + d]);
      amax = fmaxf(amax, fabsf(v[k]));
    }
    uint32_t packed[4] = {0, 0, 0, 0};
    uint32_t ebyte = 0;
    if (amax > 0.f) {
      const uint32_t bits = __float_as_uint(fmaxf(amax, kFltMin));
      int e = (int)(bits >> 23) - 127 + (((bits >> 16) & 0x7fu) >= 26u ? 1 : 0);  // 26/128 = 0.203125
      e = min(max(e, -126), 127);
      ebyte = (uint32_t)(e + 127);
      const float step = fmaxf(__uint_as_float((uint32_t)(e + 127) << 23) / 6.0f, kFltMin);
      const float r = __frcp_rn(step);
      const uint64_t r2 = pack2(r, r), nd2 = pack2(-step, -step);
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        uint64_t q[8];
#pragma unroll
        for (int k = 0; k < 8; ++k) q[k] = div2_exact(pack2(v[16 * h + 2 * k], v[16 * h + 2 * k + 1]), r2, nd2);
        e2m1_pack16(q, packed[2 * h], packed[2 * h + 1]);
      }
    }
    *reinterpret_cast<uint4*>(codes + ((size_t)bh * D + d) * (S / 2) + kt * 64 + kb * 16) = make_uint4(packed[0], packed[1], packed[2], packed[3]);
    page[page_offset((uint32_t)d, (uint32_t)kb)] = (uint8_t)ebyte;
  }
  __syncthreads();
  if (t < 32) *reinterpret_cast<uint4*>(pages + ((size_t)bh * (S / 128) + kt) * 512 + t * 16) = *reinterpret_cast<const uint4*>(&page[t * 16]);
}

__device__ __forceinline__ float e5m2_to_f32(uint32_t byte) { return __half2float(__ushort_as_half((unsigned short)(byte << 8))); }

// dO5 = E5M2(4 dO); dstat = -4 sum_d O * float(dO5); lstat = 8 - LSE * log2e.  With `zero16` > 0 the launch also
// clears the backward's dQ accumulator, zero16 16-byte words per thread (the accumulator is a whole number of such
// rounds: 2 or 4 bytes per element of O), in place of a memset of its own between this kernel and the backward.
template <int D>
__global__ void __launch_bounds__(256) bwd_preprocess_kernel(HeadView o, HeadView dout, const float* __restrict__ lse, int S,
                                                             int64_t n_rows, uint8_t* __restrict__ do_fp8,
                                                             float* __restrict__ dstat, float* __restrict__ lstat,
                                                             uint4* __restrict__ zero_base, int zero16) {
  constexpr int kLanes = D / 8;  // threads per row, 8 elements each
  const int64_t row = (int64_t)blockIdx.x * (256 / kLanes) + threadIdx.x / kLanes;
  const int c = threadIdx.x % kLanes;
  for (int k = 0; k < zero16; ++k)
    zero_base[((int64_t)k * gridDim.x + blockIdx.x) * 256 + threadIdx.x] = make_uint4(0u, 0u, 0u, 0u);
  float acc = 0.f;
  if (row < n_rows) {
    const int bh = (int)(row / S), s = (int)(row % S);
    const uint4 ov = __ldg(reinterpret_cast<const uint4*>(o.row(bh, s)) + c);
    const uint4 dv = __ldg(reinterpret_cast<const uint4*>(dout.row(bh, s)) + c);
    const uint32_t ow[4] = {ov.x, ov.y, ov.z, ov.w}, dw[4] = {dv.x, dv.y, dv.z, dv.w};
    uint32_t packed[2];
#pragma unroll
    for (int k = 0; k < 2; ++k) {
      packed[k] = cvt_e5m2x4(4.f * bf16_bits_to_f32(dw[2 * k] & 0xffffu), 4.f * bf16_bits_to_f32(dw[2 * k] >> 16),
                             4.f * bf16_bits_to_f32(dw[2 * k + 1] & 0xffffu), 4.f * bf16_bits_to_f32(dw[2 * k + 1] >> 16));
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const uint32_t ob = ow[2 * k + (e >> 1)];
        const float of = bf16_bits_to_f32((e & 1) ? (ob >> 16) : (ob & 0xffffu));
        acc = fmaf(of, e5m2_to_f32((packed[k] >> (8 * e)) & 0xffu), acc);
      }
    }
    *reinterpret_cast<uint2*>(do_fp8 + row * D + c * 8) = make_uint2(packed[0], packed[1]);
  }
#pragma unroll
  for (int off = kLanes / 2; off; off >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, off);
  if (row < n_rows && c == 0) {
    dstat[row] = -4.0f * acc;
    lstat[row] = kPLift - lse[row] * kLog2e;
  }
}

// Fold a partial attention result into a running one (rows of D values, D / 8 threads per row):
// lse' = log(e^lse_acc + e^lse_part), o' = o_acc e^(lse_acc - lse') + o_part e^(lse_part - lse').
template <int D>
__global__ void __launch_bounds__(256) merge_kernel(float* __restrict__ o_acc, float* __restrict__ lse_acc,
                                                    const __nv_bfloat16* __restrict__ o_part, const float* __restrict__ lse_part,
                                                    int64_t n_rows, __nv_bfloat16* __restrict__ o_out) {
  constexpr int kLanes = D / 8;
  const int64_t row = (int64_t)blockIdx.x * (256 / kLanes) + threadIdx.x / kLanes;
  const int c = threadIdx.x % kLanes;
  float la = -INFINITY, lp = -INFINITY;
  if (row < n_rows) {
    la = lse_acc[row];
    lp = lse_part[row];
  }
  const float m = fmaxf(la, lp);
  float ln = m, wa = 0.f, wp = 0.f;
  if (m > -INFINITY) {
    const float ea = __expf(la - m), ep = __expf(lp - m);
    ln = m + __logf(ea + ep);
    wa = ea / (ea + ep);
    wp = ep / (ea + ep);
  }
  __syncwarp();  // every lane of the row has read lse_acc before one of them replaces it
  if (row < n_rows) {
    float* oa = o_acc + row * D + c * 8;
    const float4 a0 = *reinterpret_cast<const float4*>(oa), a1 = *reinterpret_cast<const float4*>(oa + 4);
    const uint4 pv = __ldg(reinterpret_cast<const uint4*>(o_part + row * D + c * 8));
    const uint32_t w[4] = {pv.x, pv.y, pv.z, pv.w};
    float r[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      r[2 * k] = r[2 * k] * wa + bf16_bits_to_f32(w[k] & 0xffffu) * wp;
      r[2 * k + 1] = r[2 * k + 1] * wa + bf16_bits_to_f32(w[k] >> 16) * wp;
    }
    *reinterpret_cast<float4*>(oa) = make_float4(r[0], r[1], r[2], r[3]);
    *reinterpret_cast<float4*>(oa + 4) = make_float4(r[4], r[5], r[6], r[7]);
    if (o_out) {
      uint32_t ow[4];
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const __nv_bfloat162 h = __floats2bfloat162_rn(r[2 * k], r[2 * k + 1]);
        ow[k] = *reinterpret_cast<const uint32_t*>(&h);
      }
      *reinterpret_cast<uint4*>(o_out + row * D + c * 8) = make_uint4(ow[0], ow[1], ow[2], ow[3]);
    }
    if (c == 0) lse_acc[row] = ln;
  }
}

__global__ void __launch_bounds__(256) accumulate_kernel(float* __restrict__ acc, const __nv_bfloat16* __restrict__ part, int64_t n_vec,
                                                         __nv_bfloat16* __restrict__ out) {
  for (int64_t i = (int64_t)blockIdx.x * 256 + threadIdx.x; i < n_vec; i += (int64_t)gridDim.x * 256) {
    const uint4 pv = __ldg(reinterpret_cast<const uint4*>(part) + i);
    float4 a0 = reinterpret_cast<float4*>(acc)[2 * i], a1 = reinterpret_cast<float4*>(acc)[2 * i + 1];
    a0.x += bf16_bits_to_f32(pv.x & 0xffffu); a0.y += bf16_bits_to_f32(pv.x >> 16);
    a0.z += bf16_bits_to_f32(pv.y & 0xffffu); a0.w += bf16_bits_to_f32(pv.y >> 16);
    a1.x += bf16_bits_to_f32(pv.z & 0xffffu); a1.y += bf16_bits_to_f32(pv.z >> 16);
    a1.z += bf16_bits_to_f32(pv.w & 0xffffu); a1.w += bf16_bits_to_f32(pv.w >> 16);
    reinterpret_cast<float4*>(acc)[2 * i] = a0;
    reinterpret_cast<float4*>(acc)[2 * i + 1] = a1;
    if (out) {
      const __nv_bfloat162 h0 = __floats2bfloat162_rn(a0.x, a0.y), h1 = __floats2bfloat162_rn(a0.z, a0.w);
      const __nv_bfloat162 h2 = __floats2bfloat162_rn(a1.x, a1.y), h3 = __floats2bfloat162_rn(a1.z, a1.w);
      reinterpret_cast<uint4*>(out)[i] = make_uint4(*reinterpret_cast<const uint32_t*>(&h0), *reinterpret_cast<const uint32_t*>(&h1),
                                                    *reinterpret_cast<const uint32_t*>(&h2), *reinterpret_cast<const uint32_t*>(&h3));
    }
  }
}

int launch_attn_accumulate(float* acc, const void* part, int64_t n, void* out, cudaStream_t st) {
  FA4B_REQUIRE(acc && part && n > 0 && n % 8 == 0, FA4B_BAD_ARG, "fa4b_attn_accumulate: NULL pointer or n not a positive multiple of 8");
  FA4B_REQUIRE(((reinterpret_cast<uintptr_t>(acc) | reinterpret_cast<uintptr_t>(part) | reinterpret_cast<uintptr_t>(out)) & 15) == 0, FA4B_BAD_ALIGN,
               "fa4b_attn_accumulate: 16-byte alignment");
  const int64_t n_vec = n / 8;
  const unsigned grid = (unsigned)std::min<int64_t>((n_vec + 255) / 256, (int64_t)std::max(sm_count(), 1) * 16);
  accumulate_kernel<<<grid, 256, 0, st>>>(acc, static_cast<const __nv_bfloat16*>(part), n_vec, static_cast<__nv_bfloat16*>(out));
  FA4B_CUDA(cudaGetLastError());
  return FA4B_OK;
}

int launch_attn_merge(float* o_acc, float* lse_acc, const void* o_part, const float* lse_part, int64_t n_rows, int D, void* o_out,
                      cudaStream_t st) {
  FA4B_REQUIRE(o_acc && lse_acc && o_part && lse_part, FA4B_BAD_ARG, "fa4b_attn_merge: NULL pointer");
  FA4B_REQUIRE(n_rows > 0 && (D == 64 || D == 128), FA4B_BAD_SHAPE, "fa4b_attn_merge: n_rows must be positive and D 64 or 128");
  FA4B_REQUIRE(((reinterpret_cast<uintptr_t>(o_acc) | reinterpret_cast<uintptr_t>(o_part) | reinterpret_cast<uintptr_t>(o_out)) & 15) == 0,
               FA4B_BAD_ALIGN, "fa4b_attn_merge: 16-byte alignment");
  const int rows_per_cta = 256 / (D / 8);
  const unsigned grid = (unsigned)((n_rows + rows_per_cta - 1) / rows_per_cta);
  const auto* op = static_cast<const __nv_bfloat16*>(o_part);
  auto* oo = static_cast<__nv_bfloat16*>(o_out);
  if (D == 128) merge_kernel<128><<<grid, 256, 0, st>>>(o_acc, lse_acc, op, lse_part, n_rows, oo);
  else merge_kernel<64><<<grid, 256, 0, st>>>(o_acc, lse_acc, op, lse_part, n_rows, oo);
  FA4B_CUDA(cudaGetLastError());
  return FA4B_OK;
}

// the amax words of tensors whose global decode scale is to be exactly one: amax / 2688 = 1
__global__ void publish_unit_amax_kernel(int* __restrict__ amax_bits, int n) {
  const int i = blockIdx.x * 256 + threadIdx.x;
  if (i < n) amax_bits[i] = __float_as_int(kNvfp4GlobalDiv);
}

static int check_view(const void* p, const fa4b_strides& s, const char* name) {
  FA4B_REQUIRE(p != nullptr, FA4B_BAD_ARG, "%s is NULL", name);
  FA4B_REQUIRE((reinterpret_cast<uintptr_t>(p) & 15) == 0 && s.batch % 8 == 0 && s.head % 8 == 0 && s.seq % 8 == 0, FA4B_BAD_ALIGN,
               "%s: base must be 16-byte aligned and strides multiples of 8 elements", name);
  return FA4B_OK;
}

static HeadView view(const void* p, const fa4b_strides& s, int H) {
  return HeadView{static_cast<const __nv_bfloat16*>(p), s.batch, s.head, s.seq, H};
}

template <int D>
static int prepare_impl(const fa4b_attn_prepare_args& a, cudaStream_t st, bool skip_q) {
  const fa4b_attn_dims& d = a.dims;
  const fa4b_attn_ws_layout l = make_ws_layout(d);
  uint8_t* ws = static_cast<uint8_t*>(a.ws);
  const int nq = d.B * d.Hq, nk = d.B * d.Hkv;
  int* amax_bits = reinterpret_cast<int*>(ws + l.amax_bits);
  const HeadView q = view(a.q, a.q_strides, d.Hq), k = view(a.k, a.k_strides, d.Hkv), v = view(a.v, a.v_strides, d.Hkv);
  const bool unit = d.global_scale_mode == FA4B_GLOBAL_ONE;
  const bool mx = d.pv_format == FA4B_PV_MXFP4_E8M0;
  PublishSide sq{q, amax_bits, ws + l.q_codes, ws + l.q_scales, reinterpret_cast<float*>(ws + l.q_global), ws + l.q_fp8};
  PublishSide sk{k, amax_bits + nq, ws + l.k_codes, ws + l.k_scales, reinterpret_cast<float*>(ws + l.k_global), ws + l.k_fp8};
  PublishSide sv{v, nullptr, nullptr, nullptr, nullptr, ws + l.v_fp8};
  if (a.phase != FA4B_PREPARE_QUANTIZE && !unit) {
    // one statistics launch over the heads of Q and K
    FA4B_CUDA(cudaMemsetAsync(amax_bits, 0, (size_t)(nq + nk) * 4, st));
    const int rows_per_cta = 512;
    const unsigned chunks = (unsigned)((d.S + rows_per_cta - 1) / rows_per_cta);
    head_amax_kernel<D><<<dim3(chunks, nq + nk), 256, 0, st>>>(q, k, nq, d.S, rows_per_cta, amax_bits);
    FA4B_CUDA(cudaGetLastError());
  }
  if (a.phase == FA4B_PREPARE_AMAX) {
    if (unit) {  // the words a caller may read between the phases: 2688 = a unit global scale
      publish_unit_amax_kernel<<<(nq + nk + 255) / 256, 256, 0, st>>>(amax_bits, nq + nk);
      FA4B_CUDA(cudaGetLastError());
    }
    return FA4B_OK;
  }
  // one publication launch: Q and K codes, pages, global scales and E4M3 copies, and E4M3 V.  With a unit global
  // scale and phase ALL this is the only launch in front of the forward kernel.
  const bool unit_here = unit && a.phase == FA4B_PREPARE_ALL;
  const int nq_pub = skip_q ? 0 : nq;  // the kernel numbers its CTAs Q heads, K heads, V heads
  publish_heads_kernel<D><<<dim3(d.S / 128, nq_pub + nk + (mx ? 0 : nk)), 256, 0, st>>>(sq, sk, sv, nq_pub, nk, d.S, unit_here ? 1 : 0);
  FA4B_CUDA(cudaGetLastError());
  if (mx) {
    // the V section of the cache holds the MXFP4 codes, then (1024-aligned) the scale pages
    v_to_mx_kernel<D><<<dim3(d.S / 128, nk), 256, 0, st>>>(v, d.S, ws + l.v_fp8, ws + l.v_fp8 + v_mx_pages_offset(d));
    FA4B_CUDA(cudaGetLastError());
  }
  return FA4B_OK;
}

int launch_attn_prepare(const fa4b_attn_prepare_args& a, cudaStream_t st, bool skip_q) {
  if (int s = check_dims(a.dims)) return s;
  if (int s = check_view(a.q, a.q_strides, "q")) return s;
  if (int s = check_view(a.k, a.k_strides, "k")) return s;
  if (int s = check_view(a.v, a.v_strides, "v")) return s;
  FA4B_REQUIRE(a.phase >= FA4B_PREPARE_ALL && a.phase <= FA4B_PREPARE_QUANTIZE, FA4B_BAD_ARG, "unknown prepare phase %d", a.phase);
  FA4B_REQUIRE(a.ws != nullptr && (reinterpret_cast<uintptr_t>(a.ws) & 1023) == 0, FA4B_BAD_ALIGN,
               "workspace must be non-NULL and 1024-byte aligned");
  return a.dims.D == 128 ? prepare_impl<128>(a, st, skip_q) : prepare_impl<64>(a, st, skip_q);
}

template <int D>
static int preprocess_impl(const fa4b_attn_bwd_args& a, cudaStream_t st, bool zero_dq) {
  const fa4b_attn_dims& d = a.dims;
  const fa4b_attn_ws_layout l = make_ws_layout(d);
  uint8_t* ws = transient_base(a, l);
  const int64_t n_rows = (int64_t)d.B * d.Hq * d.S;
  constexpr int kRowsPerCta = 256 / (D / 8);
  // n_rows is a multiple of 128 (S is): every CTA is full, and one 16-byte word per thread covers two bytes per element
  const int zero16 = zero_dq ? (bwd_dq_half(d, a.flags) ? 1 : 2) : 0;
  bwd_preprocess_kernel<D><<<(unsigned)((n_rows + kRowsPerCta - 1) / kRowsPerCta), 256, 0, st>>>(
      view(a.o, a.o_strides, d.Hq), view(a.dout, a.do_strides, d.Hq), a.lse, d.S, n_rows, ws + l.do_fp8,
      reinterpret_cast<float*>(ws + l.dstat), reinterpret_cast<float*>(ws + l.lstat), reinterpret_cast<uint4*>(ws + l.dq_accum), zero16);
  FA4B_CUDA(cudaGetLastError());
  return FA4B_OK;
}

int launch_attn_bwd_preprocess(const fa4b_attn_bwd_args& a, cudaStream_t st, bool zero_dq) {
  if (int s = check_dims(a.dims)) return s;
  if (int s = check_view(a.o, a.o_strides, "o")) return s;
  if (int s = check_view(a.dout, a.do_strides, "dout")) return s;
  FA4B_REQUIRE(a.lse != nullptr, FA4B_BAD_ARG, "lse is NULL");
  FA4B_REQUIRE(a.ws != nullptr && (reinterpret_cast<uintptr_t>(a.ws) & 1023) == 0, FA4B_BAD_ALIGN,
               "workspace must be non-NULL and 1024-byte aligned");
  FA4B_REQUIRE((reinterpret_cast<uintptr_t>(a.scratch) & 1023) == 0, FA4B_BAD_ALIGN, "scratch must be 1024-byte aligned");
  return a.dims.D == 128 ? preprocess_impl<128>(a, st, zero_dq) : preprocess_impl<64>(a, st, zero_dq);
}

}  // namespace fa4b

using namespace fa4b;

extern "C" int fa4b_attn_prepare(const fa4b_attn_prepare_args* a, void* stream) {
  FA4B_REQUIRE(a != nullptr, FA4B_BAD_ARG, "args is NULL");
  return launch_attn_prepare(*a, static_cast<cudaStream_t>(stream));
}

extern "C" int fa4b_attn_bwd_preprocess(const fa4b_attn_bwd_args* a, void* stream) {
  FA4B_REQUIRE(a != nullptr, FA4B_BAD_ARG, "args is NULL");
  return launch_attn_bwd_preprocess(*a, static_cast<cudaStream_t>(stream));
}

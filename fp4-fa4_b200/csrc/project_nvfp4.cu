// Y[M, N] = A[M, K] . W[N, K]^T for two prepared NVFP4 operands (packed E2M1 codes, E4M3 scales of 16 values in
// 512-byte pages, one FP32 global scale each), BF16 out.  Replaces project_nvfp4_generic behind
// b300_project_nvfp4 (tk_fa4/interface.py:1619-1640).
//
// One persistent CTA per SM walks 128 x 256 output tiles.  Per K step of 256 values a stage holds the A codes
// (128 rows x 128 bytes), the W codes (256 rows x 128 bytes) and their scale pages (4 + 8).  Roles: a producer
// warp fills the four stages by TMA; an issuer warp copies each stage's scale pages to TMEM (tcgen05.cp) and
// issues four block-scaled tcgen05 MMAs (M128 N256 K64) per stage into a 256-column FP32 accumulator; eight
// epilogue warps read the accumulator out of TMEM (128 columns in flight each), hand it back to the issuer,
// apply the two global scales and store BF16 rows through small swizzled boxes and TMA stores, beside the next
// tile's MMAs.
//
// (K steps of 128 values in eight stages, three stages with larger store boxes, four epilogue warps storing straight
// from registers, and scale-page copies on a warp of their own were all slower than this arrangement.)
#include <algorithm>
#include <mutex>

#include <cuda_bf16.h>

#include "attn.cuh"
#include "common.cuh"
#include "tc_sm100.cuh"

namespace fa4b {

constexpr int kProjThreads = 320;  // warp 0 producer, warp 1 issuer, warps 2-9 epilogue
constexpr int kProjTileM = 128, kProjTileN = 256, kProjStepK = 256;
constexpr int kProjStages = kProjStepK == 256 ? 4 : 8;
constexpr int kRowBytes = kProjStepK / 2;   // code bytes per row and stage: 128 (128-byte swizzle) or 64
constexpr int kStepMmas = kProjStepK / 64;  // K64 MMAs, and scale pages per 128 rows, per stage

struct ProjStage {
  alignas(1024) uint8_t a[kProjTileM * kRowBytes];
  alignas(1024) uint8_t w[kProjTileN * kRowBytes];
  alignas(16) uint8_t a_sf[kStepMmas * 512];
  alignas(16) uint8_t w_sf[2][kStepMmas * 512];
};
constexpr uint32_t kProjStageBytes = (kProjTileM + kProjTileN) * kRowBytes + 3 * kStepMmas * 512;

struct ProjSmem {
  ProjStage stage[kProjStages];
  // per epilogue warp: one box of 8 rows x 64 bf16 (128-byte rows, 128-byte swizzle), the source of a TMA store;
  // four stages leave no room for more
  alignas(1024) uint8_t out[8][8 * 128];
  alignas(8) uint64_t full[kProjStages];
  uint64_t empty[kProjStages];
  uint64_t acc_full, acc_free, mma_drained;
  uint32_t tmem_base;
  volatile uint32_t abort_flag;
  StepTable steps;  // PUBLISH: steps of the 127 scale bytes at a unit global scale
};

struct ProjParams {
  const uint8_t* a_sf;   // [M/128, K/64, 512]
  const uint8_t* w_sf;   // [N/128, K/64, 512]
  const float* a_global;
  const float* w_global;
  __nv_bfloat16* y;
  int64_t ldy;
  int M, N, K;
  uint32_t* status;
  // publication mode (PUBLISH): the output columns are Hq query heads, Hkv key heads, Hkv value heads of 128 features;
  // instead of BF16 rows the epilogue writes the attention operands of every head into the attention workspace
  const __nv_bfloat16* rope_cos;  // [S, 64]
  const __nv_bfloat16* rope_sin;
  int S, Hq, Hkv;
  uint8_t *q_codes, *q_pages, *q_fp8, *k_codes, *k_pages, *k_fp8, *v_fp8;
  float *q_global, *k_global;
  // dO publication mode: the output columns are the Hq heads of dO; O rows [M, Hq * 128] bf16 and LSE [B, Hq, S] in
  const __nv_bfloat16* o_rows;
  const float* lse;
  uint8_t* do_fp8;
  float *dstat, *lstat;
};

// TMEM columns: accumulator 0-255; scale factors of a stage: A 8 columns, W 16 columns, two slots
constexpr uint32_t kColSf = 256, kSfSlot = 12 * kStepMmas;

// MODE 0: BF16 rows out; 1: QKV projection publishing the attention operands; 2: output projection's input-gradient
// GEMM publishing dO and the row statistics of the attention backward
template <int MODE>
__global__ void __launch_bounds__(kProjThreads, 1)
project_nvfp4_kernel(const ProjParams p, const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_w,
                     const __grid_constant__ CUtensorMap map_y) {
  // the dynamic shared memory of a kernel without static shared memory starts on a 1024-byte boundary of the
  // CTA's window; four stages leave no room to round the pointer up, so the kernel checks and refuses otherwise
  extern __shared__ __align__(1024) uint8_t raw[];
  ProjSmem& s = *reinterpret_cast<ProjSmem*>(raw);
  const int t = threadIdx.x, warp = t >> 5, lane = t & 31;
  if ((smem_u32(raw) & 1023u) != 0u) {  // CTA-uniform
    if (t == 0 && atomicCAS(p.status, 0u, 1u) == 0u) {
      p.status[1] = 400;
      p.status[2] = blockIdx.x;
      p.status[3] = smem_u32(raw);
    }
    return;
  }
  const int tiles_n = p.N / kProjTileN, n_tiles = (p.M / kProjTileM) * tiles_n, n_k = p.K / kProjStepK;
  const int64_t pages_k = p.K / 64;

  if (t == 0) {
    for (int i = 0; i < kProjStages; ++i) {
      mbar_init(&s.full[i], 1);
      mbar_init(&s.empty[i], 1);
    }
    mbar_init(&s.acc_full, 1);
    mbar_init(&s.acc_free, 8);
    mbar_init(&s.mma_drained, 1);
    s.abort_flag = 0;
    fence_barrier_init();
  }
  constexpr bool PUBLISH = MODE == 1;
  if (PUBLISH) {
    fill_step_table(s.steps, 1.0f, t);
    if (blockIdx.x == 0) {  // unit global decode scales of every (batch, head)
      const int B = p.M / p.S;
      for (int i = t; i < B * p.Hq; i += kProjThreads) p.q_global[i] = 1.0f;
      for (int i = t; i < B * p.Hkv; i += kProjThreads) p.k_global[i] = 1.0f;
    }
  }
  if (warp == 0) tmem_alloc(&s.tmem_base, 512);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tm = s.tmem_base;

  if (warp == 0) {
    // ------------------------------------------------------------------ producer
    if (lane == 0) {
      tma_prefetch_desc(&map_a);
      tma_prefetch_desc(&map_w);
      int it = 0, issued = 0;
      bool ok = true;
      for (int tile = blockIdx.x; ok && tile < n_tiles; tile += gridDim.x) {
        const int tm_i = tile / tiles_n, tn_i = tile % tiles_n;
        for (int kb = 0; kb < n_k; ++kb, ++it) {
          const int st = it % kProjStages;
          if (it >= kProjStages && !mbar_wait(&s.empty[st], ((it / kProjStages) - 1) & 1, &s.abort_flag, p.status, 410, it)) {
            ok = false;
            break;
          }
          issued = it + 1;
          ProjStage& g = s.stage[st];
          mbar_expect_tx(&s.full[st], kProjStageBytes);
          tma_load_2d(g.a, &map_a, kb * kRowBytes, tm_i * kProjTileM, &s.full[st]);
          tma_load_2d(g.w, &map_w, kb * kRowBytes, tn_i * kProjTileN, &s.full[st]);
          bulk_load(g.a_sf, p.a_sf + ((int64_t)tm_i * pages_k + kb * kStepMmas) * 512, kStepMmas * 512, &s.full[st]);
          bulk_load(g.w_sf[0], p.w_sf + ((int64_t)(2 * tn_i) * pages_k + kb * kStepMmas) * 512, kStepMmas * 512, &s.full[st]);
          bulk_load(g.w_sf[1], p.w_sf + ((int64_t)(2 * tn_i + 1) * pages_k + kb * kStepMmas) * 512, kStepMmas * 512, &s.full[st]);
        }
      }
      // no copy of this CTA may still be in flight when its shared memory is given up
      // and the tensor core's last arrivals on the stage barriers must have landed (nobody else waits for them)
      for (int j = issued > kProjStages ? issued - kProjStages : 0; j < issued; ++j) {
        mbar_wait_teardown(&s.full[j % kProjStages], (j / kProjStages) & 1);
        if (ok && !s.abort_flag) mbar_wait_teardown(&s.empty[j % kProjStages], (j / kProjStages) & 1);
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    const bool leader = elect_one();
    constexpr uint32_t idesc = idesc_fp4(kProjTileM, kProjTileN, 0, 0, 0);
    int it = 0, n_done = 0;
    bool ok = true;
    for (int tile = blockIdx.x; ok && tile < n_tiles; tile += gridDim.x, ++n_done) {
      // the epilogue has read the previous tile's accumulator out of TMEM
      if (n_done > 0 && !mbar_wait_warp(&s.acc_free, (n_done - 1) & 1, &s.abort_flag, p.status, 420, tile)) {
        ok = false;
        break;
      }
      tc_fence_after();
      for (int kb = 0; kb < n_k; ++kb, ++it) {
        const int st = it % kProjStages;
        if (!mbar_wait_warp(&s.full[st], (it / kProjStages) & 1, &s.abort_flag, p.status, 421, it)) {
          ok = false;
          break;
        }
        tc_fence_after();
        if (leader) {
          ProjStage& g = s.stage[st];
          const uint32_t sf = tm + kColSf + (it & 1) * kSfSlot;
#pragma unroll
          for (int k = 0; k < kStepMmas; ++k) {
            tmem_cp_page(sf + 4 * k, make_page_desc(smem_u32(g.a_sf + 512 * k)));
            tmem_cp_page(sf + 4 * kStepMmas + 8 * k, make_page_desc(smem_u32(g.w_sf[0] + 512 * k)));
            tmem_cp_page(sf + 4 * kStepMmas + 8 * k + 4, make_page_desc(smem_u32(g.w_sf[1] + 512 * k)));
          }
          const uint64_t da = make_tile_desc(smem_u32(g.a), kRowBytes), dw = make_tile_desc(smem_u32(g.w), kRowBytes);
#pragma unroll
          for (int k = 0; k < kStepMmas; ++k)
            mma_nvfp4_ss(tm, da + 2 * k, dw + 2 * k, idesc, sf + 4 * k, sf + 4 * kStepMmas + 8 * k, (kb > 0 || k > 0) ? 1u : 0u);
          mma_commit(&s.empty[st]);
          if (kb == n_k - 1) mma_commit(&s.acc_full);
        }
        __syncwarp();
      }
    }
    // every tensor-core operation of this CTA has finished before TMEM is freed
    if (leader) {
      mma_commit(&s.mma_drained);
      mbar_wait_teardown(&s.mma_drained, 0);
    }
    __syncwarp();
  } else {
    // ------------------------------------------------------------------ epilogue (warps 2-9)
    // two warps per TMEM lane quarter, 128 accumulator columns each: all four loads of a warp are in flight at
    // once and the accumulator goes back to the issuer as soon as they have landed
    const int quarter = warp & 3, half = (warp - 2) >> 2;
    const uint32_t lane_base = tm + ((uint32_t)(quarter * 32) << 16) + half * 128;
    const float gscale = __ldg(p.a_global) * __ldg(p.w_global);
    uint8_t* const box = s.out[warp - 2];
    const uint32_t swz = (uint32_t)(lane & 7);
    int n_done = 0;
    for (int tile = blockIdx.x; tile < n_tiles; tile += gridDim.x, ++n_done) {
      const int tm_i = tile / tiles_n, tn_i = tile % tiles_n;
      if (!mbar_wait_warp(&s.acc_full, n_done & 1, &s.abort_flag, p.status, 430, tile)) break;
      tc_fence_after();
      uint32_t v[4][32];
#pragma unroll
      for (int c = 0; c < 4; ++c) tmem_ld32(lane_base + c * 32, v[c]);
      tmem_ld_wait(v[0]);
      tmem_ld_wait(v[1]);
      tmem_ld_wait(v[2]);
      tmem_ld_wait(v[3]);
      tc_fence_before();
      mbar_arrive_warp(&s.acc_free);
      if constexpr (PUBLISH) {
        // This warp holds 32 tokens x the 128 features of one head.  Per 32 features: round to BF16 (the projection's
        // output), rotate Q and K in packed BF16 (the arithmetic of rope_pair_kernel), then publish what the attention
        // kernels read: E4M3(4x) rows, and for Q and K the NVFP4 codes and scale bytes at a unit global scale
        // (fused in the reference's projection epilogue, projection_fp4_epilogue.cuh:1453-1579, 873-983).
        const int hh = tn_i * 2 + half;
        const int m = tm_i * kProjTileM + quarter * 32 + lane;
        const int bi = m / p.S, si = m % p.S;
        const bool is_v = hh >= p.Hq + p.Hkv;
        const bool is_q = hh < p.Hq;
        const int bh = is_q ? bi * p.Hq + hh : (is_v ? bi * p.Hkv + hh - p.Hq - p.Hkv : bi * p.Hkv + hh - p.Hq);
        const size_t row_index = (size_t)bh * p.S + si;
        uint8_t* fp8 = (is_q ? p.q_fp8 : is_v ? p.v_fp8 : p.k_fp8) + row_index * 128;
        uint8_t* codes = (is_q ? p.q_codes : p.k_codes) + row_index * 64;
        uint8_t* pages = (is_q ? p.q_pages : p.k_pages) + ((size_t)bh * (p.S / 128) + si / 128) * 2 * 512 + lane * 16 + quarter * 4;
        const uint4* ct = reinterpret_cast<const uint4*>(p.rope_cos + (size_t)si * 64);
        const uint4* st4 = reinterpret_cast<const uint4*>(p.rope_sin + (size_t)si * 64);
        uint32_t sc4 = 0;
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          uint32_t w[16];
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            const __nv_bfloat162 h2 = __floats2bfloat162_rn(__uint_as_float(v[c][2 * i]) * gscale, __uint_as_float(v[c][2 * i + 1]) * gscale);
            w[i] = *reinterpret_cast<const uint32_t*>(&h2);
          }
          if (!is_v) {
            const uint4 c0 = __ldg(ct + 2 * c), c1 = __ldg(ct + 2 * c + 1), s0 = __ldg(st4 + 2 * c), s1 = __ldg(st4 + 2 * c + 1);
            const uint32_t cw[8] = {c0.x, c0.y, c0.z, c0.w, c1.x, c1.y, c1.z, c1.w}, sw[8] = {s0.x, s0.y, s0.z, s0.w, s1.x, s1.y, s1.z, s1.w};
#pragma unroll
            for (int i = 0; i < 16; ++i) {
              const uint32_t cc = ((cw[i >> 1] >> (16 * (i & 1))) & 0xffffu) * 0x00010001u;
              const uint32_t s2 = ((sw[i >> 1] >> (16 * (i & 1))) & 0xffffu) * 0x00010001u;
              const uint32_t perp = ((w[i] << 16) | (w[i] >> 16)) ^ 0x00008000u;  // (x, y) -> (-y, x)
              const __nv_bfloat162 r = __hfma2(*reinterpret_cast<const __nv_bfloat162*>(&perp), *reinterpret_cast<const __nv_bfloat162*>(&s2),
                                               __hmul2(*reinterpret_cast<const __nv_bfloat162*>(&w[i]), *reinterpret_cast<const __nv_bfloat162*>(&cc)));
              w[i] = *reinterpret_cast<const uint32_t*>(&r);
            }
          }
#pragma unroll
          for (int blk = 0; blk < 2; ++blk) {  // 16 features
            uint64_t xp[8];
            float bamax = 0.f;
#pragma unroll
            for (int k = 0; k < 8; ++k) {
              xp[k] = bf16x2_to_f32x2(w[8 * blk + k]);
              bamax = absmax3(bamax, xp[k]);
            }
            uint32_t o8[4];
            const uint64_t four = pack2(4.f, 4.f);
#pragma unroll
            for (int k = 0; k < 4; ++k) {
              float a0, a1, b0, b1;
              unpack2(mul2(xp[2 * k], four), a0, a1);
              unpack2(mul2(xp[2 * k + 1], four), b0, b1);
              o8[k] = cvt_e4m3x4(a0, a1, b0, b1);
            }
            *reinterpret_cast<uint4*>(fp8 + c * 32 + blk * 16) = make_uint4(o8[0], o8[1], o8[2], o8[3]);
            if (!is_v) {
              const int kb = 2 * c + blk;
              const uint32_t sbyte = nvfp4_scale_byte(bamax, 1.0f, 1.0f / 6.0f);
              uint32_t lo, hi;
              nvfp4_codes16(xp, bamax, s.steps, sbyte, lo, hi);
              *reinterpret_cast<uint2*>(codes + kb * 8) = make_uint2(lo, hi);
              sc4 |= sbyte << (8 * (kb & 3));
              if ((kb & 3) == 3) {  // the four scale bytes of this row in one page
                *reinterpret_cast<uint32_t*>(pages + (kb >> 2) * 512) = sc4;
                sc4 = 0;
              }
            }
          }
        }
        continue;
      }
      if constexpr (MODE == 2) {
        // This warp holds dO of 32 tokens x one head.  Round to BF16 (the GEMM's output), then what
        // bwd_preprocess_kernel makes of it: E5M2(4 dO), dstat = -4 sum_d O float(dO5) with that kernel's
        // association order (sixteen partial sums of eight features, then a balanced tree), lstat = 8 - LSE log2e
        // (fused in the reference's output-projection dgrad epilogue, projection_fp4_epilogue.cuh:4049-4127).
        const int hh = tn_i * 2 + half;
        const int m = tm_i * kProjTileM + quarter * 32 + lane;
        const int bi = m / p.S, si = m % p.S;
        const size_t row_index = ((size_t)bi * p.Hq + hh) * p.S + si;
        const uint4* orow = reinterpret_cast<const uint4*>(p.o_rows + (size_t)m * p.Hq * 128 + hh * 128);
        uint8_t* dst = p.do_fp8 + row_index * 128;
        float part[16];
#pragma unroll
        for (int c = 0; c < 4; ++c) {
#pragma unroll
          for (int g8 = 0; g8 < 4; ++g8) {  // eight features
            uint32_t dw[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              const __nv_bfloat162 h2 = __floats2bfloat162_rn(__uint_as_float(v[c][8 * g8 + 2 * i]) * gscale,
                                                               __uint_as_float(v[c][8 * g8 + 2 * i + 1]) * gscale);
              dw[i] = *reinterpret_cast<const uint32_t*>(&h2);
            }
            const uint4 ov = __ldg(orow + 4 * c + g8);
            const uint32_t ow[4] = {ov.x, ov.y, ov.z, ov.w};
            uint32_t packed[2];
            float acc = 0.f;
#pragma unroll
            for (int k = 0; k < 2; ++k) {
              packed[k] = cvt_e5m2x4(4.f * bf16_bits_to_f32(dw[2 * k] & 0xffffu), 4.f * bf16_bits_to_f32(dw[2 * k] >> 16),
                                     4.f * bf16_bits_to_f32(dw[2 * k + 1] & 0xffffu), 4.f * bf16_bits_to_f32(dw[2 * k + 1] >> 16));
#pragma unroll
              for (int e = 0; e < 4; ++e) {
                const uint32_t ob = ow[2 * k + (e >> 1)];
                const float of = bf16_bits_to_f32((e & 1) ? (ob >> 16) : (ob & 0xffffu));
                acc = fmaf(of, __half2float(__ushort_as_half((unsigned short)(((packed[k] >> (8 * e)) & 0xffu) << 8))), acc);
              }
            }
            *reinterpret_cast<uint2*>(dst + (4 * c + g8) * 8) = make_uint2(packed[0], packed[1]);
            part[4 * c + g8] = acc;
          }
        }
#pragma unroll
        for (int i = 0; i < 8; ++i) part[i] += part[i + 8];
#pragma unroll
        for (int i = 0; i < 4; ++i) part[i] += part[i + 4];
        part[0] += part[2];
        part[1] += part[3];
        p.dstat[row_index] = -4.0f * (part[0] + part[1]);
        p.lstat[row_index] = kPLift - __ldg(p.lse + row_index) * kLog2e;
        continue;
      }
      const int col = tn_i * kProjTileN + half * 128, row = tm_i * kProjTileM + quarter * 32;
      // BF16 in place: word 16 * c + i of `o` = columns 32 * c + 2 * i, + 1 of this lane's row
      uint32_t o[64];
#pragma unroll
      for (int c = 0; c < 4; ++c)
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          const __nv_bfloat162 h2 = __floats2bfloat162_rn(__uint_as_float(v[c][2 * i]) * gscale, __uint_as_float(v[c][2 * i + 1]) * gscale);
          o[16 * c + i] = *reinterpret_cast<const uint32_t*>(&h2);
        }
      // eight stores of 8 rows x 64 columns: the lanes of the row group write their 128 bytes, lane 0 stores the box
#pragma unroll
      for (int b2 = 0; b2 < 2; ++b2) {
#pragma unroll 1
        for (int rg = 0; rg < 4; ++rg) {
          if (lane == 0) tma_store_wait_read();  // the box is free once the store that read it last has done so
          __syncwarp();
          if ((lane >> 3) == rg) {
#pragma unroll
            for (int ch = 0; ch < 8; ++ch)
              *reinterpret_cast<uint4*>(box + (lane & 7) * 128 + (((uint32_t)ch ^ swz) << 4)) =
                  make_uint4(o[32 * b2 + 4 * ch], o[32 * b2 + 4 * ch + 1], o[32 * b2 + 4 * ch + 2], o[32 * b2 + 4 * ch + 3]);
          }
          fence_async_smem();
          __syncwarp();
          if (lane == 0) {
            tma_store_2d(&map_y, box, col + 64 * b2, row + 8 * rg);
            tma_store_commit();
          }
        }
      }
    }
    // shared memory stays valid until the stores have read it
    if (lane == 0) tma_store_wait_read();
    __syncwarp();
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tm, 512);
}

}  // namespace fa4b

using namespace fa4b;

static int project_check(const fa4b_project_nvfp4_args* a, bool need_y) {
  FA4B_REQUIRE(a != nullptr, FA4B_BAD_ARG, "args is NULL");
  FA4B_REQUIRE(a->a_codes && a->a_scales && a->a_global && a->w_codes && a->w_scales && a->w_global && (a->y || !need_y) && a->status, FA4B_BAD_ARG,
               "fa4b_project_nvfp4: NULL pointer");
  FA4B_REQUIRE(a->M > 0 && a->N > 0 && a->K > 0 && a->M % kProjTileM == 0 && a->N % kProjTileN == 0 && a->K % kProjStepK == 0, FA4B_BAD_SHAPE,
               "M=%lld N=%lld K=%lld: M must be a multiple of 128, N of 256 and K of %d", (long long)a->M, (long long)a->N, (long long)a->K, kProjStepK);
  FA4B_REQUIRE(a->M < (1ll << 31) && a->N < (1ll << 31) && a->K < (1ll << 31), FA4B_BAD_SHAPE, "dimensions must fit 31 bits");
  FA4B_REQUIRE(((reinterpret_cast<uintptr_t>(a->a_codes) | reinterpret_cast<uintptr_t>(a->w_codes) | reinterpret_cast<uintptr_t>(a->a_scales) |
                 reinterpret_cast<uintptr_t>(a->w_scales)) & 15) == 0, FA4B_BAD_ALIGN, "operands must be 16-byte aligned");
  return FA4B_OK;
}

template <int MODE>
static int project_launch(const fa4b_project_nvfp4_args* a, ProjParams p, const CUtensorMap& my, cudaStream_t st) {
  FA4B_CUDA(cudaMemsetAsync(a->status, 0, 4 * sizeof(uint32_t), st));
  CUtensorMap ma{}, mw{};
  if (int s = make_tensor_map(&ma, a->a_codes, 1, (uint64_t)a->K / 2, (uint64_t)a->M, 0, (uint64_t)a->K / 2, 0, kRowBytes, kProjTileM)) return s;
  if (int s = make_tensor_map(&mw, a->w_codes, 1, (uint64_t)a->K / 2, (uint64_t)a->N, 0, (uint64_t)a->K / 2, 0, kRowBytes, kProjTileN)) return s;
  int dev = 0, sms = 0;
  FA4B_CUDA(cudaGetDevice(&dev));
  FA4B_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
  const int smem = sizeof(ProjSmem);
  // the attribute belongs to the current device's context: set on every call (cheap) so that a second GPU of the process gets it too
  FA4B_CUDA(cudaFuncSetAttribute(project_nvfp4_kernel<MODE>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
  p.a_sf = a->a_scales; p.w_sf = a->w_scales;
  p.a_global = a->a_global; p.w_global = a->w_global;
  p.M = (int)a->M; p.N = (int)a->N; p.K = (int)a->K;
  p.status = a->status;
  const int n_tiles = (p.M / kProjTileM) * (p.N / kProjTileN);
  project_nvfp4_kernel<MODE><<<std::min(n_tiles, sms), kProjThreads, smem, st>>>(p, ma, mw, my);
  FA4B_CUDA(cudaGetLastError());
  return FA4B_OK;
}

int fa4b_project_nvfp4(const fa4b_project_nvfp4_args* a, void* stream) {
  if (int s = project_check(a, true)) return s;
  FA4B_REQUIRE(a->ldy >= a->N && a->ldy % 8 == 0 && (reinterpret_cast<uintptr_t>(a->y) & 15) == 0, FA4B_BAD_ALIGN,
               "y must be 16-byte aligned with a row stride >= N that is a multiple of 8 elements");
  CUtensorMap my{};
  if (int s = make_tensor_map(&my, a->y, 2, (uint64_t)a->N, (uint64_t)a->M, 0, (uint64_t)a->ldy * 2, 0, 64, 8)) return s;
  ProjParams p{};
  p.y = static_cast<__nv_bfloat16*>(a->y); p.ldy = a->ldy;
  return project_launch<0>(a, p, my, static_cast<cudaStream_t>(stream));
}

int fa4b_project_qkv_publish(const fa4b_project_nvfp4_args* a, const fa4b_attn_dims* d, const void* rope_cos, const void* rope_sin, void* ws,
                             void* stream) {
  if (int s = project_check(a, false)) return s;
  FA4B_REQUIRE(d && rope_cos && rope_sin && ws, FA4B_BAD_ARG, "fa4b_project_qkv_publish: NULL pointer");
  if (int s = check_dims(*d)) return s;
  FA4B_REQUIRE(d->D == 128 && d->pv_format == FA4B_PV_FP8_E4M3 && d->global_scale_mode == FA4B_GLOBAL_ONE, FA4B_UNSUPPORTED,
               "the fused publication serves head dim 128, FP8 P.V and the unit global scale");
  FA4B_REQUIRE(a->M == (int64_t)d->B * d->S && a->N == (int64_t)(d->Hq + 2 * d->Hkv) * 128, FA4B_BAD_SHAPE,
               "M=%lld N=%lld do not match B*S=%lld and (Hq + 2 Hkv) * 128 = %lld", (long long)a->M, (long long)a->N, (long long)d->B * d->S,
               (long long)(d->Hq + 2 * d->Hkv) * 128);
  FA4B_REQUIRE((reinterpret_cast<uintptr_t>(ws) & 1023) == 0 && ((reinterpret_cast<uintptr_t>(rope_cos) | reinterpret_cast<uintptr_t>(rope_sin)) & 15) == 0,
               FA4B_BAD_ALIGN, "workspace must be 1024-byte aligned, rope tables 16-byte aligned");
  const fa4b_attn_ws_layout l = make_ws_layout(*d);
  uint8_t* w8 = static_cast<uint8_t*>(ws);
  ProjParams p{};
  p.rope_cos = static_cast<const __nv_bfloat16*>(rope_cos); p.rope_sin = static_cast<const __nv_bfloat16*>(rope_sin);
  p.S = d->S; p.Hq = d->Hq; p.Hkv = d->Hkv;
  p.q_codes = w8 + l.q_codes; p.q_pages = w8 + l.q_scales; p.q_fp8 = w8 + l.q_fp8; p.q_global = reinterpret_cast<float*>(w8 + l.q_global);
  p.k_codes = w8 + l.k_codes; p.k_pages = w8 + l.k_scales; p.k_fp8 = w8 + l.k_fp8; p.k_global = reinterpret_cast<float*>(w8 + l.k_global);
  p.v_fp8 = w8 + l.v_fp8;
  CUtensorMap my{};  // unused in this mode
  return project_launch<1>(a, p, my, static_cast<cudaStream_t>(stream));
}

int fa4b_project_dout_publish(const fa4b_project_nvfp4_args* a, const fa4b_attn_dims* d, const void* o_rows, const float* lse, void* ws,
                              void* stream) {
  if (int s = project_check(a, false)) return s;
  FA4B_REQUIRE(d && o_rows && lse && ws, FA4B_BAD_ARG, "fa4b_project_dout_publish: NULL pointer");
  if (int s = check_dims(*d)) return s;
  FA4B_REQUIRE(d->D == 128 && d->pv_format == FA4B_PV_FP8_E4M3, FA4B_UNSUPPORTED, "the fused dO publication serves head dim 128 and FP8 P.V");
  FA4B_REQUIRE(a->M == (int64_t)d->B * d->S && a->N == (int64_t)d->Hq * 128, FA4B_BAD_SHAPE,
               "M=%lld N=%lld do not match B*S=%lld and Hq * 128 = %lld", (long long)a->M, (long long)a->N, (long long)d->B * d->S,
               (long long)d->Hq * 128);
  FA4B_REQUIRE((reinterpret_cast<uintptr_t>(ws) & 1023) == 0 && (reinterpret_cast<uintptr_t>(o_rows) & 15) == 0, FA4B_BAD_ALIGN,
               "workspace must be 1024-byte aligned, the O rows 16-byte aligned");
  const fa4b_attn_ws_layout l = make_ws_layout(*d);
  uint8_t* w8 = static_cast<uint8_t*>(ws);
  ProjParams p{};
  p.S = d->S; p.Hq = d->Hq; p.Hkv = d->Hkv;
  p.o_rows = static_cast<const __nv_bfloat16*>(o_rows); p.lse = lse;
  p.do_fp8 = w8 + l.do_fp8; p.dstat = reinterpret_cast<float*>(w8 + l.dstat); p.lstat = reinterpret_cast<float*>(w8 + l.lstat);
  CUtensorMap my{};  // unused in this mode
  return project_launch<2>(a, p, my, static_cast<cudaStream_t>(stream));
}

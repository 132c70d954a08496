// Y[M, N] = A[M, K] . W[N, K]^T for two prepared NVFP4 operands (packed E2M1 codes, E4M3 scales of 16 values in
// 512-byte pages, one FP32 global scale each), BF16 out.  Replaces project_nvfp4_generic behind
// b300_project_nvfp4 (tk_fa4/interface.py:1619-1640).
//
// One persistent CTA per SM walks 128 x 256 output tiles.  Per K step of 256 values a stage holds the A codes
// (128 rows x 128 bytes), the W codes (256 rows x 128 bytes) and their scale pages (4 + 8); a producer warp
// fills the stages by TMA, an issuer warp copies the scale pages to TMEM and issues four block-scaled
// tcgen05 MMAs (M128 N256 K64) per stage into a 256-column FP32 accumulator, and four epilogue warps read the
// accumulator out of TMEM, apply the two global scales and store BF16.  The accumulator is handed back to the
// issuer as soon as it is in registers, so the next tile's MMAs run beside the stores.
#include <algorithm>
#include <mutex>

#include <cuda_bf16.h>

#include "common.cuh"
#include "fa4b.h"
#include "tc_sm100.cuh"

namespace fa4b {

constexpr int kProjStages = 4;
constexpr int kProjThreads = 192;  // warp 0 producer, warp 1 issuer, warps 2-5 epilogue
constexpr int kProjTileM = 128, kProjTileN = 256, kProjStepK = 256;

struct ProjStage {
  alignas(1024) uint8_t a[kProjTileM * 128];
  alignas(1024) uint8_t w[kProjTileN * 128];
  alignas(16) uint8_t a_sf[4 * 512];
  alignas(16) uint8_t w_sf[2][4 * 512];
};
constexpr uint32_t kProjStageBytes = kProjTileM * 128 + kProjTileN * 128 + 4 * 512 + 8 * 512;

struct ProjSmem {
  ProjStage stage[kProjStages];
  alignas(8) uint64_t full[kProjStages];
  uint64_t empty[kProjStages];
  uint64_t acc_full, acc_free, mma_drained;
  uint32_t tmem_base;
  volatile uint32_t abort_flag;
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
};

// TMEM columns: accumulator 0-255; scale factors of a stage: A 16 columns, W 32 columns, two slots
constexpr uint32_t kColSf = 256, kSfSlot = 48;

__global__ void __launch_bounds__(kProjThreads, 1)
project_nvfp4_kernel(const ProjParams p, const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_w) {
  extern __shared__ uint8_t raw[];
  ProjSmem& s = *reinterpret_cast<ProjSmem*>((reinterpret_cast<uintptr_t>(raw) + 1023) & ~uintptr_t(1023));
  const int t = threadIdx.x, warp = t >> 5, lane = t & 31;
  const int tiles_n = p.N / kProjTileN, n_tiles = (p.M / kProjTileM) * tiles_n, n_k = p.K / kProjStepK;
  const int64_t pages_k = p.K / 64;

  if (t == 0) {
    for (int i = 0; i < kProjStages; ++i) {
      mbar_init(&s.full[i], 1);
      mbar_init(&s.empty[i], 1);
    }
    mbar_init(&s.acc_full, 1);
    mbar_init(&s.acc_free, 4);
    mbar_init(&s.mma_drained, 1);
    s.abort_flag = 0;
    fence_barrier_init();
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
          tma_load_2d(g.a, &map_a, kb * 128, tm_i * kProjTileM, &s.full[st]);
          tma_load_2d(g.w, &map_w, kb * 128, tn_i * kProjTileN, &s.full[st]);
          bulk_load(g.a_sf, p.a_sf + ((int64_t)tm_i * pages_k + kb * 4) * 512, 4 * 512, &s.full[st]);
          bulk_load(g.w_sf[0], p.w_sf + ((int64_t)(2 * tn_i) * pages_k + kb * 4) * 512, 4 * 512, &s.full[st]);
          bulk_load(g.w_sf[1], p.w_sf + ((int64_t)(2 * tn_i + 1) * pages_k + kb * 4) * 512, 4 * 512, &s.full[st]);
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
          for (int k = 0; k < 4; ++k) {
            tmem_cp_page(sf + 4 * k, make_page_desc(smem_u32(g.a_sf + 512 * k)));
            tmem_cp_page(sf + 16 + 8 * k, make_page_desc(smem_u32(g.w_sf[0] + 512 * k)));
            tmem_cp_page(sf + 16 + 8 * k + 4, make_page_desc(smem_u32(g.w_sf[1] + 512 * k)));
          }
          const uint64_t da = make_tile_desc(smem_u32(g.a), 128), dw = make_tile_desc(smem_u32(g.w), 128);
#pragma unroll
          for (int k = 0; k < 4; ++k)
            mma_nvfp4_ss(tm, da + 2 * k, dw + 2 * k, idesc, sf + 4 * k, sf + 16 + 8 * k, (kb > 0 || k > 0) ? 1u : 0u);
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
    // ------------------------------------------------------------------ epilogue (warps 2-5)
    const int quarter = warp & 3;  // the TMEM lanes this warp may read
    const uint32_t lane_base = tm + ((uint32_t)(quarter * 32) << 16);
    const float gscale = __ldg(p.a_global) * __ldg(p.w_global);
    int n_done = 0;
    for (int tile = blockIdx.x; tile < n_tiles; tile += gridDim.x, ++n_done) {
      const int tm_i = tile / tiles_n, tn_i = tile % tiles_n;
      if (!mbar_wait_warp(&s.acc_full, n_done & 1, &s.abort_flag, p.status, 430, tile)) break;
      tc_fence_after();
      __nv_bfloat16* yrow = p.y + (int64_t)(tm_i * kProjTileM + quarter * 32 + lane) * p.ldy + (int64_t)tn_i * kProjTileN;
#pragma unroll 1
      for (int c = 0; c < kProjTileN / 32; ++c) {
        uint32_t v[32];
        tmem_ld32(lane_base + c * 32, v);
        tmem_ld_wait(v);
        if (c == kProjTileN / 32 - 1) {  // the accumulator is in registers: the next tile may overwrite it
          tc_fence_before();
          mbar_arrive_warp(&s.acc_free);
        }
        uint32_t w[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          const __nv_bfloat162 h2 = __floats2bfloat162_rn(__uint_as_float(v[2 * i]) * gscale, __uint_as_float(v[2 * i + 1]) * gscale);
          w[i] = *reinterpret_cast<const uint32_t*>(&h2);
        }
#pragma unroll
        for (int i = 0; i < 4; ++i) *reinterpret_cast<uint4*>(yrow + c * 32 + 8 * i) = make_uint4(w[4 * i], w[4 * i + 1], w[4 * i + 2], w[4 * i + 3]);
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tm, 512);
}

}  // namespace fa4b

using namespace fa4b;

int fa4b_project_nvfp4(const fa4b_project_nvfp4_args* a, void* stream) {
  FA4B_REQUIRE(a != nullptr, FA4B_BAD_ARG, "args is NULL");
  FA4B_REQUIRE(a->a_codes && a->a_scales && a->a_global && a->w_codes && a->w_scales && a->w_global && a->y && a->status, FA4B_BAD_ARG,
               "fa4b_project_nvfp4: NULL pointer");
  FA4B_REQUIRE(a->M > 0 && a->N > 0 && a->K > 0 && a->M % kProjTileM == 0 && a->N % kProjTileN == 0 && a->K % kProjStepK == 0, FA4B_BAD_SHAPE,
               "M=%lld N=%lld K=%lld: M must be a multiple of 128, N and K of 256", (long long)a->M, (long long)a->N, (long long)a->K);
  FA4B_REQUIRE(a->M < (1ll << 31) && a->N < (1ll << 31) && a->K < (1ll << 31), FA4B_BAD_SHAPE, "dimensions must fit 31 bits");
  FA4B_REQUIRE(a->ldy >= a->N && a->ldy % 8 == 0 && (reinterpret_cast<uintptr_t>(a->y) & 15) == 0, FA4B_BAD_ALIGN,
               "y must be 16-byte aligned with a row stride >= N that is a multiple of 8 elements");
  FA4B_REQUIRE(((reinterpret_cast<uintptr_t>(a->a_codes) | reinterpret_cast<uintptr_t>(a->w_codes) | reinterpret_cast<uintptr_t>(a->a_scales) |
                 reinterpret_cast<uintptr_t>(a->w_scales)) & 15) == 0, FA4B_BAD_ALIGN, "operands must be 16-byte aligned");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  FA4B_CUDA(cudaMemsetAsync(a->status, 0, 4 * sizeof(uint32_t), st));
  CUtensorMap ma{}, mw{};
  if (int s = make_tensor_map(&ma, a->a_codes, 1, (uint64_t)a->K / 2, (uint64_t)a->M, 0, (uint64_t)a->K / 2, 0, 128, kProjTileM)) return s;
  if (int s = make_tensor_map(&mw, a->w_codes, 1, (uint64_t)a->K / 2, (uint64_t)a->N, 0, (uint64_t)a->K / 2, 0, 128, kProjTileN)) return s;
  int dev = 0, sms = 0;
  FA4B_CUDA(cudaGetDevice(&dev));
  FA4B_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
  const int smem = sizeof(ProjSmem) + 1024;
  static std::once_flag once;
  static cudaError_t attr_err = cudaSuccess;
  std::call_once(once, [&] { attr_err = cudaFuncSetAttribute(project_nvfp4_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem); });
  FA4B_CUDA(attr_err);
  ProjParams p{};
  p.a_sf = a->a_scales; p.w_sf = a->w_scales;
  p.a_global = a->a_global; p.w_global = a->w_global;
  p.y = static_cast<__nv_bfloat16*>(a->y); p.ldy = a->ldy;
  p.M = (int)a->M; p.N = (int)a->N; p.K = (int)a->K;
  p.status = a->status;
  const int n_tiles = (p.M / kProjTileM) * (p.N / kProjTileN);
  project_nvfp4_kernel<<<std::min(n_tiles, sms), kProjThreads, smem, st>>>(p, ma, mw);
  FA4B_CUDA(cudaGetLastError());
  return FA4B_OK;
}

// Tensor-core self tests: one 128x128xK product per launch through the same
// tcgen05 instruction forms, shared-memory descriptors, swizzles and TMEM
// layouts that the attention kernels use.  Also home of the tensor-map helper.
#include <mutex>

#include "common.cuh"
#include "tc_sm100.cuh"

namespace fa4b {

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult qr;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qr) == cudaSuccess && qr == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  });
  return fn;
}

int make_tensor_map(CUtensorMap* out, const void* base, int elem_bytes, uint64_t inner, uint64_t rows, uint64_t outer,
                    uint64_t row_stride_bytes, uint64_t outer_stride_bytes, uint32_t box_inner, uint32_t box_rows) {
  EncodeTiledFn fn = encode_fn();
  FA4B_REQUIRE(fn != nullptr, FA4B_CUDA_ERROR, "cuTensorMapEncodeTiled is not available from this driver");
  FA4B_REQUIRE(elem_bytes == 1 || elem_bytes == 2, FA4B_BAD_ARG, "tensor map element size %d", elem_bytes);
  const uint32_t inner_bytes = box_inner * elem_bytes;
  CUtensorMapSwizzle swz = inner_bytes == 128 ? CU_TENSOR_MAP_SWIZZLE_128B
                           : inner_bytes == 64 ? CU_TENSOR_MAP_SWIZZLE_64B
                           : inner_bytes == 32 ? CU_TENSOR_MAP_SWIZZLE_32B
                                               : CU_TENSOR_MAP_SWIZZLE_NONE;
  const bool three = outer > 0;  // outer == 0 asks for a 2-D map
  cuuint64_t dims[3] = {inner, rows, outer ? outer : 1};
  cuuint64_t strides[2] = {row_stride_bytes, outer_stride_bytes};
  cuuint32_t box[3] = {box_inner, box_rows, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = fn(out, elem_bytes == 1 ? CU_TENSOR_MAP_DATA_TYPE_UINT8 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, three ? 3 : 2,
                  const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, swz,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  FA4B_REQUIRE(r == CUDA_SUCCESS, FA4B_CUDA_ERROR, "cuTensorMapEncodeTiled failed with CUresult %d", (int)r);
  return FA4B_OK;
}

int make_tensor_map_4d_bf16(CUtensorMap* out, const void* base, uint64_t inner, uint64_t rows, uint64_t d2, uint64_t d3,
                            uint64_t row_stride_bytes, uint64_t d2_stride_bytes, uint64_t d3_stride_bytes, uint32_t box_inner,
                            uint32_t box_rows) {
  EncodeTiledFn fn = encode_fn();
  if (fn == nullptr || box_inner * 2 != 128) return FA4B_CUDA_ERROR;
  // a dimension of extent 1 carries no stride of its own: give it the next inner one's span so that the encoder's
  // checks (multiples of 16, non-decreasing is not required) pass whatever the caller's view says
  cuuint64_t dims[4] = {inner, rows, d2, d3};
  cuuint64_t strides[3] = {row_stride_bytes, d2 > 1 ? d2_stride_bytes : row_stride_bytes * rows,
                           d3 > 1 ? d3_stride_bytes : (d2 > 1 ? d2_stride_bytes * d2 : row_stride_bytes * rows)};
  for (int i = 0; i < 3; ++i)
    if (strides[i] == 0 || (strides[i] & 15) != 0 || strides[i] >= (1ull << 40)) return FA4B_BAD_ALIGN;
  cuuint32_t box[4] = {box_inner, box_rows, 1, 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? FA4B_OK : FA4B_CUDA_ERROR;
}

struct GateSmem {
  alignas(1024) uint8_t a[128 * 128];
  alignas(1024) uint8_t b[128 * 128];
  alignas(16) uint8_t sfa[2 * 512];
  alignas(16) uint8_t sfb[2 * 512];
  alignas(8) uint64_t bar;
  alignas(8) uint64_t tma_bar;
  uint32_t tmem_base;
  alignas(8) volatile uint32_t abort_flag;
  uint32_t pad_;
};

// kinds: see fa4b_microgate in the public header; kind 7 = kind 1 with TMA loads
__global__ void __launch_bounds__(128, 1) microgate_kernel(int kind, int K, const uint8_t* __restrict__ a, const uint8_t* __restrict__ b,
                                                           const uint8_t* __restrict__ sfa, const uint8_t* __restrict__ sfb,
                                                           float* __restrict__ out, uint32_t* status,
                                                           const __grid_constant__ CUtensorMap map_a,
                                                           const __grid_constant__ CUtensorMap map_b) {
  extern __shared__ uint8_t raw[];
  GateSmem& s = *reinterpret_cast<GateSmem*>((reinterpret_cast<uintptr_t>(raw) + 1023) & ~uintptr_t(1023));
  const int t = threadIdx.x, warp = t >> 5;
  const bool fp4 = kind == 0 || kind == 6;
  const bool a_mn = kind == 4, b_mn = kind == 3 || kind == 4 || kind == 5;
  const bool a_tmem = kind == 5;
  // bytes per operand row in shared memory
  const uint32_t a_row = a_mn ? 128u : (fp4 ? K / 2 : K), b_row = b_mn ? 128u : (fp4 ? K / 2 : K);
  const uint32_t a_rows = a_mn ? K : 128u, b_rows = b_mn ? K : 128u;

  if (t == 0) {
    mbar_init(&s.bar, 1);
    mbar_init(&s.tma_bar, 1);
    s.abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == 0) tmem_alloc(&s.tmem_base, 256);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tm = s.tmem_base;
  const uint32_t tm_d = tm, tm_a = tm + 128, tm_sfa = tm + 192, tm_sfb = tm + 208;

  bool ok = true;
  if (kind == 7) {
    if (t == 0) {
      mbar_expect_tx(&s.tma_bar, 2 * 128 * K);
      tma_load_2d(s.a, &map_a, 0, 0, &s.tma_bar);
      tma_load_2d(s.b, &map_b, 0, 0, &s.tma_bar);
    }
    ok = mbar_wait(&s.tma_bar, 0, &s.abort_flag, status, 1);
  } else {
    // manual swizzled staging, 16-byte chunks
    if (!a_tmem) {
      const uint32_t chunks = a_rows * a_row / 16;
      for (uint32_t c = t; c < chunks; c += 128) {
        const uint32_t r = (c * 16) / a_row, cb = (c * 16) % a_row;
        *reinterpret_cast<uint4*>(&s.a[swizzled_offset(r, cb, a_row)]) = *reinterpret_cast<const uint4*>(a + (size_t)r * a_row + cb);
      }
    }
    const uint32_t chunks = b_rows * b_row / 16;
    for (uint32_t c = t; c < chunks; c += 128) {
      const uint32_t r = (c * 16) / b_row, cb = (c * 16) % b_row;
      *reinterpret_cast<uint4*>(&s.b[swizzled_offset(r, cb, b_row)]) = *reinterpret_cast<const uint4*>(b + (size_t)r * b_row + cb);
    }
    if (fp4) {
      const int pages = kind == 0 ? K / 64 : (K + 127) / 128;
      for (int c = t; c < pages * 32; c += 128) {
        *reinterpret_cast<uint4*>(&s.sfa[c * 16]) = *reinterpret_cast<const uint4*>(sfa + c * 16);
        *reinterpret_cast<uint4*>(&s.sfb[c * 16]) = *reinterpret_cast<const uint4*>(sfb + c * 16);
      }
    }
  }
  if (a_tmem) {
    // this thread's row of A (K bytes of E4M3) goes to TMEM columns tm_a .. tm_a + K/4
    const uint32_t lane_addr = tm_a + ((uint32_t)(warp * 32) << 16);
    for (int k0 = 0; k0 < K; k0 += 32) {
      uint32_t w[8];
      const uint4 v0 = *reinterpret_cast<const uint4*>(a + (size_t)t * K + k0);
      const uint4 v1 = *reinterpret_cast<const uint4*>(a + (size_t)t * K + k0 + 16);
      w[0] = v0.x; w[1] = v0.y; w[2] = v0.z; w[3] = v0.w; w[4] = v1.x; w[5] = v1.y; w[6] = v1.z; w[7] = v1.w;
      tmem_st8(lane_addr + k0 / 4, w);
    }
    tmem_st_wait();
  }
  fence_async_smem();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();

  if (t == 0 && ok) {
    const uint32_t sa = smem_u32(s.a), sb = smem_u32(s.b);
    if (fp4) {
      const bool mx = kind == 6;
      const int pages = mx ? (K + 127) / 128 : K / 64;
      for (int p = 0; p < pages; ++p) {
        tmem_cp_page(tm_sfa + 4 * p, make_page_desc(smem_u32(s.sfa + 512 * p)));
        tmem_cp_page(tm_sfb + 4 * p, make_page_desc(smem_u32(s.sfb + 512 * p)));
      }
      for (int k = 0; k < K / 64; ++k) {
        const uint64_t ad = make_tile_desc(sa + 32 * k, a_row), bd = make_tile_desc(sb + 32 * k, b_row);
        if (mx) {
          const uint32_t id = idesc_fp4(128, 128, 1, (k & 1) * 2, (k & 1) * 2);
          mma_mxfp4_ss(tm_d, ad, bd, id, tm_sfa + 4 * (k / 2), tm_sfb + 4 * (k / 2), k > 0);
        } else {
          mma_nvfp4_ss(tm_d, ad, bd, idesc_fp4(128, 128, 0, 0, 0), tm_sfa + 4 * k, tm_sfb + 4 * k, k > 0);
        }
      }
    } else {
      const uint32_t id = idesc_f8(128, 128, 0, kind == 2 ? 1 : 0, a_mn, b_mn);
      for (int k = 0; k < K / 32; ++k) {
        // K-major: 32 bytes further along the row; MN-major: 32 rows further down
        const uint64_t bd = make_tile_desc(sb + (b_mn ? 32 * 128 * k : 32 * k), b_row);
        if (a_tmem) {
          mma_f8_ts(tm_d, tm_a + 8 * k, bd, id, k > 0);
        } else {
          const uint64_t ad = make_tile_desc(sa + (a_mn ? 32 * 128 * k : 32 * k), a_row);
          mma_f8_ss(tm_d, ad, bd, id, k > 0);
        }
      }
    }
    mma_commit(&s.bar);
  }
  if (ok) ok = mbar_wait(&s.bar, 0, &s.abort_flag, status, 2);
  tc_fence_after();
  if (ok) {
    const uint32_t lane_addr = tm_d + ((uint32_t)(warp * 32) << 16);
#pragma unroll 1
    for (int c0 = 0; c0 < 128; c0 += 32) {
      uint32_t r[32];
      tmem_ld32(lane_addr + c0, r);
      tmem_ld_wait(r);
#pragma unroll
      for (int j = 0; j < 32; ++j) out[(size_t)t * 128 + c0 + j] = __uint_as_float(r[j]);
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tm, 256);
}

// ---- tensor-core peak: every SM issues a long run of MMAs on operands that stay in shared memory ----
// kind 0: kind::f8f6f4 E4M3 x E4M3, M128 N256 K32;  kind 1: kind::mxf4nvf4 block-scaled E2M1, M128 N256 K64.
// Operands are pseudo-random bytes (scale bytes 1.0), two 256-column accumulators alternate.
struct PeakSmem {
  alignas(1024) uint8_t a[128 * 128];
  alignas(1024) uint8_t b[256 * 128];
  alignas(16) uint8_t sf[512];
  alignas(8) uint64_t done;
  uint32_t tmem_base;
  alignas(8) volatile uint32_t abort_flag;
  uint32_t pad_;
};
__global__ void __launch_bounds__(128, 1) tensor_peak_kernel(int kind, int iters, uint32_t* status) {
  extern __shared__ uint8_t raw[];
  PeakSmem& s = *reinterpret_cast<PeakSmem*>((reinterpret_cast<uintptr_t>(raw) + 1023) & ~uintptr_t(1023));
  const int t = threadIdx.x, warp = t >> 5;
  for (int i = t; i < (128 + 256) * 128 / 4; i += 128) {
    uint32_t h = (uint32_t)i * 2654435761u + blockIdx.x * 40503u;
    h ^= h >> 15; h *= 2246822519u; h ^= h >> 13;
    // keep FP8 bytes finite (clear the top exponent bit of every byte): the timing does not depend on it, the power does not either
    reinterpret_cast<uint32_t*>(s.a)[i] = h & 0xBFBFBFBFu;
  }
  for (int i = t; i < 128; i += 128) reinterpret_cast<uint32_t*>(s.sf)[i] = 0x38383838u;  // E4M3 1.0
  if (t == 0) {
    mbar_init(&s.done, 1);
    s.abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == 0) tmem_alloc(&s.tmem_base, 512);
  fence_async_smem();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tm = s.tmem_base;
  if (warp == 1) {
    const bool leader = elect_one();
    if (leader) {
      if (kind == 0) {
        constexpr uint32_t id = idesc_f8(128, 256, 0, 0, 0, 0);
        for (int i = 0; i < iters; ++i) {
          const uint32_t acc = tm + ((i >> 2) & 1) * 256;
          const int k = i & 3;
          mma_f8_ss(acc, make_tile_desc(smem_u32(s.a) + 32 * k, 128), make_tile_desc(smem_u32(s.b) + 32 * k, 128), id, 1);
        }
      } else {
        // FP4 needs only 256 accumulator columns at a time here; the scale factors sit above them
        constexpr uint32_t id = idesc_fp4(128, 256, 0, 0, 0);
        const uint32_t sfa = tm + 480, sfb = tm + 488;
        tmem_cp_page(sfa, make_page_desc(smem_u32(s.sf)));
        tmem_cp_page(sfb, make_page_desc(smem_u32(s.sf)));
        tmem_cp_page(sfb + 4, make_page_desc(smem_u32(s.sf)));
        for (int i = 0; i < iters; ++i) {
          const int k = i & 3;
          mma_nvfp4_ss(tm + ((i >> 2) & 1) * 224, make_tile_desc(smem_u32(s.a) + 32 * k, 128), make_tile_desc(smem_u32(s.b) + 32 * k, 128), id, sfa,
                       sfb, 1);
        }
      }
      mma_commit(&s.done);
    }
    __syncwarp();
    mbar_wait_warp(&s.done, 0, &s.abort_flag, status, 300);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tm, 512);
}

}  // namespace fa4b

using namespace fa4b;

extern "C" int fa4b_microgate(int kind, int K, const void* a, const void* b, const void* sfa, const void* sfb, float* out,
                              uint32_t* status_out, void* stream) {
  FA4B_REQUIRE(kind >= 0 && kind <= 7, FA4B_UNSUPPORTED, "microgate kind %d", kind);
  FA4B_REQUIRE(a && b && out && status_out, FA4B_BAD_ARG, "microgate: NULL pointer");
  const bool fp4 = kind == 0 || kind == 6;
  FA4B_REQUIRE(!fp4 || (sfa && sfb), FA4B_BAD_ARG, "microgate: block-scaled kinds need scale pages");
  const bool mn = kind == 3 || kind == 4 || kind == 5;
  if (fp4) FA4B_REQUIRE(K == 64 || K == 128, FA4B_BAD_SHAPE, "microgate: FP4 K must be 64 or 128");
  else if (mn) FA4B_REQUIRE(K % 32 == 0 && K >= 32 && K <= 128, FA4B_BAD_SHAPE, "microgate: K must be 32..128, multiple of 32");
  else FA4B_REQUIRE(K == 32 || K == 64 || K == 128, FA4B_BAD_SHAPE, "microgate: K must be 32, 64 or 128");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  FA4B_CUDA(cudaMemsetAsync(status_out, 0, 4 * sizeof(uint32_t), st));
  CUtensorMap ma{}, mb{};
  if (kind == 7) {
    if (int s = make_tensor_map(&ma, a, 1, K, 128, 0, K, 0, K, 128)) return s;
    if (int s = make_tensor_map(&mb, b, 1, K, 128, 0, K, 0, K, 128)) return s;
  }
  const int smem = sizeof(GateSmem) + 1024;
  // the attribute belongs to the current device's context: set on every call (cheap) so that a second GPU of the process gets it too
  FA4B_CUDA(cudaFuncSetAttribute(microgate_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
  microgate_kernel<<<1, 128, smem, st>>>(kind, K, static_cast<const uint8_t*>(a), static_cast<const uint8_t*>(b),
                                         static_cast<const uint8_t*>(sfa), static_cast<const uint8_t*>(sfb), out, status_out, ma, mb);
  FA4B_CUDA(cudaGetLastError());
  return FA4B_OK;
}

extern "C" int fa4b_tensor_peak(int kind, int iters, uint32_t* status_out, void* stream) {
  FA4B_REQUIRE(kind == 0 || kind == 1, FA4B_UNSUPPORTED, "tensor_peak kind %d", kind);
  FA4B_REQUIRE(iters > 0 && iters <= (1 << 20) && status_out, FA4B_BAD_ARG, "tensor_peak: iters must be in 1..2^20, status_out non-NULL");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  FA4B_CUDA(cudaMemsetAsync(status_out, 0, 4 * sizeof(uint32_t), st));
  int dev = 0, sms = 0;
  FA4B_CUDA(cudaGetDevice(&dev));
  FA4B_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
  const int smem = sizeof(PeakSmem) + 1024;
  // the attribute belongs to the current device's context: set on every call (cheap) so that a second GPU of the process gets it too
  FA4B_CUDA(cudaFuncSetAttribute(tensor_peak_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
  tensor_peak_kernel<<<sms, 128, smem, st>>>(kind, iters, status_out);
  FA4B_CUDA(cudaGetLastError());
  return FA4B_OK;
}

// ---- wait self-test ------------------------------------------------------------------------------------------
// The give-up path of the bounded waits, exercised without a fault: two warps wait, with a short cycle budget, on
// barriers that are initialised and never armed -- nothing asynchronous is in flight, nothing is allocated in TMEM.
// Warp 0 uses the one-thread form, warp 1 the whole-warp form and (once warp 0 has raised the CTA's abort flag, or
// on its own budget) returns as well; both record where they gave up in `status` exactly as the attention kernels do.
__global__ void __launch_bounds__(64, 1) wait_selftest_kernel(long long limit, uint32_t* status, uint32_t* seen) {
  __shared__ alignas(8) uint64_t bar[2];
  __shared__ volatile uint32_t abort_flag;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    mbar_init(&bar[0], 1);
    mbar_init(&bar[1], 1);
    abort_flag = 0;
    fence_barrier_init();
  }
  __syncthreads();
  bool ok;
  if (warp == 0) {
    ok = lane == 0 ? mbar_wait(&bar[0], 0, &abort_flag, status, 900, 7, limit) : false;
    if (lane == 0) seen[0] = ok ? 1u : 0u;
  } else {
    ok = mbar_wait_warp(&bar[1], 0, &abort_flag, status, 901, 8, 4 * limit);
    if (lane == 0) seen[1] = ok ? 1u : 0u;
  }
  __syncthreads();
  if (threadIdx.x == 0) seen[2] = abort_flag;
}

extern "C" int fa4b_wait_selftest(int64_t limit_cycles, uint32_t* status_out, void* stream) {
  FA4B_REQUIRE(status_out != nullptr, FA4B_BAD_ARG, "wait_selftest: status_out is NULL");
  FA4B_REQUIRE(limit_cycles > 0 && limit_cycles <= (int64_t)100 * 1000 * 1000, FA4B_BAD_ARG,
               "wait_selftest: the cycle budget must be in 1..1e8 (this entry point is a short self-test)");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  FA4B_CUDA(cudaMemsetAsync(status_out, 0, 8 * sizeof(uint32_t), st));
  wait_selftest_kernel<<<1, 64, 0, st>>>((long long)limit_cycles, status_out, status_out + 4);
  FA4B_CUDA(cudaGetLastError());
  uint32_t host[8] = {};
  FA4B_CUDA(cudaMemcpyAsync(host, status_out, sizeof(host), cudaMemcpyDeviceToHost, st));
  FA4B_CUDA(cudaStreamSynchronize(st));
  // the barriers are never armed: a wait that reports success, or a missing give-up record, is the failure here
  FA4B_REQUIRE(host[4] == 0 && host[5] == 0 && host[6] == 1, FA4B_CUDA_ERROR, "wait_selftest: a wait on an unarmed barrier did not give up");
  FA4B_REQUIRE(host[0] == 0, FA4B_TIMEOUT, "a device-side wait ran out (site %u, block %u, detail %u)", host[1], host[2], host[3]);
  return FA4B_OK;
}

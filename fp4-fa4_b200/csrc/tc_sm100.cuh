// sm_100a primitives used by the attention kernels: mbarrier with bounded
// waits, TMA tile loads, TMEM allocation, tcgen05 MMA / commit / ld / st / cp,
// and the shared-memory and instruction descriptors they take.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace fa4b {

// every device-side wait gives up after this many SM clock cycles (about 0.4 s at 2 GHz),
// records where, and the kernel tears down (TMEM freed) instead of spinning
constexpr long long kWaitLimitCycles = 800ll * 1000 * 1000;

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

// ---- mbarrier ----------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void fence_barrier_init() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
// A failed try parks the thread until the phase completes or the hardware's time limit passes (a few microseconds).
// No suspend-time hint: with one, a try is a longer instruction sequence for every waiting warp, which cost the
// attention kernels 1 % (forward) and 3 % (backward) of their time once their waits had become short.
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{ .reg .pred p; mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2; selp.u32 %0, 1, 0, p; }"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
// Bounded wait.  `abort_flag` lives in shared memory: once any role has given up, every
// other wait of the CTA returns false at once so that all roles reach the teardown.
// status[0] = 1, status[1] = site, status[2] = block, status[3] = caller's detail word.
// The cycle counter is only consulted after a burst of polls, so a wait that is about to
// be satisfied never pays for it.
static __device__ __noinline__ bool mbar_wait_slow(uint64_t* bar, uint32_t parity, volatile uint32_t* abort_flag, uint32_t* status,
                                                   uint32_t where, uint32_t detail, long long limit) {
  const long long t0 = clock64();
  for (;;) {
#pragma unroll 1
    for (int i = 0; i < 64; ++i)
      if (mbar_try_wait(bar, parity)) return true;
    if (*abort_flag) return false;
    if (clock64() - t0 > limit) break;
  }
  *abort_flag = 1u;
  if (status && atomicCAS(status, 0u, 1u) == 0u) {
    status[1] = where;
    status[2] = blockIdx.x;
    status[3] = detail;
  }
  return false;
}
// Teardown wait: lets a role that has given up (or finished) make sure the asynchronous work it
// started -- bulk copies into its shared memory, tensor-core operations on its TMEM -- has landed
// before the CTA frees TMEM and exits.  Bounded (about 50 ms); ignores the abort flag.
static __device__ __noinline__ bool mbar_wait_teardown(uint64_t* bar, uint32_t parity) {
  const long long t0 = clock64();
  for (;;) {
#pragma unroll 1
    for (int i = 0; i < 64; ++i)
      if (mbar_try_wait(bar, parity)) return true;
    if (clock64() - t0 > kWaitLimitCycles / 8) return false;
  }
}

// `limit`: the cycle budget of this wait (the kernels use the default; the wait self-test passes a short one)
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, volatile uint32_t* abort_flag, uint32_t* status,
                                          uint32_t where, uint32_t detail = 0, long long limit = kWaitLimitCycles) {
  // one try parks the thread until the phase completes (or the hardware's limit passes), so the first one nearly always succeeds
  if (mbar_try_wait(bar, parity)) return true;
  return mbar_wait_slow(bar, parity, abort_flag, status, where, detail, limit);
}

// Whole-warp forms.  Every lane runs the same loop on a warp-wide vote, so the warp is still
// converged when the wait returns: the warp-collective tcgen05.ld/st that follow fault when lanes
// arrive separately (a version that put the polling loop under `if (lane == 0)`, and one whose
// lanes left their own polling loops at different iterations, both left lanes on paths of their
// own).  All 32 lanes poll: measured inside the running kernels that costs less than one
// predicated poll plus a broadcast (about 115 against 155 cycles; 16 and 28 on an idle SM).
__device__ __forceinline__ bool mbar_try_wait_uniform(uint64_t* bar, uint32_t parity) {
  return __all_sync(0xffffffffu, mbar_try_wait(bar, parity));
}
// non-blocking form for a warp that serves several barriers: test_wait never parks the thread
// (a failed try_wait may sleep for microseconds)
__device__ __forceinline__ bool mbar_test_uniform(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{ .reg .pred p; mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2; selp.u32 %0, 1, 0, p; }"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return __all_sync(0xffffffffu, ok != 0u);
}
static __device__ __noinline__ bool mbar_wait_warp_slow(uint64_t* bar, uint32_t parity, volatile uint32_t* abort_flag, uint32_t* status,
                                                        uint32_t where, uint32_t detail, long long limit) {
  const long long t0 = clock64();
  for (;;) {
#pragma unroll 1
    for (int i = 0; i < 64; ++i)
      if (mbar_try_wait_uniform(bar, parity)) return true;
    // lane 0 decides for the warp: 1 = another role gave up, 2 = out of time
    uint32_t stop = *abort_flag ? 1u : (clock64() - t0 > limit ? 2u : 0u);  // branch-free on every lane
    stop = __shfl_sync(0xffffffffu, stop, 0);
    if (stop == 1u) return false;
    if (stop == 2u) break;
  }
  if ((threadIdx.x & 31) == 0) {
    *abort_flag = 1u;
    if (status && atomicCAS(status, 0u, 1u) == 0u) {
      status[1] = where;
      status[2] = blockIdx.x;
      status[3] = detail;
    }
  }
  __syncwarp();
  return false;
}
__device__ __forceinline__ bool mbar_wait_warp(uint64_t* bar, uint32_t parity, volatile uint32_t* abort_flag, uint32_t* status,
                                               uint32_t where, uint32_t detail = 0, long long limit = kWaitLimitCycles) {
  if (mbar_try_wait_uniform(bar, parity)) return true;
  return mbar_wait_warp_slow(bar, parity, abort_flag, status, where, detail, limit);
}
// every lane must have issued its own fences before the call; the barrier counts one arrival per warp
__device__ __forceinline__ void mbar_arrive_warp(uint64_t* bar) {
  __syncwarp();
  asm volatile("{ .reg .pred q; setp.eq.u32 q, %1, 0; @q mbarrier.arrive.shared::cta.b64 _, [%0]; }" ::"r"(smem_u32(bar)),
               "r"(threadIdx.x & 31u)
               : "memory");
}

// ---- proxies and fences -----------------------------------------------------------
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// ---- TMA ---------------------------------------------------------------------------
__device__ __forceinline__ void tma_load_2d(void* smem_dst, const CUtensorMap* map, int x, int y, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];" ::"r"(
          smem_u32(smem_dst)),
      "l"(map), "r"(smem_u32(bar)), "r"(x), "r"(y)
      : "memory");
}
__device__ __forceinline__ void tma_load_3d(void* smem_dst, const CUtensorMap* map, int x, int y, int z, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];" ::"r"(
          smem_u32(smem_dst)),
      "l"(map), "r"(smem_u32(bar)), "r"(x), "r"(y), "r"(z)
      : "memory");
}
__device__ __forceinline__ void tma_load_4d(void* smem_dst, const CUtensorMap* map, int x, int y, int z, int w, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];" ::"r"(
          smem_u32(smem_dst)),
      "l"(map), "r"(smem_u32(bar)), "r"(x), "r"(y), "r"(z), "r"(w)
      : "memory");
}
// TMA store of one box from shared memory (bulk async-group completion)
__device__ __forceinline__ void tma_store_2d(const CUtensorMap* map, const void* smem_src, int x, int y) {
  asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];" ::"l"(map), "r"(smem_u32(smem_src)), "r"(x),
               "r"(y)
               : "memory");
}
__device__ __forceinline__ void tma_store_3d(const CUtensorMap* map, const void* smem_src, int x, int y, int z) {
  asm volatile("cp.async.bulk.tensor.3d.global.shared::cta.bulk_group [%0, {%2, %3, %4}], [%1];" ::"l"(map), "r"(smem_u32(smem_src)),
               "r"(x), "r"(y), "r"(z)
               : "memory");
}
// untiled bulk copy shared -> global (16-byte aligned, size % 16 == 0), same completion group as the TMA stores
__device__ __forceinline__ void bulk_store(void* gdst, const void* smem_src, uint32_t bytes) {
  asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(gdst), "r"(smem_u32(smem_src)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void tma_store_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
// every committed store group of this thread has finished reading its shared-memory source
__device__ __forceinline__ void tma_store_wait_read() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }
__device__ __forceinline__ void tma_prefetch_desc(const CUtensorMap* map) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(map) : "memory");
}
// untiled bulk copy global -> shared (16-byte aligned, size % 16 == 0)
__device__ __forceinline__ void bulk_load(void* smem_dst, const void* gsrc, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(smem_u32(smem_dst)),
               "l"(gsrc), "r"(bytes), "r"(smem_u32(bar))
               : "memory");
}

// ---- TMEM --------------------------------------------------------------------------
// one full warp; writes the base address to *dst (shared)
__device__ __forceinline__ void tmem_alloc(uint32_t* dst, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(dst)), "r"(ncols) : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}

#define FA4B_R8(r, o) "=r"(r[o + 0]), "=r"(r[o + 1]), "=r"(r[o + 2]), "=r"(r[o + 3]), "=r"(r[o + 4]), "=r"(r[o + 5]), "=r"(r[o + 6]), "=r"(r[o + 7])
// 32 consecutive f32 columns of this thread's lane
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
      : FA4B_R8(r, 0), FA4B_R8(r, 8), FA4B_R8(r, 16), FA4B_R8(r, 24)
      : "r"(taddr));
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
      : FA4B_R8(r, 0), FA4B_R8(r, 8)
      : "r"(taddr));
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
#define FA4B_RW8(r, o) "+r"(r[o + 0]), "+r"(r[o + 1]), "+r"(r[o + 2]), "+r"(r[o + 3]), "+r"(r[o + 4]), "+r"(r[o + 5]), "+r"(r[o + 6]), "+r"(r[o + 7])
// wait for the loads and make the compiler treat the registers as produced here
__device__ __forceinline__ void tmem_ld_wait(uint32_t (&r)[32]) {
  asm volatile("tcgen05.wait::ld.sync.aligned;" : FA4B_RW8(r, 0), FA4B_RW8(r, 8), FA4B_RW8(r, 16), FA4B_RW8(r, 24)::"memory");
}
__device__ __forceinline__ void tmem_ld_wait16(uint32_t (&r)[16]) {
  asm volatile("tcgen05.wait::ld.sync.aligned;" : FA4B_RW8(r, 0), FA4B_RW8(r, 8)::"memory");
}
__device__ __forceinline__ void tmem_st8(uint32_t taddr, const uint32_t (&r)[8]) {
  asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};" ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]),
               "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7])
               : "memory");
}
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};" ::"r"(
          taddr),
      "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]),
      "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]),
      "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
      : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// ---- descriptors ---------------------------------------------------------------------
// Shared-memory matrix descriptor: start address >> 4 in bits 0-13, leading byte
// offset >> 4 in 16-29, stride byte offset >> 4 in 32-45, version 1 in 46-47,
// swizzle mode in 61-63 (0 none, 2 = 128 B, 4 = 64 B, 6 = 32 B).
enum : uint32_t { kSwzNone = 0, kSwz128 = 2, kSwz64 = 4, kSwz32 = 6 };
__device__ __forceinline__ uint64_t make_sdesc(uint32_t smem_addr, uint32_t lbo_bytes, uint32_t sbo_bytes, uint32_t swizzle) {
  return (uint64_t)((smem_addr & 0x3FFFFu) >> 4) | ((uint64_t)(lbo_bytes >> 4) << 16) | ((uint64_t)(sbo_bytes >> 4) << 32) |
         (1ull << 46) | ((uint64_t)swizzle << 61);
}
// A tile whose rows are `row_bytes` (32, 64 or 128) wide, swizzled with the mode of
// that width, eight rows per swizzle atom.  Serves K-major operands (rows = M or N)
// and MN-major operands (rows = K) alike; the major-ness is in the instruction descriptor.
__device__ __forceinline__ uint64_t make_tile_desc(uint32_t smem_addr, uint32_t row_bytes) {
  const uint32_t swz = row_bytes == 128 ? kSwz128 : row_bytes == 64 ? kSwz64 : kSwz32;
  return make_sdesc(smem_addr, 16, 8 * row_bytes, swz);
}
// 512-byte scale page: 32 rows x 16 bytes, no swizzle
__device__ __forceinline__ uint64_t make_page_desc(uint32_t smem_addr) { return make_sdesc(smem_addr, 128, 128, kSwzNone); }

// byte offset of (row, byte column) inside a swizzled tile with `row_bytes` rows
__device__ __host__ __forceinline__ uint32_t swizzled_offset(uint32_t row, uint32_t col_byte, uint32_t row_bytes) {
  const uint32_t lin = row * row_bytes + col_byte;
  const uint32_t mask = row_bytes == 128 ? 7u : row_bytes == 64 ? 3u : 1u;
  return lin ^ (((lin >> 7) & mask) << 4);
}

// Instruction descriptor, kind::f8f6f4, f32 accumulate.  fmt: 0 = E4M3, 1 = E5M2;
// *_mn = 1 for an MN-major operand.
__device__ __host__ constexpr uint32_t idesc_f8(uint32_t M, uint32_t N, uint32_t a_fmt, uint32_t b_fmt, uint32_t a_mn, uint32_t b_mn) {
  return (1u << 4) | (a_fmt << 7) | (b_fmt << 10) | (a_mn << 15) | (b_mn << 16) | ((N >> 3) << 17) | ((M >> 4) << 24);
}
// Block-scaled FP4 (kind::mxf4nvf4 with UE4M3 scales, or kind::mxf4 with UE8M0):
// E2M1 operands (format code 1), both K-major, K = 64 per instruction.
__device__ __host__ constexpr uint32_t idesc_fp4(uint32_t M, uint32_t N, uint32_t e8m0_scales, uint32_t a_sf_id, uint32_t b_sf_id) {
  return (b_sf_id << 4) | (1u << 7) | (1u << 10) | ((N >> 3) << 17) | (e8m0_scales << 23) | ((M >> 4) << 24) | (a_sf_id << 29);
}

// one lane of a fully converged warp; the same lane every time
__device__ __forceinline__ bool elect_one() {
  uint32_t pred;
  asm volatile("{ .reg .pred p; elect.sync _|p, 0xffffffff; selp.u32 %0, 1, 0, p; }" : "=r"(pred));
  return pred != 0;
}

// ---- MMA issue (one thread) --------------------------------------------------------------
__device__ __forceinline__ void mma_f8_ss(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{ .reg .pred p; setp.ne.b32 p, %4, 0; tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, p; }" ::"r"(d_tmem),
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void mma_f8_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{ .reg .pred p; setp.ne.b32 p, %4, 0; tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], [%1], %2, %3, p; }" ::"r"(d_tmem),
      "r"(a_tmem), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void mma_nvfp4_ss(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t sfa_tmem,
                                             uint32_t sfb_tmem, uint32_t accumulate) {
  asm volatile(
      "{ .reg .pred p; setp.ne.b32 p, %4, 0; "
      "tcgen05.mma.cta_group::1.kind::mxf4nvf4.block_scale.scale_vec::4X [%0], %1, %2, %3, [%5], [%6], p; }" ::"r"(d_tmem),
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(sfa_tmem), "r"(sfb_tmem)
      : "memory");
}
__device__ __forceinline__ void mma_mxfp4_ss(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t sfa_tmem,
                                             uint32_t sfb_tmem, uint32_t accumulate) {
  asm volatile(
      "{ .reg .pred p; setp.ne.b32 p, %4, 0; "
      "tcgen05.mma.cta_group::1.kind::mxf4.block_scale.scale_vec::2X [%0], %1, %2, %3, [%5], [%6], p; }" ::"r"(d_tmem),
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(sfa_tmem), "r"(sfb_tmem)
      : "memory");
}
// all previously issued MMAs of this thread arrive on `bar` when they complete
__device__ __forceinline__ void mma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
// 32 rows x 16 bytes from shared memory to 4 TMEM columns, replicated to the four lane quarters
__device__ __forceinline__ void tmem_cp_page(uint32_t taddr, uint64_t sdesc) {
  asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;" ::"r"(taddr), "l"(sdesc) : "memory");
}

// ---- host: tensor maps --------------------------------------------------------------------
// Row-major tensor of `elem_bytes` elements, 3-D [outer, rows, inner] (2-D when outer == 0);
// the box is box_inner x box_rows (x 1), swizzled with the mode that matches the inner box
// width in bytes.
int make_tensor_map(CUtensorMap* out, const void* base, int elem_bytes, uint64_t inner, uint64_t rows, uint64_t outer,
                    uint64_t row_stride_bytes, uint64_t outer_stride_bytes, uint32_t box_inner, uint32_t box_rows);

// bf16 tensor [d3][d2][rows][inner] whose three outer strides (in bytes, multiples of 16) are free; the box is
// box_inner x box_rows x 1 x 1 with the 128-byte swizzle (box_inner = 64).  Returns a status without setting the
// error text when the driver refuses the strides: the caller then takes its path without TMA.
int make_tensor_map_4d_bf16(CUtensorMap* out, const void* base, uint64_t inner, uint64_t rows, uint64_t d2, uint64_t d3,
                            uint64_t row_stride_bytes, uint64_t d2_stride_bytes, uint64_t d3_stride_bytes, uint32_t box_inner,
                            uint32_t box_rows);

}  // namespace fa4b

// Causal GQA backward.  One CTA owns a 128-key tile of one kv head: dK and dV of
// that tile accumulate in TMEM over every query head of the group and every
// query tile at or after the key tile; dQ contributions leave as reductions
// (f16 pairs through the copy engine, or FP32) into a scratch accumulator that a
// second kernel rounds to bf16.
//
// Per query sub-tile (QT = 64 rows at D = 128, 128 rows at D = 64) five MMAs:
//   S^T  = Knvfp4 . Qnvfp4^T            block-scaled FP4   -> TMEM St  [key, q]
//   dP^T = V8 . dO5^T                   E4M3 x E5M2        -> TMEM dPt [key, q]
//   dV  += P8^T . dO5                   A = P8^T (smem), B = dO5 MN-major
//   dK  += dS8^T . Q8                   A = dS8^T (smem), B = Q8 MN-major
//   dQ   = dS8 . K8  (D = 64)  or  dQ^T = K8^T . dS8^T (D = 128), both operands MN-major
// with P8 = E4M3(2^min(S2 + lstat, 8)) and dS8 = E4M3((dP16 + dstat) * P8 * scale/16)
// computed by two groups of eight warps (two threads per key row each); group 0 takes the even
// sub-tiles and group 1 the odd ones, so one group's exponentials overlap the other group's waits.
// Each group owns one TMEM buffer that first holds S^T and then, once P has been read out of it,
// dP^T of the same sub-tile.  A group's chain S^T -> P -> dP^T -> dS -> next S^T sets the kernel's rate (two
// sub-tiles are in flight; a third group's buffer does not fit the 512 TMEM columns beside a 64-column dQ
// accumulator), so both tensor-core round trips of the chain are taken off it: dP^T is issued as soon as the
// group has READ the scores out of the buffer (it forms while the group computes P) and the next S^T as soon as
// it has READ dP^T (it forms while the group computes dS).
//
// Warps: 0-7 compute group 0, 8-15 compute group 1, 16-19 drain dQ, 20 TMA producer, 21-23 MMA issuers.
#include <cstdlib>
#include <mutex>

#include "attn.cuh"

namespace fa4b {

constexpr int kBwdThreads = 768;
constexpr int kBwdStages = 5;

template <int D>
struct BwdCfg {
  static constexpr int QT = (D == 128) ? 64 : 128;  // query rows per iteration
  static constexpr int kPages = D / 64;
  static constexpr uint32_t colDK = 0, colDV = D, colX = 2 * D, colDQ = 2 * D + 2 * QT;  // colX + g * QT: S^T / dP^T of group g
  static constexpr uint32_t colSfa = colDQ + 64, colSfb = colSfa + 8;
  static_assert(colSfb + 8 <= 512, "TMEM budget");
};

template <int D>
struct BwdSmem {
  using C = BwdCfg<D>;
  alignas(1024) uint8_t k_codes[128 * D / 2];
  alignas(1024) uint8_t k8[128 * D];
  alignas(1024) uint8_t v8[128 * D];
  alignas(1024) uint8_t q_codes[kBwdStages][C::QT * D / 2];
  alignas(1024) uint8_t q8[kBwdStages][C::QT * D];
  alignas(1024) uint8_t do5[kBwdStages][C::QT * D];
  alignas(1024) uint8_t pt[2][128 * C::QT];   // P8^T  [key][q], rows of QT bytes, swizzled
  alignas(1024) uint8_t dst[2][128 * C::QT];  // dS8^T [key][q]
  alignas(16) uint8_t k_sf[C::kPages * 512];
  alignas(16) uint8_t q_sf[kBwdStages][C::kPages * 512];
  alignas(16) float lstat[kBwdStages][C::QT];
  alignas(16) float dstat[kBwdStages][C::QT];
  alignas(16) float dq_patch[D == 64 ? 4 : 1][D == 64 ? 32 * 33 : 1];  // D = 64: per drain warp, 32 x 32 transposition patch
  // D = 128, f16 dQ sums: per drain warp the sub-tile's 32 row pairs x 32 features as words, in the accumulator's own
  // order, two buffers: the source of one bulk reduction per warp and sub-tile
  alignas(128) uint32_t dq_tile[D == 128 ? 2 : 1][D == 128 ? 4 : 1][D == 128 ? 32 * 32 : 4];
  alignas(16) float c2[16];  // per query head of the group: global scales * softmax scale * log2(e)
  alignas(8) uint64_t kv_full, in_full[kBwdStages], in_empty[kBwdStages], st_full[2], dp_full[2], dv_done[2], pt_ready[2], s_read[2], x_free[2], ds_ready[2], dq_full, dq_free,
      acc_done, mma_drained;
  uint32_t tmem_base;
  alignas(8) volatile uint32_t abort_flag;
  uint32_t pad_;
};

static_assert(sizeof(BwdSmem<128>) + 1024 <= 227 * 1024 && sizeof(BwdSmem<64>) + 1024 <= 227 * 1024, "shared memory budget");

struct BwdParams {
  int B, Hq, Hkv, S;
  int causal;  // 0: every key of the tile is visible to every query (a key shard that precedes the query shard)
  float scale;
  const uint8_t* q_sf;
  const uint8_t* k_sf;
  const float* q_global;
  const float* k_global;
  const float* lstat;
  const float* dstat;
  float* dq_accum;  // [B*Hq, S, D] f32, zeroed before launch; or (dq_half) packed f16 pairs, see below
  // dq_half: the dQ sums are kept as f16 (32 * dQ), two per 32-bit word, so that a drain warp's reduction still
  // moves 128 contiguous bytes but twice the values.  D = 128 (a drain lane holds one feature of 64 query rows): a
  // word holds row q (even) in its low half and row q + 1 in its high half; the 32 x 128 words of a sub-tile of 64
  // query rows form one block, ordered (feature / 32, row pair, feature % 32) so that what one drain warp adds is
  // contiguous: word ((bh * S / 2 + q / 64 * 32) * D + d / 32 * 1024 + q % 64 / 2 * 32 + d % 32).
  // D = 64 (a drain lane holds one query row): plain rows, word ((bh * S + q) * D / 2 + d / 2).
  int dq_half;
  __nv_bfloat16* dk;
  int64_t dk_sb, dk_sh, dk_ss;
  __nv_bfloat16* dv;
  int64_t dv_sb, dv_sh, dv_ss;
  uint32_t* status;
  // work list: every key tile's query range is cut into parts of at most `chunk` query tiles
  int chunk;           // query tiles per work item
  int items_per_head;  // work items of one (batch, kv head)
  int head_group;      // (batch, kv head) units whose items are launched side by side
  float* dk_accum;     // [B*Hkv, S, D] f32 each: sums of the parts of key tiles that were cut (zeroed before launch)
  float* dv_accum;
};


// f16 dQ sums hold the accumulator's value (1024 dQ) times this: 32 dQ, finite up to |dQ| = 2047
constexpr float kDqHalfScale = 1.0f / 32.0f;

__device__ __forceinline__ float ex2_approx_b(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
// The drain warps' reductions go through the same load/store queue as every other warp of their scheduler; 64 of
// them back to back fill it, and the barrier polls, shared-memory accesses and MMA issues of the compute and issuer
// warps wait behind them.  So the drain stops for about 60 cycles after every eighth reduction (a spin on the cycle
// counter: a sleep or a chain of dependent shared-memory loads in its place was slower).
__device__ __forceinline__ void drain_pause() {
  const long long t0 = clock64();
  while (clock64() - t0 < 60) {
  }
}
// four adjacent FP32 sums in one reduction (16-byte aligned)
__device__ __forceinline__ void red_add_v4(float* addr, float a, float b, float c, float d) {
  asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(addr), "f"(a), "f"(b), "f"(c), "f"(d) : "memory");
}
__device__ __forceinline__ float2 e4m3x2_to_f32(uint32_t two_bytes) {
  uint32_t h2;
  const uint16_t in = (uint16_t)two_bytes;
  asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(h2) : "h"(in));
  return __half22float2(*reinterpret_cast<const __half2*>(&h2));
}

template <int D>
__global__ void __launch_bounds__(kBwdThreads, 1)
attn_bwd_kernel(const BwdParams p, const __grid_constant__ CUtensorMap map_kc, const __grid_constant__ CUtensorMap map_k8,
                const __grid_constant__ CUtensorMap map_v8, const __grid_constant__ CUtensorMap map_qc,
                const __grid_constant__ CUtensorMap map_q8, const __grid_constant__ CUtensorMap map_do) {
  using C = BwdCfg<D>;
  constexpr int QT = C::QT;
  constexpr int kPages = C::kPages;
  extern __shared__ uint8_t raw[];
  // aligned by offsetting the shared array itself, so that accesses stay shared-space loads and stores
  BwdSmem<D>& s = *reinterpret_cast<BwdSmem<D>*>(raw + ((1024u - (smem_u32(raw) & 1023u)) & 1023u));
  const int t = threadIdx.x, warp = t >> 5, lane = t & 31;

  const int n_tiles = p.S / 128;
  // Work item = (key tile, part of the tile's query range, batch and kv head).  The (batch, kv head) units run in
  // groups of `head_group`: inside a group the order is key-tile-major -- the key tiles that see the most query
  // tiles start first, the group's heads side by side -- and the group is small enough that the FP32 dQ rows its
  // CTAs add into stay in L2 until their last partial sum has arrived (all heads at once evict and re-fetch every
  // line several times; one head at a time was slower: its long key tiles start late).  When the launch has few
  // units a tile's query range is cut into parts of at most `chunk` query tiles, so that the work still spreads
  // over every SM.
  const int heads_kv = p.B * p.Hkv;
  const int per_group = p.items_per_head * p.head_group;
  const int first_head = ((int)blockIdx.x / per_group) * p.head_group;
  const int in_group = (int)blockIdx.x % per_group;
  const int group_heads = min(p.head_group, heads_kv - first_head);  // the last group may be short
  const BwdItem item = bwd_item_of(in_group / group_heads, n_tiles, p.chunk, p.causal != 0);
  const int kt = item.kt;
  const int bhk = first_head + in_group % group_heads;
  const int b = bhk / p.Hkv, hk = bhk % p.Hkv;
  const int G = p.Hq / p.Hkv;
  const int sub_per_tile = 128 / QT;
  const int n_sub = (item.qt_hi - item.qt_lo) * sub_per_tile;  // query sub-tiles per head
  const int n_it = G * n_sub;
  const int sub0 = item.qt_lo * sub_per_tile;
  // it -> (it / n_sub, it % n_sub) without a division per use: exact for it * n_sub < 2^32
  const uint32_t n_sub_inv = 0xFFFFFFFFu / (uint32_t)n_sub + 1u;
  auto head_of = [&](int it) { return n_sub == 1 ? it : (int)__umulhi((uint32_t)it, n_sub_inv); };
  {
    // an earlier CTA of this launch gave up: leave at once, as one (the decision is CTA-uniform)
    __shared__ uint32_t skip;
    if (t == 0) skip = *reinterpret_cast<volatile uint32_t*>(p.status);
    __syncthreads();
    if (skip != 0u) return;
  }

  if (t == 0) {
    mbar_init(&s.kv_full, 1);
    for (int i = 0; i < kBwdStages; ++i) {
      mbar_init(&s.in_full[i], 1);
      mbar_init(&s.in_empty[i], 2);  // the S/dK stream and the dQ stream each release a stage
    }
    for (int i = 0; i < 2; ++i) {  // one set per compute group
      mbar_init(&s.st_full[i], 1);
      mbar_init(&s.dp_full[i], 1);
      mbar_init(&s.dv_done[i], 1);
      mbar_init(&s.pt_ready[i], 8);  // one arrival per compute warp
      mbar_init(&s.x_free[i], 8);
      mbar_init(&s.s_read[i], 8);
      mbar_init(&s.ds_ready[i], 8);
    }
    mbar_init(&s.dq_full, 1);
    mbar_init(&s.dq_free, 4);
    mbar_init(&s.acc_done, 3);     // one commit per issuer warp
    mbar_init(&s.mma_drained, 3);
    s.abort_flag = 0;
    fence_barrier_init();
    // the key tile's operands start on their way at once: their latency runs under the rest of the set-up
    mbar_expect_tx(&s.kv_full, 128 * D / 2 + kPages * 512 + 2 * 128 * D);
    tma_load_3d(s.k_codes, &map_kc, 0, kt * 128, bhk, &s.kv_full);
    bulk_load(s.k_sf, p.k_sf + ((size_t)bhk * n_tiles + kt) * kPages * 512, kPages * 512, &s.kv_full);
    tma_load_3d(s.k8, &map_k8, 0, kt * 128, bhk, &s.kv_full);
    tma_load_3d(s.v8, &map_v8, 0, kt * 128, bhk, &s.kv_full);
  }
  if (t < 16) s.c2[t] = (t < G) ? p.k_global[bhk] * p.scale * kLog2e * p.q_global[b * p.Hq + hk * G + t] : 0.f;
  if (warp == 20) tmem_alloc(&s.tmem_base, 512);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tm = s.tmem_base;

  if (warp == 20) {
    // ------------------------------------------------------------------ producer
    if (lane == 0) {
      int issued = 0;
      for (int it = 0; it < n_it; ++it) {
        const int st = it % kBwdStages;
        if (it >= kBwdStages && !mbar_wait(&s.in_empty[st], ((it / kBwdStages) - 1) & 1, &s.abort_flag, p.status, 110, it)) break;
        issued = it + 1;
        const int g = head_of(it), qs = sub0 + it - g * n_sub;
        const int bh = b * p.Hq + hk * G + g;
        const int q0 = qs * QT;
        mbar_expect_tx(&s.in_full[st], QT * D / 2 + kPages * 512 + 2 * QT * D + 2 * QT * 4);
        tma_load_3d(s.q_codes[st], &map_qc, 0, q0, bh, &s.in_full[st]);
        bulk_load(s.q_sf[st], p.q_sf + ((size_t)bh * n_tiles + q0 / 128) * kPages * 512, kPages * 512, &s.in_full[st]);
        tma_load_3d(s.q8[st], &map_q8, 0, q0, bh, &s.in_full[st]);
        tma_load_3d(s.do5[st], &map_do, 0, q0, bh, &s.in_full[st]);
        bulk_load(s.lstat[st], p.lstat + (size_t)bh * p.S + q0, QT * 4, &s.in_full[st]);
        bulk_load(s.dstat[st], p.dstat + (size_t)bh * p.S + q0, QT * 4, &s.in_full[st]);
      }
      // no copy of this CTA may still be in flight when its shared memory is given up, and the
      // tensor core's arrivals on the stage barriers must have landed too (nobody else waits for
      // the last ones)
      mbar_wait_teardown(&s.kv_full, 0);
      for (int it = issued > kBwdStages ? issued - kBwdStages : 0; it < issued; ++it) {
        mbar_wait_teardown(&s.in_full[it % kBwdStages], (it / kBwdStages) & 1);
        if (issued == n_it && !s.abort_flag) mbar_wait_teardown(&s.in_empty[it % kBwdStages], (it / kBwdStages) & 1);
      }
    }
  } else if (warp >= 21) {
    // ------------------------------------------------------------------ MMA issuers (warps 21-23)
    // Three warps, one per in-order stream of tensor-core work, so that no stream's wait holds up another's
    // issue: warp 21 answers pt_ready (dV, dP); warp 22 answers ds_ready with S of the group's next sub-tile
    // and dK; warp 23 answers ds_ready with dQ once the drain has handed the dQ accumulator back.  A whole
    // warp runs each loop so that control flow and descriptors stay warp-uniform; one elected lane (always
    // the same) issues the tensor-core instructions and their commits.  A commit covers only the issuing
    // thread's operations, so every reuse of a buffer that another stream reads is ordered through a barrier
    // that the reader's own stream commits, or through the compute warps' observation of one.
    {
      const int stream = warp - 21;  // 0: dV, dP   1: S, dK   2: dQ
      const bool leader = elect_one();
      constexpr uint32_t id_s = idesc_fp4(128, QT, 0, 0, 0);
      constexpr uint32_t id_dp = idesc_f8(128, QT, 0, 1, 0, 0);   // V8 (E4M3, K-major) x dO5 (E5M2, K-major)
      constexpr uint32_t id_dv = idesc_f8(128, D, 0, 1, 0, 1);    // P8^T (K-major) x dO5 (MN-major)
      constexpr uint32_t id_dk = idesc_f8(128, D, 0, 0, 0, 1);    // dS8^T (K-major) x Q8 (MN-major)
      constexpr uint32_t id_dq = idesc_f8(128, 64, 0, 0, 1, 1);   // both MN-major
      // The issuing thread shares its scheduler with busy compute warps, so its instruction count
      // bounds the issue rate: every descriptor is a precomputed base plus a small constant
      // (the address field counts 16-byte units).
      const uint64_t d_kc = make_tile_desc(smem_u32(s.k_codes), D / 2), d_k8 = make_tile_desc(smem_u32(s.k8), D);
      const uint64_t d_v8 = make_tile_desc(smem_u32(s.v8), D);
      const uint64_t d_qc0 = make_tile_desc(smem_u32(s.q_codes[0]), D / 2), d_q80 = make_tile_desc(smem_u32(s.q8[0]), D);
      const uint64_t d_do0 = make_tile_desc(smem_u32(s.do5[0]), D);
      const uint64_t d_pt0 = make_tile_desc(smem_u32(s.pt[0]), QT), d_ds0 = make_tile_desc(smem_u32(s.dst[0]), QT);
      const uint64_t d_sfq0 = make_page_desc(smem_u32(s.q_sf[0]));
      constexpr uint32_t kQc16 = (QT * D / 2) >> 4, kQ816 = (QT * D) >> 4, kSf16 = (kPages * 512) >> 4, kPt16 = (128 * QT) >> 4;
      constexpr uint32_t kRow32D = (32 * D) >> 4, kRow32Q = (32 * QT) >> 4;
      bool ok = mbar_wait_warp(&s.kv_full, 0, &s.abort_flag, p.status, 120);
      if (ok) {
        tc_fence_after();
#pragma unroll
        for (int pg = 0; pg < kPages; ++pg)
          if (leader && stream == 1) tmem_cp_page(tm + C::colSfa + 4 * pg, make_page_desc(smem_u32(s.k_sf + 512 * pg)));
      }
      // S^T of sub-tile `it` (inputs in its stage) into the buffer of the sub-tile's group; the caller
      // has made sure the buffer is free
      auto stage_of = [](int it) { return (uint32_t)(it % kBwdStages); };
      // in two parts: the scale factors go to TMEM as soon as the stage has landed (in order behind the
      // previous S on this thread), the MMAs follow when the buffer is free
      auto prep_s = [&](int it) -> bool {
        const uint32_t st = stage_of(it);
        if (!mbar_wait_warp(&s.in_full[st], (it / kBwdStages) & 1, &s.abort_flag, p.status, 121, it)) return false;
        tc_fence_after();
        if (leader) {
#pragma unroll
          for (int pg = 0; pg < kPages; ++pg) tmem_cp_page(tm + C::colSfb + 4 * pg, d_sfq0 + st * kSf16 + (pg * 512 >> 4));
        }
        __syncwarp();
        return true;
      };
      auto fire_s = [&](int it) {
        const uint32_t st = stage_of(it), g = it & 1;
        // D = 128: which 64 rows of the 128-row scale page (sub-tiles alternate, sub0 is even)
        const uint32_t sf_shift = (QT == 64) ? 2u * (uint32_t)(it & 1) : 0u;  // n_sub is even at QT = 64
        if (leader) {
          const uint64_t qc = d_qc0 + st * kQc16;
#pragma unroll
          for (int k = 0; k < D / 64; ++k)
            mma_nvfp4_ss(tm + C::colX + g * QT, d_kc + 2 * k, qc + 2 * k, id_s, tm + C::colSfa + 4 * k, tm + C::colSfb + 4 * k + sf_shift, k > 0);
          mma_commit(&s.st_full[g]);
        }
        __syncwarp();
      };
      // The two compute groups alternate sub-tiles and each runs  P(it); dS(it).  Per sub-tile:
      //   s_read(it)   -> dP(it) into the group's buffer (the scores have been read out of it), committed on its own
      //                   because the group's dS step waits for it
      //   pt_ready(it) -> dV(it), whose completion the group observes before ds_ready
      //   x_free(it)   -> S(it+2) into the same buffer (dP has been read out of it)
      //   ds_ready(it) -> dK(it); dQ(it)
      // Each stream runs in sub-tile order (the dQ drain relies on that order).
      auto pt_phase = [&](int it) -> bool {
        const uint32_t st = stage_of(it), g = it & 1;
        // dO of the stage arrives through the async proxy: this thread observes its barrier itself
        if (!mbar_wait_warp(&s.in_full[st], (it / kBwdStages) & 1, &s.abort_flag, p.status, 126, it)) return false;
        // dP^T as soon as the scores have been read out of the group's buffer: it forms while the group computes P
        if (!mbar_wait_warp(&s.s_read[g], (it >> 1) & 1, &s.abort_flag, p.status, 129, it)) return false;
        tc_fence_after();
        const uint64_t dd = d_do0 + st * kQ816, pt = d_pt0 + g * kPt16;
        if (leader) {
#pragma unroll
          for (int k = 0; k < D / 32; ++k) mma_f8_ss(tm + C::colX + g * QT, d_v8 + 2 * k, dd + 2 * k, id_dp, k > 0);
          mma_commit(&s.dp_full[g]);
        }
        __syncwarp();
        if (!mbar_wait_warp(&s.pt_ready[g], (it >> 1) & 1, &s.abort_flag, p.status, 122, it)) return false;
        tc_fence_after();
        if (leader) {
          const uint32_t acc = it > 0 ? 1u : 0u;
#pragma unroll
          for (int k = 0; k < QT / 32; ++k) mma_f8_ss(tm + C::colDV, pt + 2 * k, dd + kRow32D * k, id_dv, k > 0 ? 1u : acc);
          mma_commit(&s.dv_done[g]);
        }
        __syncwarp();
        return true;
      };
      auto ds_phase = [&](int it) -> bool {
        const uint32_t st = stage_of(it), g = it & 1;
        // the group's next scores as soon as dP^T of this sub-tile has been read out of the group's buffer: they
        // form while the group still computes dS
        if (it + 2 < n_it) {
          if (!mbar_wait_warp(&s.x_free[g], (it >> 1) & 1, &s.abort_flag, p.status, 128, it)) return false;
          tc_fence_after();
          fire_s(it + 2);
        }
        if (!mbar_wait_warp(&s.ds_ready[g], (it >> 1) & 1, &s.abort_flag, p.status, 123, it)) return false;
        tc_fence_after();
        const uint32_t acc = it > 0 ? 1u : 0u;
        const uint64_t q8 = d_q80 + st * kQ816, ds = d_ds0 + g * kPt16;
        if (leader) {
#pragma unroll
          for (int k = 0; k < QT / 32; ++k) mma_f8_ss(tm + C::colDK, ds + 2 * k, q8 + kRow32D * k, id_dk, k > 0 ? 1u : acc);
          mma_commit(&s.in_empty[st]);  // one of two arrivals: S and dK have read the stage
        }
        __syncwarp();
        if (it + 3 < n_it && !prep_s(it + 3)) return false;
        return true;
      };
      auto dq_phase = [&](int it) -> bool {
        const uint32_t st = stage_of(it), g = it & 1;
        if (!mbar_wait_warp(&s.ds_ready[g], (it >> 1) & 1, &s.abort_flag, p.status, 127, it)) return false;
        if (it > 0 && !mbar_wait_warp(&s.dq_free, (it - 1) & 1, &s.abort_flag, p.status, 124, it)) return false;
        tc_fence_after();
        const uint64_t ds = d_ds0 + g * kPt16;
        if (leader) {
#pragma unroll
          for (int k = 0; k < 4; ++k) {  // 128 keys, 32 per step
            if (D == 128) {  // dQ^T[d, q] = K8^T . dS8^T
              mma_f8_ss(tm + C::colDQ, d_k8 + kRow32D * k, ds + kRow32Q * k, id_dq, k > 0);
            } else {  // dQ[q, d] = dS8 . K8
              mma_f8_ss(tm + C::colDQ, ds + kRow32Q * k, d_k8 + kRow32D * k, id_dq, k > 0);
            }
          }
          mma_commit(&s.dq_full);
          mma_commit(&s.in_empty[st]);  // the other arrival: the last reader of the group's dS buffer
        }
        __syncwarp();
        return true;
      };
      if (stream == 0) {
        for (int it = 0; ok && it < n_it; ++it) ok = pt_phase(it);
      } else if (stream == 1) {
        for (int it = 0; ok && it < 3 && it < n_it; ++it) {
          ok = prep_s(it);
          if (ok && it < 2) fire_s(it);
        }
        for (int it = 0; ok && it < n_it; ++it) ok = ds_phase(it);
      } else {
        for (int it = 0; ok && it < n_it; ++it) ok = dq_phase(it);
      }
      if (ok && leader) mma_commit(&s.acc_done);
      // every tensor-core operation of this CTA has finished before TMEM is freed
      if (leader) mma_commit(&s.mma_drained);
      if (leader) mbar_wait_teardown(&s.mma_drained, 0);
      __syncwarp();
    }
  } else if (warp >= 16) {
    // ------------------------------------------------------------------ dQ drain (warps 16-19)
    // The partial dQ of a sub-tile leaves TMEM for registers and the accumulator is handed back to the
    // issuer at once; the reductions into the scratch accumulator then run beside the next sub-tile's MMAs.
    const int w4 = warp & 3;
    const uint32_t lane_base = tm + ((uint32_t)(w4 * 32) << 16);
    const int r = w4 * 32 + lane;  // TMEM lane: d (D = 128) or query row (D = 64)
    const bool bulk = D == 128 && p.dq_half;
    for (int it = 0; it < n_it; ++it) {
      if (!mbar_wait_warp(&s.dq_full, it & 1, &s.abort_flag, p.status, 130, it)) break;
      tc_fence_after();
      const int g = head_of(it), qs = sub0 + it - g * n_sub;
      const int bh = b * p.Hq + hk * G + g;
      float* base = p.dq_accum + ((size_t)bh * p.S + (size_t)qs * QT) * D;
      uint32_t v0[32], v1[32];
      tmem_ld32(lane_base + C::colDQ, v0);
      tmem_ld32(lane_base + C::colDQ + 32, v1);
      tmem_ld_wait(v0);
      tmem_ld_wait(v1);
      tc_fence_before();
      mbar_arrive_warp(&s.dq_free);  // the next dQ may overwrite the accumulator now
      if (D == 128 && p.dq_half) {
        // lane = d, registers i, i + 1 = two adjacent query rows -> one f16x2 word per row pair.  The accumulator keeps
        // a warp's 32 row pairs x 32 features of a sub-tile as 4 contiguous KB, so each warp stages them in shared memory
        // and sends them as ONE bulk reduction: the copy engine carries the traffic, and the load/store queue that every
        // warp of the SM shares sees 32 shared-memory stores per thread instead of 32 global reductions (which held it
        // up for the compute warps' accesses).  No warp waits for another.
        uint32_t* tile = s.dq_tile[it & 1][w4];
        // this warp's reduction of two sub-tiles ago has finished reading the buffer
        if (lane == 0) asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory");
        __syncwarp();
#pragma unroll
        for (int hh = 0; hh < 2; ++hh) {
          const uint32_t(&v)[32] = hh ? v1 : v0;
#pragma unroll
          for (int i = 0; i < 32; i += 2) {
            float lo, hi;  // one packed multiplication and one conversion per word
            unpack2(mul2(pack2u(v[i], v[i + 1]), pack2(kDqHalfScale, kDqHalfScale)), lo, hi);
            const __half2 h2 = __floats2half2_rn(lo, hi);
            tile[((32 * hh + i) >> 1) * 32 + lane] = *reinterpret_cast<const uint32_t*>(&h2);
          }
        }
        fence_async_smem();
        __syncwarp();
        if (lane == 0) {
          uint32_t* words = reinterpret_cast<uint32_t*>(p.dq_accum) + ((size_t)bh * p.S + (size_t)qs * QT) * (D / 2) + w4 * (32 * 32);
          asm volatile("cp.reduce.async.bulk.global.shared::cta.bulk_group.add.noftz.f16 [%0], [%1], %2;" ::"l"(words), "r"(smem_u32(tile)),
                       "r"(32 * 32 * 4)
                       : "memory");
          tma_store_commit();
        }
      } else if (D == 128) {
        // lane = d, register i = query row: one coalesced 128-byte reduction per row
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          atomicAdd(base + (size_t)i * D + r, __uint_as_float(v0[i]));
          if ((i & 7) == 7) drain_pause();
        }
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          atomicAdd(base + (size_t)(32 + i) * D + r, __uint_as_float(v1[i]));
          if ((i & 7) == 7) drain_pause();
        }
      } else if (p.dq_half) {
        // lane = query row, registers 2 j, 2 j + 1 = two adjacent features: the row's 32 f16 pairs pass through this
        // warp's shared-memory patch so that every reduction covers the 128 contiguous bytes of one row
        uint32_t* words = reinterpret_cast<uint32_t*>(p.dq_accum) + ((size_t)bh * p.S + (size_t)qs * QT + w4 * 32) * (D / 2) + lane;
        uint32_t* patch = reinterpret_cast<uint32_t*>(s.dq_patch[w4]);
        __syncwarp();
#pragma unroll
        for (int j = 0; j < 32; ++j) {
          const uint32_t(&v)[32] = j < 16 ? v0 : v1;
          const __half2 h2 = __floats2half2_rn(__uint_as_float(v[(2 * j) & 31]) * kDqHalfScale, __uint_as_float(v[(2 * j + 1) & 31]) * kDqHalfScale);
          patch[lane * 33 + j] = *reinterpret_cast<const uint32_t*>(&h2);
        }
        __syncwarp();
#pragma unroll
        for (int rr = 0; rr < 32; ++rr)
          asm volatile("red.global.add.noftz.f16x2 [%0], %1;" ::"l"(words + (size_t)rr * (D / 2)), "r"(patch[rr * 33 + lane]) : "memory");
      } else {
        // lane = query row, register i = feature: transpose 32 x 32 blocks through this warp's shared-memory patch
        // so that every reduction instruction covers 128 contiguous bytes of one row (vector reductions of 16 bytes
        // per lane, one row per lane, ran at half the rate of these in a stand-alone test)
        float* patch = s.dq_patch[w4];
#pragma unroll
        for (int hh = 0; hh < 2; ++hh) {
          const uint32_t(&v)[32] = hh ? v1 : v0;
          __syncwarp();
#pragma unroll
          for (int i = 0; i < 32; ++i) patch[lane * 33 + i] = __uint_as_float(v[i]);
          __syncwarp();
#pragma unroll
          for (int rr = 0; rr < 32; ++rr) atomicAdd(base + (size_t)(w4 * 32 + rr) * D + 32 * hh + lane, patch[rr * 33 + lane]);  // no pauses: at D = 64 the drain has no time to spare
        }
      }
    }
    // the bulk reductions of this CTA have completed before its shared memory is given up
    if (bulk && lane == 0) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
  } else {
    // ------------------------------------------------------------------ compute (warps 0-15)
    constexpr int CW = QT / 2;                   // query columns per thread
    const int grp = warp >> 3;                   // compute group: sub-tiles with it % 2 == grp
    const int half = (warp >> 2) & 1;
    const int row = (warp & 3) * 32 + lane;      // key row inside the tile = TMEM lane
    const uint32_t lane_base = tm + ((uint32_t)((warp & 3) * 32) << 16);
    const int key = kt * 128 + row;
    const float beta = p.scale / 16.0f;
    bool ok = true;
    // P8^T of sub-tile `it`: St -> 2^min(s2 + lstat, 8) -> E4M3 -> shared memory (A operand of dV);
    // the packed bytes also stay in registers for the dS step
    // this thread's row in the swizzled [key][q] tiles: byte offset of 16-byte chunk c is
    // row_base + (c ^ swz) (the swizzle XORs address bits 4-6 with the row bits above bit 7)
    const uint32_t row_base = row * QT;
    const uint32_t swz = (QT == 128 ? (row & 7u) : ((row >> 1) & 3u)) << 4;
    auto do_p = [&](int it, uint32_t (&pk)[CW / 4]) -> bool {
      const int st = it % kBwdStages;
      const int g = head_of(it), qs = sub0 + it - g * n_sub;
      const uint64_t c2c2 = pack2(s.c2[g], s.c2[g]);
      const int q_first = qs * QT + half * CW;     // global query index of this thread's first column
      const bool diag = p.causal && qs * QT < kt * 128 + 128;  // sub-tile overlaps the key tile: mask needed
      // the row statistics arrive through the async proxy: observe their barrier before reading them
      if (!mbar_wait_warp(&s.in_full[st], (it / kBwdStages) & 1, &s.abort_flag, p.status, 143, it)) return false;
      // step of that sub-tile, was committed by the same thread after dV(it-2)
      if (!mbar_wait_warp(&s.st_full[grp], (it >> 1) & 1, &s.abort_flag, p.status, 140, it)) return false;
      tc_fence_after();
      const float* ls = &s.lstat[st][half * CW];
      uint8_t* dst_row = &s.pt[grp][row_base];
#pragma unroll
      for (int c0 = 0; c0 < CW; c0 += 32) {
        uint32_t v[32];
        tmem_ld32(lane_base + C::colX + grp * QT + half * CW + c0, v);
        tmem_ld_wait(v);
        if (c0 + 32 >= CW) {  // the last read of the scores: dP^T of this sub-tile may take the buffer
          tc_fence_before();
          mbar_arrive_warp(&s.s_read[grp]);
        }
        // LSE, and E4M3 rounds 2^8.0x back to 256.  The masked variant is a separate, warp-uniform
        // path so that the common one carries no compare/select per element.
        if (diag) {
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const float4 l4 = *reinterpret_cast<const float4*>(ls + c0 + 4 * i);
            float x0, x1, x2, x3;
            unpack2(fma2(pack2u(v[4 * i], v[4 * i + 1]), c2c2, pack2(l4.x, l4.y)), x0, x1);
            unpack2(fma2(pack2u(v[4 * i + 2], v[4 * i + 3]), c2c2, pack2(l4.z, l4.w)), x2, x3);
            const int q = q_first + c0 + 4 * i;  // keys after the query get no weight
            const float p0 = (key > q) ? 0.f : ex2_approx_b(x0), p1 = (key > q + 1) ? 0.f : ex2_approx_b(x1);
            const float p2 = (key > q + 2) ? 0.f : ex2_approx_b(x2), p3 = (key > q + 3) ? 0.f : ex2_approx_b(x3);
            pk[c0 / 4 + i] = cvt_e4m3x4(p0, p1, p2, p3);
          }
        } else {
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const float4 l4 = *reinterpret_cast<const float4*>(ls + c0 + 4 * i);
            float x0, x1, x2, x3;
            unpack2(fma2(pack2u(v[4 * i], v[4 * i + 1]), c2c2, pack2(l4.x, l4.y)), x0, x1);
            unpack2(fma2(pack2u(v[4 * i + 2], v[4 * i + 3]), c2c2, pack2(l4.z, l4.w)), x2, x3);
            pk[c0 / 4 + i] = cvt_e4m3x4(ex2_approx_b(x0), ex2_approx_b(x1), ex2_approx_b(x2), ex2_approx_b(x3));
          }
        }
#pragma unroll
        for (int i = 0; i < 2; ++i)
          *reinterpret_cast<uint4*>(dst_row + ((uint32_t)(half * CW + c0 + 16 * i) ^ swz)) =
              make_uint4(pk[c0 / 4 + 4 * i], pk[c0 / 4 + 4 * i + 1], pk[c0 / 4 + 4 * i + 2], pk[c0 / 4 + 4 * i + 3]);
      }
      fence_async_smem();
      tc_fence_before();
      mbar_arrive_warp(&s.pt_ready[grp]);
      return true;
    };
    // dS8^T of sub-tile `it`: (dP16 + dstat) * P8 * scale/16 -> E4M3 -> shared memory
    const uint64_t bb = pack2(beta, beta);
    auto do_ds = [&](int it, const uint32_t (&pk)[CW / 4]) -> bool {
      const int st = it % kBwdStages;
      // the release of their input stage is committed after them
      if (it >= 2 && !mbar_wait_warp(&s.in_empty[(it - 2) % kBwdStages], ((it - 2) / kBwdStages) & 1, &s.abort_flag, p.status, 144, it))
        return false;
      if (!mbar_wait_warp(&s.dp_full[grp], (it >> 1) & 1, &s.abort_flag, p.status, 141, it)) return false;
      tc_fence_after();
      const float* dsm = &s.dstat[st][half * CW];
      uint8_t* dst_row = &s.dst[grp][row_base];
#pragma unroll
      for (int c0 = 0; c0 < CW; c0 += 32) {
        uint32_t v[32];
        tmem_ld32(lane_base + C::colX + grp * QT + half * CW + c0, v);
        tmem_ld_wait(v);
        if (c0 + 32 >= CW) {  // the last read of the group's buffer for this sub-tile: S of the next one may take it
          tc_fence_before();
          mbar_arrive_warp(&s.x_free[grp]);
        }
        uint32_t dk4[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const uint32_t w = pk[c0 / 4 + i];
          const float2 p01 = e4m3x2_to_f32(w & 0xffffu), p23 = e4m3x2_to_f32(w >> 16);
          const float4 d4 = *reinterpret_cast<const float4*>(dsm + c0 + 4 * i);
          float d0, d1, d2, d3;
          unpack2(mul2(mul2(add2(pack2u(v[4 * i], v[4 * i + 1]), pack2(d4.x, d4.y)), pack2(p01.x, p01.y)), bb), d0, d1);
          unpack2(mul2(mul2(add2(pack2u(v[4 * i + 2], v[4 * i + 3]), pack2(d4.z, d4.w)), pack2(p23.x, p23.y)), bb), d2, d3);
          dk4[i] = cvt_e4m3x4(d0, d1, d2, d3);
        }
#pragma unroll
        for (int i = 0; i < 2; ++i)
          *reinterpret_cast<uint4*>(dst_row + ((uint32_t)(half * CW + c0 + 16 * i) ^ swz)) =
              make_uint4(dk4[4 * i], dk4[4 * i + 1], dk4[4 * i + 2], dk4[4 * i + 3]);
      }
      // dV of this sub-tile has read P^T and dO by now: ds_ready hands both buffers on
      if (!mbar_wait_warp(&s.dv_done[grp], (it >> 1) & 1, &s.abort_flag, p.status, 145, it)) return false;
      fence_async_smem();
      tc_fence_before();
      mbar_arrive_warp(&s.ds_ready[grp]);
      return true;
    };
    // this group's sub-tiles; the other group works on the ones in between
    uint32_t pk[CW / 4];
    for (int it = grp; ok && it < n_it; it += 2) {
      ok = do_p(it, pk);
      if (ok) ok = do_ds(it, pk);
    }
    // ------------------------------------------------------------------ dK, dV of this key tile
    if (ok) ok = mbar_wait_warp(&s.acc_done, 0, &s.abort_flag, p.status, 142);
    if (ok) {
      // each of the four warps of a TMEM lane quarter writes a quarter of the columns
      tc_fence_after();
      constexpr float inv = 1.0f / 1024.0f;
      constexpr int EW = D / 4;
      const int slice = grp * 2 + half;
      __nv_bfloat16* dkrow = p.dk + (int64_t)b * p.dk_sb + (int64_t)hk * p.dk_sh + (int64_t)key * p.dk_ss + EW * slice;
      __nv_bfloat16* dvrow = p.dv + (int64_t)b * p.dv_sb + (int64_t)hk * p.dv_sh + (int64_t)key * p.dv_ss + EW * slice;
      const size_t acc_at = ((size_t)bhk * p.S + key) * D + EW * slice;
#pragma unroll
      for (int which = 0; which < 2; ++which) {
        __nv_bfloat16* dst = which ? dvrow : dkrow;
        const uint32_t col = (which ? C::colDV : C::colDK) + EW * slice;
        uint32_t v[EW];
        if constexpr (EW == 32) {
          tmem_ld32(lane_base + col, v);
          tmem_ld_wait(v);
        } else {
          tmem_ld16(lane_base + col, v);
          tmem_ld_wait16(v);
        }
        if (item.parts > 1) {
          // one of several parts of this key tile: the FP32 sums are rounded by a second kernel
          float* acc = (which ? p.dv_accum : p.dk_accum) + acc_at;
#pragma unroll
          for (int i = 0; i < EW / 4; ++i)
            red_add_v4(acc + 4 * i, __uint_as_float(v[4 * i]), __uint_as_float(v[4 * i + 1]), __uint_as_float(v[4 * i + 2]),
                       __uint_as_float(v[4 * i + 3]));
          continue;
        }
        uint32_t w[EW / 2];
#pragma unroll
        for (int i = 0; i < EW / 2; ++i) {
          const __nv_bfloat162 h2 = __floats2bfloat162_rn(__uint_as_float(v[2 * i]) * inv, __uint_as_float(v[2 * i + 1]) * inv);
          w[i] = *reinterpret_cast<const uint32_t*>(&h2);
        }
#pragma unroll
        for (int i = 0; i < EW / 8; ++i)
          *reinterpret_cast<uint4*>(dst + 8 * i) = make_uint4(w[4 * i], w[4 * i + 1], w[4 * i + 2], w[4 * i + 3]);
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 20) tmem_dealloc(tm, 512);
}

// out = bf16(accumulator / 1024) through the caller's strides, for the first `rows_per_head` rows of every head;
// up to three accumulators (dQ, dK, dV) in one launch, each with its own range of CTAs
struct ConvertJob {
  const float* acc;
  __nv_bfloat16* out;
  int64_t sb, sh, ss;
  int64_t n_rows;  // heads * rows_per_head
  int H, rows_per_head;
  unsigned first_cta, n_cta;
  int half_pairs;  // the accumulator holds f16 pairs of adjacent rows (BwdParams::dq_half)
};
struct ConvertJobs {
  ConvertJob job[3];
  int n;
};
template <int D>
__global__ void __launch_bounds__(256) accum_convert_kernel(const ConvertJobs jobs, int S) {
  constexpr int kPerRow = D / 8;
  int which = 0;
  while (which + 1 < jobs.n && blockIdx.x >= jobs.job[which + 1].first_cta) ++which;
  const ConvertJob& jb = jobs.job[which];
  if (jb.half_pairs && D == 64) {
    // plain f16 rows: one thread converts eight features of one row
    const uint32_t* acc = reinterpret_cast<const uint32_t*>(jb.acc);
    constexpr float inv = 1.0f / (1024.0f * kDqHalfScale);
    for (int64_t c = (int64_t)(blockIdx.x - jb.first_cta) * 256 + threadIdx.x; c < jb.n_rows * kPerRow; c += (int64_t)jb.n_cta * 256) {
      const int64_t r = c / kPerRow;
      const int cb = (int)(c % kPerRow) * 8;
      const int bh = (int)(r / jb.rows_per_head), sidx = (int)(r % jb.rows_per_head);
      const uint4 a = *reinterpret_cast<const uint4*>(acc + (((int64_t)bh * S + sidx) * D + cb) / 2);
      const uint32_t w[4] = {a.x, a.y, a.z, a.w};
      uint32_t o[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w[i]));
        const __nv_bfloat162 h = __floats2bfloat162_rn(f.x * inv, f.y * inv);
        o[i] = *reinterpret_cast<const uint32_t*>(&h);
      }
      *reinterpret_cast<uint4*>(jb.out + (int64_t)(bh / jb.H) * jb.sb + (int64_t)(bh % jb.H) * jb.sh + (int64_t)sidx * jb.ss + cb) =
          make_uint4(o[0], o[1], o[2], o[3]);
    }
    return;
  }
  if (jb.half_pairs) {
    // one thread: eight features of a pair of rows -- eight words in, two 16-byte stores out
    const uint32_t* acc = reinterpret_cast<const uint32_t*>(jb.acc);
    const int pairs_per_head = jb.rows_per_head / 2;
    constexpr float inv = 1.0f / (1024.0f * kDqHalfScale);
    for (int64_t c = (int64_t)(blockIdx.x - jb.first_cta) * 256 + threadIdx.x; c < jb.n_rows / 2 * kPerRow; c += (int64_t)jb.n_cta * 256) {
      const int64_t pr = c / kPerRow;
      const int cb = (int)(c % kPerRow) * 8;
      const int bh = (int)(pr / pairs_per_head), pidx = (int)(pr % pairs_per_head);
      const uint32_t* src = acc + ((int64_t)bh * (S / 2) + pidx / 32 * 32) * D + (cb / 32) * 1024 + (pidx % 32) * 32 + cb % 32;
      const uint4 a = *reinterpret_cast<const uint4*>(src), bq = *reinterpret_cast<const uint4*>(src + 4);
      const uint32_t w[8] = {a.x, a.y, a.z, a.w, bq.x, bq.y, bq.z, bq.w};
      uint32_t even[4], odd[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float2 f0 = __half22float2(*reinterpret_cast<const __half2*>(&w[2 * i]));
        const float2 f1 = __half22float2(*reinterpret_cast<const __half2*>(&w[2 * i + 1]));
        const __nv_bfloat162 e = __floats2bfloat162_rn(f0.x * inv, f1.x * inv), o = __floats2bfloat162_rn(f0.y * inv, f1.y * inv);
        even[i] = *reinterpret_cast<const uint32_t*>(&e);
        odd[i] = *reinterpret_cast<const uint32_t*>(&o);
      }
      __nv_bfloat16* dst = jb.out + (int64_t)(bh / jb.H) * jb.sb + (int64_t)(bh % jb.H) * jb.sh + (int64_t)(2 * pidx) * jb.ss + cb;
      *reinterpret_cast<uint4*>(dst) = make_uint4(even[0], even[1], even[2], even[3]);
      *reinterpret_cast<uint4*>(dst + jb.ss) = make_uint4(odd[0], odd[1], odd[2], odd[3]);
    }
    return;
  }
  for (int64_t c = (int64_t)(blockIdx.x - jb.first_cta) * 256 + threadIdx.x; c < jb.n_rows * kPerRow; c += (int64_t)jb.n_cta * 256) {
    const int64_t r = c / kPerRow;
    const int cb = (int)(c % kPerRow) * 8;
    const int bh = (int)(r / jb.rows_per_head), sidx = (int)(r % jb.rows_per_head);
    const float* src = jb.acc + ((int64_t)bh * S + sidx) * D + cb;
    const float4 a = *reinterpret_cast<const float4*>(src), bq = *reinterpret_cast<const float4*>(src + 4);
    constexpr float inv = 1.0f / 1024.0f;
    const __nv_bfloat162 h0 = __floats2bfloat162_rn(a.x * inv, a.y * inv), h1 = __floats2bfloat162_rn(a.z * inv, a.w * inv);
    const __nv_bfloat162 h2 = __floats2bfloat162_rn(bq.x * inv, bq.y * inv), h3 = __floats2bfloat162_rn(bq.z * inv, bq.w * inv);
    uint4 o;
    o.x = *reinterpret_cast<const uint32_t*>(&h0);
    o.y = *reinterpret_cast<const uint32_t*>(&h1);
    o.z = *reinterpret_cast<const uint32_t*>(&h2);
    o.w = *reinterpret_cast<const uint32_t*>(&h3);
    *reinterpret_cast<uint4*>(jb.out + (int64_t)(bh / jb.H) * jb.sb + (int64_t)(bh % jb.H) * jb.sh + (int64_t)sidx * jb.ss + cb) = o;
  }
}

template <int D>
static void add_convert_job(ConvertJobs& jobs, const float* acc, int H, int rows_per_head, int64_t n_heads, void* out, const fa4b_strides& st,
                            bool half_pairs = false) {
  const int64_t n_rows = n_heads * rows_per_head;
  if (n_rows == 0) return;
  ConvertJob& jb = jobs.job[jobs.n];
  jb = ConvertJob{acc, static_cast<__nv_bfloat16*>(out), st.batch, st.head, st.seq, n_rows, H, rows_per_head, 0, 0, half_pairs ? 1 : 0};
  jb.first_cta = jobs.n ? jobs.job[jobs.n - 1].first_cta + jobs.job[jobs.n - 1].n_cta : 0;
  jb.n_cta = (unsigned)std::min<int64_t>(((half_pairs && D == 128 ? n_rows / 2 : n_rows) * (D / 8) + 255) / 256, (int64_t)std::max(sm_count(), 1) * 16);
  ++jobs.n;
}

// dq_zeroed: the preprocess launch of this call has cleared the dQ accumulator
template <int D>
static int bwd_impl(const fa4b_attn_bwd_args& a, cudaStream_t st, bool dq_zeroed) {
  using C = BwdCfg<D>;
  const fa4b_attn_dims& d = a.dims;
  const fa4b_attn_ws_layout l = make_ws_layout(d);
  uint8_t* ws = static_cast<uint8_t*>(a.ws);
  uint8_t* tws = transient_base(a, l);  // dO5, row statistics, FP32 accumulators
  uint8_t* kvws = a.kv_ws ? static_cast<uint8_t*>(const_cast<void*>(a.kv_ws)) : ws;  // K and V operands may be another shard's
  const uint64_t S = d.S, nq = (uint64_t)d.B * d.Hq, nk = (uint64_t)d.B * d.Hkv;
  CUtensorMap m_kc, m_k8, m_v8, m_qc, m_q8, m_do;
  if (int s = make_tensor_map(&m_kc, kvws + l.k_codes, 1, D / 2, S, nk, D / 2, S * (D / 2), D / 2, 128)) return s;
  if (int s = make_tensor_map(&m_k8, kvws + l.k_fp8, 1, D, S, nk, D, S * D, D, 128)) return s;
  if (int s = make_tensor_map(&m_v8, kvws + l.v_fp8, 1, D, S, nk, D, S * D, D, 128)) return s;
  if (int s = make_tensor_map(&m_qc, ws + l.q_codes, 1, D / 2, S, nq, D / 2, S * (D / 2), D / 2, C::QT)) return s;
  if (int s = make_tensor_map(&m_q8, ws + l.q_fp8, 1, D, S, nq, D, S * D, D, C::QT)) return s;
  if (int s = make_tensor_map(&m_do, tws + l.do_fp8, 1, D, S, nq, D, S * D, D, C::QT)) return s;

  const int n_sm = sm_count();
  FA4B_REQUIRE(n_sm > 0, FA4B_CUDA_ERROR, "could not read the multiprocessor count of the current device");
  BwdParams p{};
  p.B = d.B; p.Hq = d.Hq; p.Hkv = d.Hkv; p.S = d.S;
  p.scale = resolve_scale(d);
  p.causal = d.mask == FA4B_MASK_CAUSAL;
  p.q_sf = ws + l.q_scales; p.k_sf = kvws + l.k_scales;
  p.q_global = reinterpret_cast<const float*>(ws + l.q_global);
  p.k_global = reinterpret_cast<const float*>(kvws + l.k_global);
  p.lstat = reinterpret_cast<const float*>(tws + l.lstat);
  p.dstat = reinterpret_cast<const float*>(tws + l.dstat);
  p.dq_accum = reinterpret_cast<float*>(tws + l.dq_accum);
  p.dk_accum = reinterpret_cast<float*>(tws + l.dkv_accum);
  p.dv_accum = p.dk_accum + nk * S * D;
  p.dk = static_cast<__nv_bfloat16*>(a.dk); p.dk_sb = a.dk_strides.batch; p.dk_sh = a.dk_strides.head; p.dk_ss = a.dk_strides.seq;
  p.dv = static_cast<__nv_bfloat16*>(a.dv); p.dv_sb = a.dv_strides.batch; p.dv_sh = a.dv_strides.head; p.dv_ss = a.dv_strides.seq;
  p.status = reinterpret_cast<uint32_t*>(ws + l.status);
  const int n_tiles = d.S / 128;
  p.chunk = bwd_chunk(d, n_sm);
  p.items_per_head = bwd_items_per_head(n_tiles, p.chunk, p.causal != 0);
  // f16 dQ sums: only where one call forms the whole sum (a sum kept across calls stays FP32), at D = 128
  p.dq_half = bwd_dq_half(d, a.flags) ? 1 : 0;
  p.head_group = bwd_head_group(d);
  // rows of every kv head whose key tiles are cut into parts (the tiles that see more than `chunk` query tiles):
  // their dK and dV arrive as FP32 sums
  const int split_rows = n_tiles > p.chunk ? (p.causal ? (n_tiles - p.chunk) * 128 : d.S) : 0;
  FA4B_CUDA(cudaMemsetAsync(p.status, 0, 16, st));
  if (!(a.flags & FA4B_BWD_KEEP_DQ_ACCUM) && !dq_zeroed) FA4B_CUDA(cudaMemsetAsync(p.dq_accum, 0, nq * S * D * (p.dq_half ? 2 : 4), st));
  if (split_rows)
    FA4B_CUDA(cudaMemset2DAsync(p.dk_accum, S * D * sizeof(float), 0, (size_t)split_rows * D * sizeof(float), 2 * nk, st));
  const int smem = (int)sizeof(BwdSmem<D>) + 1024;
  static std::mutex mu;
  static bool configured[64] = {};
  int dev = 0;
  FA4B_CUDA(cudaGetDevice(&dev));
  {
    std::lock_guard<std::mutex> lock(mu);
    if (dev >= 64 || !configured[dev]) {
      FA4B_CUDA(cudaFuncSetAttribute(attn_bwd_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
      if (dev < 64) configured[dev] = true;
    }
  }
  const unsigned grid = (unsigned)(nk * (uint64_t)p.items_per_head);
  if (a.ev_before) FA4B_CUDA(cudaEventRecord(static_cast<cudaEvent_t>(a.ev_before), st));
  attn_bwd_kernel<D><<<grid, kBwdThreads, smem, st>>>(p, m_kc, m_k8, m_v8, m_qc, m_q8, m_do);
  FA4B_CUDA(cudaGetLastError());
  if (a.ev_after) FA4B_CUDA(cudaEventRecord(static_cast<cudaEvent_t>(a.ev_after), st));
  // one launch rounds what arrived as FP32 sums: dQ, and dK / dV of the key tiles that were cut
  ConvertJobs jobs{};
  if (!(a.flags & FA4B_BWD_SKIP_DQ_OUT)) add_convert_job<D>(jobs, p.dq_accum, d.Hq, d.S, (int64_t)nq, a.dq, a.dq_strides, p.dq_half != 0);
  if (split_rows) {
    add_convert_job<D>(jobs, p.dk_accum, d.Hkv, split_rows, (int64_t)nk, a.dk, a.dk_strides);
    add_convert_job<D>(jobs, p.dv_accum, d.Hkv, split_rows, (int64_t)nk, a.dv, a.dv_strides);
  }
  if (jobs.n) {
    const unsigned cgrid = jobs.job[jobs.n - 1].first_cta + jobs.job[jobs.n - 1].n_cta;
    accum_convert_kernel<D><<<cgrid, 256, 0, st>>>(jobs, d.S);
    FA4B_CUDA(cudaGetLastError());
  }
  return FA4B_OK;
}

static int check_out(const void* ptr, const fa4b_strides& s, const char* name) {
  FA4B_REQUIRE(ptr != nullptr, FA4B_BAD_ARG, "%s is NULL", name);
  FA4B_REQUIRE((reinterpret_cast<uintptr_t>(ptr) & 15) == 0 && s.batch % 8 == 0 && s.head % 8 == 0 && s.seq % 8 == 0, FA4B_BAD_ALIGN,
               "%s: base must be 16-byte aligned and strides multiples of 8 elements", name);
  return FA4B_OK;
}

int launch_attn_bwd(const fa4b_attn_bwd_args& a, cudaStream_t st) {
  if (int s = check_dims(a.dims)) return s;
  FA4B_REQUIRE(a.ws != nullptr && (reinterpret_cast<uintptr_t>(a.ws) & 1023) == 0, FA4B_BAD_ALIGN,
               "workspace must be non-NULL and 1024-byte aligned");
  FA4B_REQUIRE((reinterpret_cast<uintptr_t>(a.scratch) & 1023) == 0, FA4B_BAD_ALIGN, "scratch must be 1024-byte aligned");
  FA4B_REQUIRE(!a.kv_ws || (reinterpret_cast<uintptr_t>(a.kv_ws) & 1023) == 0, FA4B_BAD_ALIGN, "kv_ws must be 1024-byte aligned");
  FA4B_REQUIRE(a.dims.pv_format == FA4B_PV_FP8_E4M3, FA4B_UNSUPPORTED, "the MXFP4 P.V route is forward only (a diagnostic route in the reference as well)");
  if (!(a.flags & FA4B_BWD_SKIP_DQ_OUT))
    if (int s = check_out(a.dq, a.dq_strides, "dq")) return s;
  if (int s = check_out(a.dk, a.dk_strides, "dk")) return s;
  if (int s = check_out(a.dv, a.dv_strides, "dv")) return s;
  const bool zero_in_preprocess = !a.preprocessed && !(a.flags & FA4B_BWD_KEEP_DQ_ACCUM);
  if (!a.preprocessed) {
    if (int s = launch_attn_bwd_preprocess(a, st, zero_in_preprocess)) return s;
  }
  return a.dims.D == 128 ? bwd_impl<128>(a, st, zero_in_preprocess) : bwd_impl<64>(a, st, zero_in_preprocess);
}

void fill_bwd_info(fa4b_info* out) {
  out->bwd_threads = kBwdThreads;
  out->bwd_smem_bytes = (int)sizeof(BwdSmem<128>) + 1024;
  out->bwd_tmem_columns = 512;
}

}  // namespace fa4b

using namespace fa4b;

extern "C" int fa4b_attn_bwd_plan(const fa4b_attn_dims* d, int32_t n_sm, fa4b_bwd_plan* out) {
  FA4B_REQUIRE(d && out, FA4B_BAD_ARG, "NULL argument");
  if (int s = check_dims(*d)) return s;
  if (n_sm <= 0) n_sm = sm_count();
  FA4B_REQUIRE(n_sm > 0, FA4B_CUDA_ERROR, "could not read the multiprocessor count of the current device");
  const int n = d->S / 128;
  const bool causal = d->mask == FA4B_MASK_CAUSAL;
  out->chunk = bwd_chunk(*d, n_sm);
  out->items_per_head = bwd_items_per_head(n, out->chunk, causal);
  out->head_group = bwd_head_group(*d);
  out->grid = (int64_t)d->B * d->Hkv * out->items_per_head;
  out->split_rows = n > out->chunk ? (causal ? (n - out->chunk) * 128 : d->S) : 0;
  return FA4B_OK;
}

extern "C" int fa4b_attn_bwd_plan_item(const fa4b_attn_dims* d, int32_t n_sm, int64_t index, int32_t out[5]) {
  fa4b_bwd_plan plan;
  if (int s = fa4b_attn_bwd_plan(d, n_sm, &plan)) return s;
  FA4B_REQUIRE(out != nullptr && index >= 0 && index < plan.grid, FA4B_BAD_ARG, "item index outside the launch's %lld work items",
               (long long)plan.grid);
  const int64_t heads = (int64_t)d->B * d->Hkv;
  const int64_t per_group = (int64_t)plan.items_per_head * plan.head_group;
  const int64_t first_head = index / per_group * plan.head_group, in_group = index % per_group;
  const int64_t group_heads = std::min<int64_t>(plan.head_group, heads - first_head);
  const BwdItem it = bwd_item_of((int)(in_group / group_heads), d->S / 128, plan.chunk, d->mask == FA4B_MASK_CAUSAL);
  out[0] = (int32_t)(first_head + in_group % group_heads);
  out[1] = it.kt;
  out[2] = it.qt_lo;
  out[3] = it.qt_hi;
  out[4] = it.parts;
  return FA4B_OK;
}

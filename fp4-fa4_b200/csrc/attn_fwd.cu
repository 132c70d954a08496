// Causal GQA forward: S = Qnvfp4 . Knvfp4^T on tcgen05 block-scaled MMA, online
// softmax in the log2 domain with an integer running maximum, P as E4M3 in
// TMEM, O += P . V8 as a TS-form FP8 MMA.
//
// One CTA per (batch, query head, pair of adjacent 128-row query tiles), heaviest
// pairs first.  K/V arrive in 128-key stages and are consumed as 64-key blocks.
// Roles: warps 0-3 softmax of the first tile, warps 4-7 softmax of the second
// (one thread per query row, 64 key columns per block, no cross-thread
// exchange), warp 8 TMA producer, warps 9 and 10 MMA issuers of the first and
// the second tile.  The two tiles run the chain QK -> softmax -> PV
// independently, each with its own issuer, accumulators and scale-factor
// columns, so the softmax of one overlaps the tensor work and the other
// tile's softmax and neither waits behind the other's events.
//
// TMEM columns (512 allocated): S0 0, S1 64, O0 128, O1 256, P0 384, P1 400,
// Q scale factors 416 / 424, K scale factors 432 + 16 tile + 8 (stage parity).
#include <cstdlib>
#include <mutex>
#include <type_traits>

#include "attn.cuh"

namespace fa4b {

constexpr int kFwdThreads = 352;
constexpr int kStages = 4;
// forward probabilities: nominal lift 2^5, reference point allowed to lag by 3 binades (P <= 2^8)
constexpr float kLift = 5.0f, kHeadroom = 3.0f;
constexpr uint32_t kColS = 0, kColO = 128, kColP = 384, kColSfq = 416, kColSfk = 432;
constexpr uint32_t kColSfp = 464, kColSfv = 472;  // MXFP4 route: P scales (4 per tile), V scales (4 per stage parity, 8 per tile)

template <int D>
struct FwdSmem {
  alignas(1024) uint8_t q_codes[2][128 * D / 2];
  alignas(1024) uint8_t k_codes[kStages][128 * D / 2];
  alignas(1024) uint8_t v[kStages][128 * D];   // E4M3 [keys][D]; MXFP4 route: codes [D][64 bytes] in the first half
  alignas(1024) uint8_t p_mx[2][128 * 32];     // MXFP4 route: P codes of one 64-key block per tile, [row][32 bytes]
  // in-kernel Q quantisation: the tile's bf16 rows as boxes of [128 rows][128 bytes] (128-byte swizzle pattern), filled
  // by coalesced loads; at D = 128 a thread's E4M3 row then takes the place of the first half of its own bf16 row
  // (that box is the source of a TMA store), at D = 64 the E4M3 rows have a buffer of their own
  alignas(1024) uint8_t q_stage[2][128 * 2 * D];
  alignas(1024) uint8_t q8_stage[2][D == 128 ? 1024 : 128 * D];
  alignas(16) uint8_t q_sf[2][(D / 64) * 512];
  alignas(16) uint8_t k_sf[kStages][(D / 64) * 512];
  alignas(16) uint8_t v_sf[kStages][512];      // MXFP4 route: E8M0 page of the stage's V (row = feature)
  alignas(16) uint8_t p_sf[2][512];            // MXFP4 route: E8M0 page of the P block (row = query row)
  StepTable steps;                             // in-kernel Q quantisation: division table of this head's global scale
  alignas(8) uint64_t q_raw, q_full, kv_full[kStages], kv_empty[2][kStages], s_full[2], s_free[2], p_ready[2][2], o_done[2], mma_drained;
  uint32_t tmem_base;
  alignas(8) volatile uint32_t abort_flag;
  uint32_t pad_;
};

struct FwdParams {
  int B, Hq, Hkv, S;
  int causal;  // 0: every key is visible to every query (an off-diagonal block of a sequence-sharded run)
  const uint8_t* v_sf;  // MXFP4 route: V scale pages [B*Hkv, S/128, 512]
  float scale_log2;  // softmax_scale * log2(e)
  const uint8_t* q_sf;
  const uint8_t* k_sf;
  const float* q_global;
  const float* k_global;
  __nv_bfloat16* o;
  int64_t o_sb, o_sh, o_ss;
  float* lse;
  uint32_t* status;
  // Q quantised inside this kernel (non-NULL q_src): the bf16 queries through their strides, the per-head amax words
  // (or a unit global scale), and where the operands go for the backward (the workspace's Q sections)
  const __nv_bfloat16* q_src;
  int64_t q_sb, q_sh, q_ss;
  int* q_amax_bits;
  int unit_global;
  uint8_t* q_codes_out;
  uint8_t* q_sf_out;
  uint8_t* q_fp8_out;
  float* q_global_out;
  int q_tma;  // the bf16 query tiles arrive by TMA (map_qsrc) instead of through the softmax threads' loads
};


__device__ __forceinline__ float ex2_approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// 2^e of two adjacent key columns: the exponential unit for most pairs, the FMA-pipe polynomial for the pairs
// ex2_pair_on_fma names (`pair` is a compile-time constant wherever this is called)
__device__ __forceinline__ void ex2_pair(uint64_t e2, int pair, float& lo, float& hi) {
  if (ex2_pair_on_fma(pair)) {
    unpack2(ex2_poly2(e2), lo, hi);
  } else {
    float a, b;
    unpack2(e2, a, b);
    lo = ex2_approx(a);
    hi = ex2_approx(b);
  }
}

template <int D, bool MX>
__global__ void __launch_bounds__(kFwdThreads, 1)
attn_fwd_kernel(const FwdParams p, const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                const __grid_constant__ CUtensorMap map_v, const __grid_constant__ CUtensorMap map_q8,
                const __grid_constant__ CUtensorMap map_qsrc) {
  extern __shared__ uint8_t raw[];
  // aligned by offsetting the shared array itself, so that accesses stay shared-space loads and stores
  FwdSmem<D>& s = *reinterpret_cast<FwdSmem<D>*>(raw + ((1024u - (smem_u32(raw) & 1023u)) & 1023u));
  constexpr int kPages = D / 64;
  constexpr uint32_t kKvBytes = 128 * D / 2 + kPages * 512 + (MX ? D * 64 + 512 : 128 * D);
  const int t = threadIdx.x, warp = t >> 5, lane = t & 31;

  // work item: heaviest (last) query-tile pairs first; the query heads of a kv group stay adjacent
  const int n_tiles = p.S / 128;
  const int n_pairs = (n_tiles + 1) / 2;
  const int heads = p.B * p.Hq;
  const int pi = n_pairs - 1 - (int)(blockIdx.x / heads);
  const int bh = blockIdx.x % heads;
  const int b = bh / p.Hq, h = bh % p.Hq;
  const int bhk = b * p.Hkv + h / (p.Hq / p.Hkv);
  // 64-key blocks each tile attends to (tile T sees keys < 128 T + 128); the odd tile may not exist
  const int nb0 = p.causal ? 2 * (2 * pi) + 2 : 2 * n_tiles;
  const int nb1 = (2 * pi + 1 < n_tiles) ? (p.causal ? 2 * (2 * pi + 1) + 2 : 2 * n_tiles) : 0;
  const int nbmax = nb0 > nb1 ? nb0 : nb1;
  const int n_stages = (nbmax + 1) / 2;
  {
    // an earlier CTA of this launch gave up: leave at once, as one (the decision is CTA-uniform)
    __shared__ uint32_t skip;
    if (t == 0) skip = *reinterpret_cast<volatile uint32_t*>(p.status);
    __syncthreads();
    if (skip != 0u) return;
  }

  if (t == 0) {
    // Q operands: one transaction barrier for the producer's copies, or one arrival per softmax warp that quantises
    mbar_init(&s.q_full, p.q_src ? (nb1 ? 8 : 4) : 1);
    for (int i = 0; i < kStages; ++i) {
      mbar_init(&s.kv_full[i], 1);
      mbar_init(&s.kv_empty[0][i], 1);  // released by each tile's issuer separately
      mbar_init(&s.kv_empty[1][i], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&s.s_full[i], 1);
      mbar_init(&s.s_free[i], 4);   // one arrival per softmax warp
      mbar_init(&s.p_ready[i][0], 4);
      mbar_init(&s.p_ready[i][1], 4);
      mbar_init(&s.o_done[i], 1);
    }
    mbar_init(&s.mma_drained, nb1 ? 2 : 1);
    mbar_init(&s.q_raw, 1);
    s.abort_flag = 0;
    fence_barrier_init();
    if (p.q_src && p.q_tma) {
      // the bf16 query rows of this CTA's tiles start on their way at once, as boxes of 128 rows x 64 features in the
      // layout the quantisation reads (their latency runs under the rest of the set-up)
      const int nq = nb1 ? 2 : 1;
      mbar_expect_tx(&s.q_raw, nq * 128 * D * 2);
      for (int i = 0; i < nq; ++i)
#pragma unroll
        for (int bx = 0; bx < D / 64; ++bx)
          tma_load_4d(&s.q_stage[i][bx * (128 * 128)], &map_qsrc, bx * 64, (2 * pi + i) * 128, h, b, &s.q_raw);
    }
  }
  if (warp == 8) tmem_alloc(&s.tmem_base, 512);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tm = s.tmem_base;

  if (warp == 8) {
    // ---------------------------------------------------------------- producer
    if (lane == 0) {
      tma_prefetch_desc(&map_q);
      tma_prefetch_desc(&map_k);
      tma_prefetch_desc(&map_v);
      const int nq = nb1 ? 2 : 1;
      if (!p.q_src) {  // published beforehand: codes and scale pages come by copy
        mbar_expect_tx(&s.q_full, nq * (128 * D / 2 + kPages * 512));
        for (int i = 0; i < nq; ++i) {
          const int qt = 2 * pi + i;
          tma_load_3d(s.q_codes[i], &map_q, 0, qt * 128, bh, &s.q_full);
          bulk_load(s.q_sf[i], p.q_sf + ((size_t)bh * n_tiles + qt) * kPages * 512, kPages * 512, &s.q_full);
        }
      }
      int issued = 0;
      for (int j = 0; j < n_stages; ++j) {
        const int st = j % kStages;
        // both tiles' issuers have released the slot (every stage but the last is used by both tiles)
        if (j >= kStages && !mbar_wait(&s.kv_empty[0][st], ((j / kStages) - 1) & 1, &s.abort_flag, p.status, 10, j)) break;
        if (j >= kStages && nb1 && !mbar_wait(&s.kv_empty[1][st], ((j / kStages) - 1) & 1, &s.abort_flag, p.status, 11, j)) break;
        mbar_expect_tx(&s.kv_full[st], kKvBytes);
        tma_load_3d(s.k_codes[st], &map_k, 0, j * 128, bhk, &s.kv_full[st]);
        bulk_load(s.k_sf[st], p.k_sf + ((size_t)bhk * n_tiles + j) * kPages * 512, kPages * 512, &s.kv_full[st]);
        if (MX) {
          tma_load_3d(s.v[st], &map_v, j * 64, 0, bhk, &s.kv_full[st]);  // codes [D][128 keys / 2]
          bulk_load(s.v_sf[st], p.v_sf + ((size_t)bhk * n_tiles + j) * 512, 512, &s.kv_full[st]);
        } else {
          tma_load_3d(s.v[st], &map_v, 0, j * 128, bhk, &s.kv_full[st]);
        }
        issued = j + 1;
      }
      // no copy of this CTA may still be in flight when its shared memory is given up, and the
      // tensor core's arrivals on the stage barriers must have landed too (nobody else waits for
      // the last ones)
      mbar_wait_teardown(&s.q_full, 0);
      if (p.q_src && p.q_tma) mbar_wait_teardown(&s.q_raw, 0);
      for (int j = issued > kStages ? issued - kStages : 0; j < issued; ++j) {
        mbar_wait_teardown(&s.kv_full[j % kStages], (j / kStages) & 1);
        if (issued == n_stages && !s.abort_flag) {
          if (j < (nb0 + 1) / 2) mbar_wait_teardown(&s.kv_empty[0][j % kStages], (j / kStages) & 1);  // tile 0 may use one stage less
          if (nb1) mbar_wait_teardown(&s.kv_empty[1][j % kStages], (j / kStages) & 1);
        }
      }
    }
  } else if (warp >= 9) {
    // ---------------------------------------------------------------- MMA issuers (warp 9: tile 0, warp 10: tile 1)
    // The whole warp runs the loop so that control flow stays warp-uniform; one elected lane (always
    // the same) issues the tensor-core instructions and their commits.  Everything a tile's chain
    // writes (S, P, O, its scale-factor columns, its stage-release barriers) belongs to that tile's
    // issuer alone; the two issuers share only the read-only K/V stages.
    const int ti = warp - 9;
    const int nb = ti ? nb1 : nb0;
    if (nb > 0) {
      const bool leader = elect_one();
      constexpr uint32_t id_qk = idesc_fp4(128, 64, 0, 0, 0);
      constexpr uint32_t id_pv = idesc_f8(128, D, 0, 0, 0, 1);  // A = P (TMEM), B = V8 [keys, D] MN-major
      static_assert((kStages & (kStages - 1)) == 0, "stage index is taken with a mask");
      const uint32_t col_s = tm + kColS + 64 * ti, col_o = tm + kColO + 128 * ti, col_p = tm + kColP + 16 * ti;
      const uint32_t col_sfq = tm + kColSfq + 8 * ti, col_sfk = tm + kColSfk + 16 * ti;
      const uint32_t col_sfp = tm + kColSfp + 4 * ti, col_sfv = tm + kColSfv + 8 * ti;
      const uint32_t q_addr = smem_u32(s.q_codes[ti]);
      bool ok = mbar_wait_warp(&s.q_full, 0, &s.abort_flag, p.status, 20);
      if (ok) {
        tc_fence_after();
        if (leader) {
#pragma unroll
          for (int pg = 0; pg < kPages; ++pg) tmem_cp_page(col_sfq + 4 * pg, make_page_desc(smem_u32(s.q_sf[ti] + 512 * pg)));
          if (p.q_src && ti == 0) {
            // the quantised queries of both tiles leave for the workspace (the backward's operands) as bulk copies
            // from the buffers the softmax warps filled; this thread waits for their reads before it exits
            for (int i = 0; i < (nb1 ? 2 : 1); ++i) {
              const int qt = 2 * pi + i;
              tma_store_3d(&map_q, s.q_codes[i], 0, qt * 128, bh);
              tma_store_2d(&map_q8, D == 128 ? s.q_stage[i] : s.q8_stage[i], 0, bh * p.S + qt * 128);
              bulk_store(p.q_sf_out + ((size_t)bh * n_tiles + qt) * kPages * 512, s.q_sf[i], kPages * 512);
            }
            tma_store_commit();
          }
        }
        __syncwarp();
      }
      // Q.K^T of 64-key block jb; the block's stage has been waited for and its scale pages copied
      auto issue_qk = [&](int jb) {
        const int st = (jb >> 1) & (kStages - 1), hb = jb & 1, sp = (jb >> 1) & 1;
        if (leader) {
          const uint32_t k_addr = smem_u32(s.k_codes[st]) + hb * 64 * (D / 2);
#pragma unroll
          for (int k = 0; k < D / 64; ++k)
            mma_nvfp4_ss(col_s, make_tile_desc(q_addr + 32 * k, D / 2), make_tile_desc(k_addr + 32 * k, D / 2), id_qk, col_sfq + 4 * k,
                         col_sfk + 8 * sp + 4 * k + 2 * hb, k > 0);
          mma_commit(&s.s_full[ti]);
        }
        __syncwarp();
      };
      auto open_stage = [&](int jb) -> bool {  // first block of a stage: wait for the data, copy the K scale pages
        const int sj = jb >> 1, st = sj & (kStages - 1);
        if (!mbar_wait_warp(&s.kv_full[st], (sj / kStages) & 1, &s.abort_flag, p.status, 21, jb)) return false;
        tc_fence_after();
        if (leader) {
#pragma unroll
          for (int pg = 0; pg < kPages; ++pg) tmem_cp_page(col_sfk + 8 * (sj & 1) + 4 * pg, make_page_desc(smem_u32(s.k_sf[st] + 512 * pg)));
          if (MX) tmem_cp_page(col_sfv + 4 * (sj & 1), make_page_desc(smem_u32(s.v_sf[st])));
        }
        __syncwarp();
        return true;
      };
      auto issue_pv = [&](int j) {
        const int st = (j >> 1) & (kStages - 1), hb = j & 1;
        if (leader) {
          if (MX) {
            // one block-scaled MMA per 64-key block: A = P codes (shared memory), B = V codes [D][keys], both K-major;
            // the block's two 32-key scale groups are bytes 0-1 of the P page and bytes 2 hb, 2 hb + 1 of the stage's V page
            tmem_cp_page(col_sfp, make_page_desc(smem_u32(s.p_sf[ti])));
            mma_mxfp4_ss(col_o, make_tile_desc(smem_u32(s.p_mx[ti]), 32), make_tile_desc(smem_u32(s.v[st]) + 32 * hb, 64),
                         idesc_fp4(128, D, 1, 0, 2 * hb), col_sfp, col_sfv + 4 * ((j >> 1) & 1), j > 0 ? 1u : 0u);
          } else {
            const uint32_t v_addr = smem_u32(s.v[st]) + hb * 64 * D;
#pragma unroll
            for (int k = 0; k < 2; ++k) mma_f8_ts(col_o, col_p + 8 * k, make_tile_desc(v_addr + 32 * k * D, D), id_pv, (j > 0 || k > 0) ? 1u : 0u);
          }
          mma_commit(&s.o_done[ti]);
          // the stage's last block for this tile: its K and V are not read again
          if ((j & 1) == 1 || j == nb - 1) mma_commit(&s.kv_empty[ti][st]);
        }
        __syncwarp();
      };
      if (ok) ok = open_stage(0);
      if (ok) issue_qk(0);
      for (int j = 0; ok && j < nb; ++j) {
        const int jn = j + 1;
        if (jn < nb) {
          if ((jn & 1) == 0) {
            ok = open_stage(jn);
            if (!ok) break;
          }
          // next block's scores as soon as this block's have been read out of TMEM
          ok = mbar_wait_warp(&s.s_free[ti], j & 1, &s.abort_flag, p.status, 23, j);
          if (!ok) break;
          tc_fence_after();
          issue_qk(jn);
        }
        ok = mbar_wait_warp(&s.p_ready[ti][j & 1], (j >> 1) & 1, &s.abort_flag, p.status, 22, j);
        if (!ok) break;
        tc_fence_after();
        issue_pv(j);
      }
      // every tensor-core operation of this CTA has finished before TMEM is freed
      if (leader) mma_commit(&s.mma_drained);
      if (leader) mbar_wait_teardown(&s.mma_drained, 0);
      if (leader && p.q_src && ti == 0) tma_store_wait_read();  // the query copies have read their shared-memory sources
      __syncwarp();
    }
  } else {
    // ---------------------------------------------------------------- softmax (warps 0-3: tile 0, warps 4-7: tile 1)
    const int ti = warp >> 2;
    const int nb = ti ? nb1 : nb0;
    const int qt = 2 * pi + ti;                 // global query tile
    const int row = (warp & 3) * 32 + lane;     // query row inside the tile = TMEM lane
    const uint32_t lane_base = tm + ((uint32_t)((warp & 3) * 32) << 16);
    float q_g = 0.f;
    if (p.q_src) {
      // ---- NVFP4 quantisation of this CTA's query rows, one row per thread (the softmax warps have nothing else to do
      // until the first scores arrive): 16-element blocks along D, E4M3 block scale, FP32 global scale of the head;
      // codes and scale pages go to shared memory in the layout the producer's copies would have left (and, with
      // E4M3(4q), to the workspace for the backward).  The arithmetic is publish_heads_kernel's.
      const float amax = p.unit_global ? kNvfp4GlobalDiv : __int_as_float(p.q_amax_bits[bh]);
      q_g = amax / kNvfp4GlobalDiv;
      const float inv6g = 1.0f / (6.0f * q_g);
      const bool all_zero = !(amax > 0.f);
      fill_step_table(s.steps, q_g, t);
      asm volatile("bar.sync 1, 256;" ::: "memory");  // the eight softmax warps
      if (nb > 0) {
        constexpr int kChunks = D / 8;
        uint4 raw[kChunks];
        if (p.q_tma) {
          // the tile's rows were asked for by TMA when the CTA started
          mbar_wait_warp(&s.q_raw, 0, &s.abort_flag, p.status, 33);
        } else {
          // the tile's rows come in by coalesced loads of its 128 threads (a row is D / 8 chunks of 16 bytes) ...
          const __nv_bfloat16* tile_src = p.q_src + (int64_t)b * p.q_sb + (int64_t)h * p.q_sh + (int64_t)(qt * 128) * p.q_ss;
#pragma unroll
          for (int i = 0; i < kChunks; ++i) {
            const int chunk = row + i * 128;
            raw[i] = __ldg(reinterpret_cast<const uint4*>(tile_src + (int64_t)(chunk / kChunks) * p.q_ss) + chunk % kChunks);
          }
#pragma unroll
          for (int i = 0; i < kChunks; ++i) {
            const int chunk = row + i * 128, r = chunk / kChunks, c = chunk % kChunks;
            *reinterpret_cast<uint4*>(&s.q_stage[ti][(c >> 3) * (128 * 128) + swizzled_offset((uint32_t)r, (uint32_t)(c & 7) * 16u, 128)]) = raw[i];
          }
          asm volatile("bar.sync %0, 128;" ::"r"(2 + ti) : "memory");  // the four warps of this tile
        }
        // ... and each thread takes its own row back (conflict-free: the eight lanes of a quarter warp are eight rows)
#pragma unroll
        for (int c = 0; c < kChunks; ++c)
          raw[c] = *reinterpret_cast<const uint4*>(&s.q_stage[ti][(c >> 3) * (128 * 128) + swizzled_offset((uint32_t)row, (uint32_t)(c & 7) * 16u, 128)]);
        uint8_t* q8 = D == 128 ? s.q_stage[ti] : s.q8_stage[ti];
        uint32_t sw = 0;
#pragma unroll
        for (int kb2 = 0; kb2 < D / 32; ++kb2) {  // two 16-element blocks at a time: 16 bytes of codes
          uint32_t cw[4] = {0, 0, 0, 0};
#pragma unroll
          for (int hb = 0; hb < 2; ++hb) {
            const int kb = 2 * kb2 + hb;
            const uint4 lo = raw[2 * kb], hi = raw[2 * kb + 1];
            const uint32_t w[8] = {lo.x, lo.y, lo.z, lo.w, hi.x, hi.y, hi.z, hi.w};
            uint64_t xp[8];
            uint32_t m2 = 0;
#pragma unroll
            for (int k = 0; k < 8; ++k) {
              m2 = absmax_bf16x2(m2, w[k]);
              xp[k] = bf16x2_to_f32x2(w[k]);
            }
            const float bamax = fmaxf(bf16_bits_to_f32(m2 & 0xffffu), bf16_bits_to_f32(m2 >> 16));
            uint32_t sbyte = 0;
            if (!all_zero) {
              sbyte = nvfp4_scale_byte(bamax, q_g, inv6g);
              nvfp4_codes16(xp, bamax, s.steps, sbyte, cw[2 * hb], cw[2 * hb + 1]);
            }
            sw |= sbyte << (8 * (kb & 3));
            uint32_t o8[4];
            const uint64_t four = pack2(4.f, 4.f);
#pragma unroll
            for (int k = 0; k < 4; ++k) {
              float a0, a1, b0, b1;
              unpack2(mul2(xp[2 * k], four), a0, a1);
              unpack2(mul2(xp[2 * k + 1], four), b0, b1);
              o8[k] = cvt_e4m3x4(a0, a1, b0, b1);
            }
            *reinterpret_cast<uint4*>(&q8[swizzled_offset((uint32_t)row, (uint32_t)kb * 16u, D)]) = make_uint4(o8[0], o8[1], o8[2], o8[3]);
          }
          *reinterpret_cast<uint4*>(&s.q_codes[ti][swizzled_offset((uint32_t)row, (uint32_t)kb2 * 16u, D / 2)]) = make_uint4(cw[0], cw[1], cw[2], cw[3]);
          if ((kb2 & 1) == 1) {  // the four scale bytes of this row in one page are one aligned word
            *reinterpret_cast<uint32_t*>(&s.q_sf[ti][(kb2 >> 1) * 512 + page_offset((uint32_t)row, 0)]) = sw;
            sw = 0;
          }
        }
        if (pi == 0 && ti == 0 && row == 0) {  // once per head
          p.q_global_out[bh] = q_g;
          if (p.unit_global) p.q_amax_bits[bh] = __float_as_int(kNvfp4GlobalDiv);
        }
        fence_async_smem();  // the tensor core reads these bytes through the async proxy
        mbar_arrive_warp(&s.q_full);
      }
    } else {
      q_g = p.q_global[bh];
    }
    const float c2 = p.scale_log2 * q_g * p.k_global[bhk];
    float mhat = -INFINITY;
    uint64_t lsum2 = pack2(0.f, 0.f);  // running row sum, as two partial sums
    const uint64_t c2c2 = pack2(c2, c2);
    bool ok = nb > 0;
    for (int j = 0; ok && j < nb; ++j) {
      ok = mbar_wait_warp(&s.s_full[ti], j & 1, &s.abort_flag, p.status, 30, j);
      if (!ok) break;
      tc_fence_after();
      uint32_t x[64];  // raw scores (FP32 bit patterns) of this row against the block's 64 keys
      {
        uint32_t(&r0)[32] = *reinterpret_cast<uint32_t(*)[32]>(&x[0]);
        uint32_t(&r1)[32] = *reinterpret_cast<uint32_t(*)[32]>(&x[32]);
        tmem_ld32(lane_base + kColS + 64 * ti, r0);
        tmem_ld32(lane_base + kColS + 64 * ti + 32, r1);
        tmem_ld_wait(r0);
        tmem_ld_wait(r1);
      }
      tc_fence_before();
      mbar_arrive_warp(&s.s_free[ti]);  // the next block's Q.K^T may overwrite S now
      const int lim = qt * 128 + row - 64 * j;  // columns <= lim are visible
      const bool diag = p.causal && j >= 2 * qt;  // warp-uniform
      // c2 >= 0: the maximum of the scaled scores is the scaled maximum of the raw ones
      float m0 = -INFINITY, m1 = -INFINITY, m2 = -INFINITY, m3 = -INFINITY;
      if (diag) {
#pragma unroll
        for (int i = 0; i < 64; i += 4) {
          m0 = fmaxf(m0, (i > lim) ? -INFINITY : __uint_as_float(x[i]));
          m1 = fmaxf(m1, (i + 1 > lim) ? -INFINITY : __uint_as_float(x[i + 1]));
          m2 = fmaxf(m2, (i + 2 > lim) ? -INFINITY : __uint_as_float(x[i + 2]));
          m3 = fmaxf(m3, (i + 3 > lim) ? -INFINITY : __uint_as_float(x[i + 3]));
        }
      } else {
#pragma unroll
        for (int i = 0; i < 64; i += 8) {  // three-input maximum: 32 instructions for 64 values
          m0 = max3(m0, __uint_as_float(x[i]), __uint_as_float(x[i + 1]));
          m1 = max3(m1, __uint_as_float(x[i + 2]), __uint_as_float(x[i + 3]));
          m2 = max3(m2, __uint_as_float(x[i + 4]), __uint_as_float(x[i + 5]));
          m3 = max3(m3, __uint_as_float(x[i + 6]), __uint_as_float(x[i + 7]));
        }
      }
      float mx = fmaxf(fmaxf(m0, m1), fmaxf(m2, m3));
      mx = (mx == -INFINITY) ? mx : mx * c2;  // a row can be fully masked in the tile's last block
      // Lazy reference point: probabilities are formed as 2^(s2 - mhat + kLift) and mhat only moves
      // when the block maximum exceeds it by more than kHeadroom, so that P stays <= 2^(kLift +
      // kHeadroom) = 256 < 448.  mhat is an integer, so every such P is the probability of the final
      // reference point times a power of two and rounds to the same E4M3 neighbour.
      const float cm = ceilf(mx);
      const bool moved = cm > mhat + kHeadroom;
      const float mnew = moved ? cm : mhat;
      // the running sum moves to the new reference point now; the accumulator follows after the
      // exponentials, once the previous block's P.V has finished
      const float f = moved ? ex2_approx(mhat - mnew) : 1.0f;
      if (__any_sync(0xffffffffu, moved)) lsum2 = mul2(lsum2, pack2(f, f));
      mhat = mnew;
      // P = 2^(x c2 - mhat + kLift): packed FMA for the exponent, the exponential unit or (6 of 16 columns) the FMA-pipe
      // polynomial for the power, packed add for the sum
      const uint64_t shift2 = pack2(kLift - mhat, kLift - mhat);
      if constexpr (!MX) {
        // The store of the previous block's P was left in flight so that its latency runs under the maximum pass
        // above: it has landed now, and that block's P.V may be issued.
        if (j > 0) {
          tmem_st_wait();
          tc_fence_before();
          mbar_arrive_warp(&s.p_ready[ti][(j - 1) & 1]);
        }
      }
      uint32_t pa[8], pb[8];  // FP8 route: P as E4M3 words; MXFP4 route: pa = the block's 64 E2M1 codes
      float pf[MX ? 64 : 1];  // MXFP4 route: the un-quantised probabilities, quantised per 32 keys below
      if (diag) {
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          float p0, p1, p2, p3;
          ex2_pair(fma2(pack2u(x[4 * i], x[4 * i + 1]), c2c2, shift2), 2 * i, p0, p1);
          ex2_pair(fma2(pack2u(x[4 * i + 2], x[4 * i + 3]), c2c2, shift2), 2 * i + 1, p2, p3);
          // keys after the query get no weight
          p0 = (4 * i > lim) ? 0.f : p0;
          p1 = (4 * i + 1 > lim) ? 0.f : p1;
          p2 = (4 * i + 2 > lim) ? 0.f : p2;
          p3 = (4 * i + 3 > lim) ? 0.f : p3;
          if constexpr (MX) {
            pf[4 * i] = p0; pf[4 * i + 1] = p1; pf[4 * i + 2] = p2; pf[4 * i + 3] = p3;
          } else {
            lsum2 = add2(lsum2, add2(pack2(p0, p1), pack2(p2, p3)));
            const uint32_t w = cvt_e4m3x4(p0, p1, p2, p3);
            if (i < 8) pa[i] = w; else pb[i - 8] = w;
          }
        }
      } else {
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          float p0, p1, p2, p3;
          ex2_pair(fma2(pack2u(x[4 * i], x[4 * i + 1]), c2c2, shift2), 2 * i, p0, p1);
          ex2_pair(fma2(pack2u(x[4 * i + 2], x[4 * i + 3]), c2c2, shift2), 2 * i + 1, p2, p3);
          if constexpr (MX) {
            pf[4 * i] = p0; pf[4 * i + 1] = p1; pf[4 * i + 2] = p2; pf[4 * i + 3] = p3;
          } else {
            lsum2 = add2(lsum2, add2(pack2(p0, p1), pack2(p2, p3)));
            const uint32_t w = cvt_e4m3x4(p0, p1, p2, p3);
            if (i < 8) pa[i] = w; else pb[i - 8] = w;
          }
        }
      }
      uint32_t p_scales = 0;  // MXFP4 route: the block's two E8M0 bytes
      if constexpr (MX) {
        // MXFP4 of P in 32-key groups: e = ceil(log2 max), step d = 2^e / 6 = RN(4/3) 2^(e-3) and its correctly rounded
        // reciprocal RN(1 / RN(4/3)) 2^(3-e) by exponent arithmetic, codes RN(p / d) -> E2M1; the row sum takes the
        // represented values (the codes decoded, times d), as the reference's MX route does
        constexpr uint32_t kD0 = 0x3FAAAAABu;  // RN(4/3)
        const uint32_t r0 = __float_as_uint(__frcp_rn(__uint_as_float(kD0)));
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          float b0 = 0.f, b1 = 0.f;
#pragma unroll
          for (int i = 0; i < 32; i += 4) {
            b0 = max3(b0, pf[32 * h + i], pf[32 * h + i + 1]);
            b1 = max3(b1, pf[32 * h + i + 2], pf[32 * h + i + 3]);
          }
          const float bmax = fmaxf(b0, b1);
          uint32_t cw[4] = {0, 0, 0, 0};
          if (bmax > 0.f) {
            const uint32_t bits = __float_as_uint(bmax);
            int e = (int)(bits >> 23) - 127 + ((bits & 0x7FFFFFu) != 0u ? 1 : 0);
            e = max(e, -100);  // below that every code is zero whatever the step
            p_scales |= (uint32_t)(e + 127) << (8 * h);
            const float step = __uint_as_float(kD0 + ((uint32_t)(e - 3) << 23)), r = __uint_as_float(r0 + ((uint32_t)(3 - e) << 23));
            const uint64_t r2 = pack2(r, r), nd2 = pack2(-step, -step);
            uint32_t hsum = 0;  // packed f16 pair: sums of the decoded low and high codes (exact: at most 16 x 6)
#pragma unroll
            for (int w = 0; w < 4; ++w) {
              uint32_t word = 0;
#pragma unroll
              for (int k = 0; k < 4; ++k) {
                float a, c;
                unpack2(div2_exact(pack2(pf[32 * h + 8 * w + 2 * k], pf[32 * h + 8 * w + 2 * k + 1]), r2, nd2), a, c);
                const uint32_t byte = cvt_e2m1x2(a, c);
                hsum = hadd2_bits(hsum, e2m1x2_to_f16x2(byte));
                word |= byte << (8 * k);
              }
              cw[w] = word;
            }
            const float2 hs = __half22float2(*reinterpret_cast<const __half2*>(&hsum));
            lsum2 = add2(lsum2, pack2((hs.x + hs.y) * step, 0.f));
          }
#pragma unroll
          for (int w = 0; w < 4; ++w) pa[4 * h + w] = cw[w];
        }
      }
      if (j > 0) {
        ok = mbar_wait_warp(&s.o_done[ti], (j - 1) & 1, &s.abort_flag, p.status, 31, j);
        if (!ok) break;
        tc_fence_after();
      }
      // tcgen05.ld/st are warp-collective: the accumulator rescale is taken by the whole warp
      // as soon as one of its rows has a new maximum (factor 1 for the rows that keep theirs)
      if (j > 0 && __any_sync(0xffffffffu, moved)) {
#pragma unroll
        for (int c0 = 0; c0 < D; c0 += 32) {
          uint32_t r[32];
          tmem_ld32(lane_base + kColO + 128 * ti + c0, r);
          tmem_ld_wait(r);
#pragma unroll
          for (int i = 0; i < 32; ++i) r[i] = __float_as_uint(__uint_as_float(r[i]) * f);
          tmem_st32(lane_base + kColO + 128 * ti + c0, r);
          tmem_st_wait();  // the store reads its registers asynchronously
        }
      }
      {
        if constexpr (MX) {
          // this row's 32 bytes of codes in the 32-byte-swizzled tile, its two scale bytes in the page
          *reinterpret_cast<uint4*>(&s.p_mx[ti][swizzled_offset(row, 0, 32)]) = make_uint4(pa[0], pa[1], pa[2], pa[3]);
          *reinterpret_cast<uint4*>(&s.p_mx[ti][swizzled_offset(row, 16, 32)]) = make_uint4(pa[4], pa[5], pa[6], pa[7]);
          *reinterpret_cast<uint16_t*>(&s.p_sf[ti][page_offset(row, 0)]) = (uint16_t)p_scales;
          fence_async_smem();
          tc_fence_before();
          mbar_arrive_warp(&s.p_ready[ti][j & 1]);
        } else {
          // completion is observed in the next iteration, or after the loop
          tmem_st8(lane_base + kColP + 16 * ti, pa);
          tmem_st8(lane_base + kColP + 16 * ti + 8, pb);
        }
      }
    }
    if constexpr (!MX) {
      if (ok) {
        tmem_st_wait();
        tc_fence_before();
        mbar_arrive_warp(&s.p_ready[ti][(nb - 1) & 1]);
      }
    }
    float lsum;
    {
      float lo, hi;
      unpack2(lsum2, lo, hi);
      lsum = lo + hi;
    }
    // ---------------------------------------------------------------- epilogue
    if (ok) ok = mbar_wait_warp(&s.o_done[ti], (nb - 1) & 1, &s.abort_flag, p.status, 32, nb);
    if (ok) {
      tc_fence_after();
      // FP8 route: V carries a factor 4.  MXFP4 route: the MMA multiplies code x 2^e on both sides while a value is
      // code x 2^e / 6, so the accumulator carries a factor 36 (the row sum above is of true values)
      const float inv = (MX ? 1.0f / 36.0f : 0.25f) / lsum;
      __nv_bfloat16* orow = p.o + (int64_t)b * p.o_sb + (int64_t)h * p.o_sh + (int64_t)(qt * 128 + row) * p.o_ss;
#pragma unroll
      for (int c0 = 0; c0 < D; c0 += 32) {
        uint32_t r[32];
        tmem_ld32(lane_base + kColO + 128 * ti + c0, r);
        tmem_ld_wait(r);
        uint32_t w[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          const __nv_bfloat162 v = __floats2bfloat162_rn(__uint_as_float(r[2 * i]) * inv, __uint_as_float(r[2 * i + 1]) * inv);
          w[i] = *reinterpret_cast<const uint32_t*>(&v);
        }
#pragma unroll
        for (int i = 0; i < 4; ++i)
          *reinterpret_cast<uint4*>(orow + c0 + 8 * i) = make_uint4(w[4 * i], w[4 * i + 1], w[4 * i + 2], w[4 * i + 3]);
      }
      p.lse[(size_t)bh * p.S + qt * 128 + row] = (mhat - kLift) * kLn2 + logf(lsum);
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 8) tmem_dealloc(tm, 512);
}

template <int D, bool MX>
static int fwd_impl(const fa4b_attn_fwd_args& a, cudaStream_t st) {
  const fa4b_attn_dims& d = a.dims;
  const fa4b_attn_ws_layout l = make_ws_layout(d);
  uint8_t* ws = static_cast<uint8_t*>(a.ws);
  // K and V operands may come from a second cache of the same layout (another sequence shard)
  uint8_t* kvws = a.kv_ws ? static_cast<uint8_t*>(const_cast<void*>(a.kv_ws)) : ws;
  CUtensorMap mq, mk, mv, mq8;
  const uint64_t S = d.S;
  if (int s = make_tensor_map(&mq, ws + l.q_codes, 1, D / 2, S, (uint64_t)d.B * d.Hq, D / 2, S * (D / 2), D / 2, 128)) return s;
  if (int s = make_tensor_map(&mk, kvws + l.k_codes, 1, D / 2, S, (uint64_t)d.B * d.Hkv, D / 2, S * (D / 2), D / 2, 128)) return s;
  if (MX) {  // codes [B*Hkv][D][S/2]: a stage is D rows x 64 bytes (128 keys)
    if (int s = make_tensor_map(&mv, kvws + l.v_fp8, 1, S / 2, D, (uint64_t)d.B * d.Hkv, S / 2, (uint64_t)D * (S / 2), 64, D)) return s;
  } else {
    if (int s = make_tensor_map(&mv, kvws + l.v_fp8, 1, D, S, (uint64_t)d.B * d.Hkv, D, S * D, D, 128)) return s;
  }
  // E4M3 queries [B*Hq*S][D]: the kernel's own quantisation writes them as boxes of 128 rows
  if (int s = make_tensor_map(&mq8, ws + l.q_fp8, 1, D, S * d.B * d.Hq, 0, D, 0, D, 128)) return s;
  CUtensorMap mqs = mq8;
  FwdParams p{};
  p.B = d.B; p.Hq = d.Hq; p.Hkv = d.Hkv; p.S = d.S;
  p.scale_log2 = resolve_scale(d) * kLog2e;
  p.causal = d.mask == FA4B_MASK_CAUSAL;
  p.q_sf = ws + l.q_scales; p.k_sf = kvws + l.k_scales;
  p.v_sf = kvws + l.v_fp8 + v_mx_pages_offset(d);
  p.q_global = reinterpret_cast<const float*>(ws + l.q_global);
  p.k_global = reinterpret_cast<const float*>(kvws + l.k_global);
  p.o = static_cast<__nv_bfloat16*>(a.o);
  p.o_sb = a.o_strides.batch; p.o_sh = a.o_strides.head; p.o_ss = a.o_strides.seq;
  p.lse = a.lse;
  p.status = reinterpret_cast<uint32_t*>(ws + l.status);
  if (!a.prepared) {  // launch_attn_fwd has published K and V and taken the amax words; Q is quantised by the kernel
    p.q_src = static_cast<const __nv_bfloat16*>(a.q);
    p.q_sb = a.q_strides.batch; p.q_sh = a.q_strides.head; p.q_ss = a.q_strides.seq;
    p.q_amax_bits = reinterpret_cast<int*>(ws + l.amax_bits);
    p.unit_global = d.global_scale_mode == FA4B_GLOBAL_ONE;
    p.q_codes_out = ws + l.q_codes; p.q_sf_out = ws + l.q_scales; p.q_fp8_out = ws + l.q_fp8;
    p.q_global_out = reinterpret_cast<float*>(ws + l.q_global);
    // bf16 queries [B][Hq][S][D] through the caller's strides; a view the tensor-map encoder refuses is loaded by threads
    p.q_tma = make_tensor_map_4d_bf16(&mqs, a.q, D, S, d.Hq, d.B, (uint64_t)a.q_strides.seq * 2, (uint64_t)a.q_strides.head * 2,
                                      (uint64_t)a.q_strides.batch * 2, 64, 128) == FA4B_OK
                  ? 1
                  : 0;
  }
  FA4B_CUDA(cudaMemsetAsync(p.status, 0, 64, st));
  const int smem = (int)sizeof(FwdSmem<D>) + 1024;
  static std::mutex mu;
  static bool configured[64] = {};  // per instantiation (D, MX)
  int dev = 0;
  FA4B_CUDA(cudaGetDevice(&dev));
  {
    std::lock_guard<std::mutex> lock(mu);
    if (dev < 64 && !configured[dev]) {
      FA4B_CUDA(cudaFuncSetAttribute(attn_fwd_kernel<D, MX>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
      configured[dev] = true;
    }
  }
  const unsigned grid = (unsigned)(d.B * d.Hq * ((d.S / 128 + 1) / 2));
  if (a.ev_before) FA4B_CUDA(cudaEventRecord(static_cast<cudaEvent_t>(a.ev_before), st));
  attn_fwd_kernel<D, MX><<<grid, kFwdThreads, smem, st>>>(p, mq, mk, mv, mq8, mqs);
  FA4B_CUDA(cudaGetLastError());
  if (a.ev_after) FA4B_CUDA(cudaEventRecord(static_cast<cudaEvent_t>(a.ev_after), st));
  return FA4B_OK;
}

int launch_attn_fwd(const fa4b_attn_fwd_args& a, cudaStream_t st) {
  if (int s = check_dims(a.dims)) return s;
  FA4B_REQUIRE(a.o && a.lse, FA4B_BAD_ARG, "o and lse are required");
  FA4B_REQUIRE(a.ws != nullptr && (reinterpret_cast<uintptr_t>(a.ws) & 1023) == 0, FA4B_BAD_ALIGN,
               "workspace must be non-NULL and 1024-byte aligned");
  FA4B_REQUIRE(!a.kv_ws || (a.prepared && (reinterpret_cast<uintptr_t>(a.kv_ws) & 1023) == 0), FA4B_BAD_ARG,
               "kv_ws needs prepared != 0 and 1024-byte alignment");
  FA4B_REQUIRE((reinterpret_cast<uintptr_t>(a.o) & 15) == 0 && a.o_strides.batch % 8 == 0 && a.o_strides.head % 8 == 0 &&
                   a.o_strides.seq % 8 == 0,
               FA4B_BAD_ALIGN, "o: base must be 16-byte aligned and strides multiples of 8 elements");
  if (!a.prepared) {
    // amax of Q and K (per-head recipe) and the publication of K and V; the forward kernel quantises Q itself
    fa4b_attn_prepare_args pa{a.dims, a.q, a.q_strides, a.k, a.k_strides, a.v, a.v_strides, a.ws};
    if (int s = launch_attn_prepare(pa, st, /*skip_q=*/true)) return s;
  }
  if (a.dims.pv_format == FA4B_PV_MXFP4_E8M0) return a.dims.D == 128 ? fwd_impl<128, true>(a, st) : fwd_impl<64, true>(a, st);
  return a.dims.D == 128 ? fwd_impl<128, false>(a, st) : fwd_impl<64, false>(a, st);
}

void fill_kernel_info(fa4b_info* out) {
  out->fwd_threads = kFwdThreads;
  out->fwd_smem_bytes = (int)sizeof(FwdSmem<128>) + 1024;
  out->fwd_tmem_columns = 512;
  out->fwd_kv_stages = kStages;
  fill_bwd_info(out);
}

}  // namespace fa4b

using namespace fa4b;

extern "C" int fa4b_attn_fwd(const fa4b_attn_fwd_args* a, void* stream) {
  FA4B_REQUIRE(a != nullptr, FA4B_BAD_ARG, "args is NULL");
  return launch_attn_fwd(*a, static_cast<cudaStream_t>(stream));
}


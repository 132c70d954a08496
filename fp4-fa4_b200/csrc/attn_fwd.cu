// Causal GQA forward: S = Qnvfp4 . Knvfp4^T on tcgen05 block-scaled MMA, online
// softmax in the log2 domain with an integer running maximum, P as E4M3 in
// TMEM, O += P . V8 as a TS-form FP8 MMA.
//
// One CTA per (batch, query head, 128-row query tile), heaviest tiles first.
// Roles: warps 0-7 softmax (two threads per query row: warps 0-3 take key
// columns 0-63 of a tile, warps 4-7 columns 64-127), warp 8 TMA producer,
// warp 9 MMA issuer.  The score accumulator is double buffered so that
// Q.K^T of tile j+1 runs under the softmax of tile j.
//
// TMEM columns (512 allocated): S[2] at 0 / 128, O at 256, P[2] at 384 / 416,
// Q scale factors at 448, K scale factors [2] at 456 / 464.
#include <mutex>

#include "attn.cuh"

namespace fa4b {

constexpr int kFwdThreads = 320;
constexpr int kStages = 4;
constexpr uint32_t kColS = 0, kColO = 256, kColP = 384, kColSfq = 448, kColSfk = 456;

template <int D>
struct FwdSmem {
  alignas(1024) uint8_t q_codes[128 * D / 2];
  alignas(1024) uint8_t k_codes[kStages][128 * D / 2];
  alignas(1024) uint8_t v[kStages][128 * D];
  alignas(16) uint8_t q_sf[(D / 64) * 512];
  alignas(16) uint8_t k_sf[kStages][(D / 64) * 512];
  alignas(16) float xchg[2][2][128];
  alignas(16) float lsum_x[2][128];
  alignas(8) uint64_t q_full, kv_full[kStages], kv_empty[kStages], s_full[2], p_ready[2], o_done;
  uint32_t tmem_base;
  volatile uint32_t abort_flag;
};

struct FwdParams {
  int B, Hq, Hkv, S;
  float scale_log2;  // softmax_scale * log2(e)
  const uint8_t* q_sf;
  const uint8_t* k_sf;
  const float* q_global;
  const float* k_global;
  __nv_bfloat16* o;
  int64_t o_sb, o_sh, o_ss;
  float* lse;
  uint32_t* status;
};

__device__ __forceinline__ float ex2_approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

__device__ __forceinline__ void named_bar_sync(int id, int threads) { asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory"); }

template <int D>
__global__ void __launch_bounds__(kFwdThreads, 1)
attn_fwd_kernel(const FwdParams p, const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                const __grid_constant__ CUtensorMap map_v) {
  extern __shared__ uint8_t raw[];
  FwdSmem<D>& s = *reinterpret_cast<FwdSmem<D>*>((reinterpret_cast<uintptr_t>(raw) + 1023) & ~uintptr_t(1023));
  constexpr int kPages = D / 64;
  constexpr uint32_t kKvBytes = 128 * D / 2 + kPages * 512 + 128 * D;
  const int t = threadIdx.x, warp = t >> 5, lane = t & 31;

  // work item: heaviest (last) query tiles first; the query heads of a kv group stay adjacent
  const int n_tiles = p.S / 128;
  const int heads = p.B * p.Hq;
  const int qt = n_tiles - 1 - (int)(blockIdx.x / heads);
  const int bh = blockIdx.x % heads;
  const int b = bh / p.Hq, h = bh % p.Hq;
  const int bhk = b * p.Hkv + h / (p.Hq / p.Hkv);
  const int n_kv = qt + 1;
  {
    // an earlier CTA of this launch gave up: leave at once, as one (the decision is CTA-uniform)
    __shared__ uint32_t skip;
    if (t == 0) skip = *reinterpret_cast<volatile uint32_t*>(p.status);
    __syncthreads();
    if (skip != 0u) return;
  }

  if (t == 0) {
    mbar_init(&s.q_full, 1);
    for (int i = 0; i < kStages; ++i) {
      mbar_init(&s.kv_full[i], 1);
      mbar_init(&s.kv_empty[i], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&s.s_full[i], 1);
      mbar_init(&s.p_ready[i], 256);
    }
    mbar_init(&s.o_done, 1);
    s.abort_flag = 0;
    fence_barrier_init();
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
      mbar_expect_tx(&s.q_full, 128 * D / 2 + kPages * 512);
      tma_load_3d(s.q_codes, &map_q, 0, qt * 128, bh, &s.q_full);
      bulk_load(s.q_sf, p.q_sf + ((size_t)bh * n_tiles + qt) * kPages * 512, kPages * 512, &s.q_full);
      for (int j = 0; j < n_kv; ++j) {
        const int st = j % kStages;
        if (j >= kStages && !mbar_wait(&s.kv_empty[st], ((j / kStages) - 1) & 1, &s.abort_flag, p.status, 10, j)) break;
        mbar_expect_tx(&s.kv_full[st], kKvBytes);
        tma_load_3d(s.k_codes[st], &map_k, 0, j * 128, bhk, &s.kv_full[st]);
        bulk_load(s.k_sf[st], p.k_sf + ((size_t)bhk * n_tiles + j) * kPages * 512, kPages * 512, &s.kv_full[st]);
        tma_load_3d(s.v[st], &map_v, 0, j * 128, bhk, &s.kv_full[st]);
      }
    }
  } else if (warp == 9) {
    // ---------------------------------------------------------------- MMA issuer
    if (lane == 0) {
      constexpr uint32_t id_qk = idesc_fp4(128, 128, 0, 0, 0);
      constexpr uint32_t id_pv = idesc_f8(128, D, 0, 0, 0, 1);  // A = P (TMEM), B = V8 [keys, D] MN-major
      bool ok = mbar_wait(&s.q_full, 0, &s.abort_flag, p.status, 20);
      if (ok) {
        tc_fence_after();
        for (int pg = 0; pg < kPages; ++pg) tmem_cp_page(tm + kColSfq + 4 * pg, make_page_desc(smem_u32(s.q_sf + 512 * pg)));
      }
      for (int j = 0; ok && j <= n_kv; ++j) {
        if (j < n_kv) {
          const int st = j % kStages, sb = j & 1;
          ok = mbar_wait(&s.kv_full[st], (j / kStages) & 1, &s.abort_flag, p.status, 21, j);
          if (!ok) break;
          tc_fence_after();
          for (int pg = 0; pg < kPages; ++pg)
            tmem_cp_page(tm + kColSfk + 8 * sb + 4 * pg, make_page_desc(smem_u32(s.k_sf[st] + 512 * pg)));
#pragma unroll
          for (int k = 0; k < D / 64; ++k)
            mma_nvfp4_ss(tm + kColS + 128 * sb, make_tile_desc(smem_u32(s.q_codes) + 32 * k, D / 2),
                         make_tile_desc(smem_u32(s.k_codes[st]) + 32 * k, D / 2), id_qk, tm + kColSfq + 4 * k,
                         tm + kColSfk + 8 * sb + 4 * k, k > 0);
          mma_commit(&s.s_full[sb]);
        }
        if (j > 0) {
          const int jj = j - 1, st = jj % kStages, sb = jj & 1;
          ok = mbar_wait(&s.p_ready[sb], (jj >> 1) & 1, &s.abort_flag, p.status, 22, j);
          if (!ok) break;
          tc_fence_after();
#pragma unroll
          for (int k = 0; k < 4; ++k)
            mma_f8_ts(tm + kColO, tm + kColP + 32 * sb + 8 * k, make_tile_desc(smem_u32(s.v[st]) + 32 * D * k, D), id_pv,
                      (jj > 0 || k > 0) ? 1u : 0u);
          mma_commit(&s.kv_empty[st]);
          mma_commit(&s.o_done);
        }
      }
    }
  } else {
    // ---------------------------------------------------------------- softmax (warps 0-7)
    const int half = warp >> 2;                 // which 64 key columns of a tile
    const int row = (warp & 3) * 32 + lane;     // query row inside the tile = TMEM lane
    const uint32_t lane_base = tm + ((uint32_t)((warp & 3) * 32) << 16);
    const float c2 = p.scale_log2 * p.q_global[bh] * p.k_global[bhk];
    float mhat = -INFINITY, lsum = 0.f;
    bool ok = true;
    // Every softmax thread runs every iteration and meets every named barrier, even after a
    // wait has given up (ok == false): a thread that left early would strand its partner.
    for (int j = 0; j < n_kv; ++j) {
      const int sb = j & 1;
      if (ok) ok = mbar_wait(&s.s_full[sb], (j >> 1) & 1, &s.abort_flag, p.status, 30, j);
      ok = __all_sync(0xffffffffu, ok);
      float x[64];
      float mx = -INFINITY;
      if (ok) {
        tc_fence_after();
        uint32_t r0[32], r1[32];
        tmem_ld32(lane_base + kColS + 128 * sb + 64 * half, r0);
        tmem_ld32(lane_base + kColS + 128 * sb + 64 * half + 32, r1);
        tmem_ld_wait(r0);
        tmem_ld_wait(r1);
        const bool diag = (j == qt);
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          x[i] = __uint_as_float(r0[i]) * c2;
          x[32 + i] = __uint_as_float(r1[i]) * c2;
        }
        if (diag) {
#pragma unroll
          for (int i = 0; i < 64; ++i)
            if (64 * half + i > row) x[i] = -INFINITY;
        }
#pragma unroll
        for (int i = 0; i < 64; ++i) mx = fmaxf(mx, x[i]);
      }
      s.xchg[sb][half][row] = mx;
      named_bar_sync(1, 256);
      mx = fmaxf(mx, s.xchg[sb][half ^ 1][row]);
      if (!ok) continue;
      const float mnew = fmaxf(mhat, ceilf(mx));
      // tcgen05.ld/st are warp-collective: the accumulator rescale is taken by the whole warp
      // as soon as one of its rows has a new maximum (factor 1 for the rows that keep theirs)
      if (j > 0 && __any_sync(0xffffffffu, mnew > mhat)) {
        const float f = ex2_approx(mhat - mnew);  // 2^0 = 1 when unchanged
        lsum *= f;
        ok = mbar_wait(&s.o_done, (j - 1) & 1, &s.abort_flag, p.status, 31, j);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) continue;
        tc_fence_after();
#pragma unroll
        for (int c0 = 0; c0 < D / 2; c0 += 32) {
          uint32_t r[32];
          tmem_ld32(lane_base + kColO + (D / 2) * half + c0, r);
          tmem_ld_wait(r);
#pragma unroll
          for (int i = 0; i < 32; ++i) r[i] = __float_as_uint(__uint_as_float(r[i]) * f);
          tmem_st32(lane_base + kColO + (D / 2) * half + c0, r);
        }
      }
      mhat = mnew;
      const float shift = kPLift - mhat;
      uint32_t pa[8], pb[8];
#pragma unroll
      for (int i = 0; i < 16; ++i) {
        const float p0 = ex2_approx(x[4 * i] + shift), p1 = ex2_approx(x[4 * i + 1] + shift);
        const float p2 = ex2_approx(x[4 * i + 2] + shift), p3 = ex2_approx(x[4 * i + 3] + shift);
        lsum += (p0 + p1) + (p2 + p3);
        const uint32_t w = cvt_e4m3x4(p0, p1, p2, p3);
        if (i < 8) pa[i] = w; else pb[i - 8] = w;
      }
      tmem_st8(lane_base + kColP + 32 * sb + 16 * half, pa);
      tmem_st8(lane_base + kColP + 32 * sb + 16 * half + 8, pb);
      tmem_st_wait();
      tc_fence_before();
      mbar_arrive(&s.p_ready[sb]);
    }
    // ---------------------------------------------------------------- epilogue
    if (ok) ok = mbar_wait(&s.o_done, (n_kv - 1) & 1, &s.abort_flag, p.status, 32, n_kv);
    ok = __all_sync(0xffffffffu, ok);
    s.lsum_x[half][row] = lsum;
    named_bar_sync(1, 256);
    if (ok) {
      tc_fence_after();
      const float l = lsum + s.lsum_x[half ^ 1][row];
      const float inv = 0.25f / l;
      __nv_bfloat16* orow = p.o + (int64_t)b * p.o_sb + (int64_t)h * p.o_sh + (int64_t)(qt * 128 + row) * p.o_ss + (D / 2) * half;
#pragma unroll
      for (int c0 = 0; c0 < D / 2; c0 += 32) {
        uint32_t r[32];
        tmem_ld32(lane_base + kColO + (D / 2) * half + c0, r);
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
      if (half == 0) p.lse[(size_t)bh * p.S + qt * 128 + row] = (mhat - kPLift) * kLn2 + logf(l);
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 8) tmem_dealloc(tm, 512);
}

template <int D>
static int fwd_impl(const fa4b_attn_fwd_args& a, cudaStream_t st) {
  const fa4b_attn_dims& d = a.dims;
  const fa4b_attn_ws_layout l = make_ws_layout(d);
  uint8_t* ws = static_cast<uint8_t*>(a.ws);
  CUtensorMap mq, mk, mv;
  const uint64_t S = d.S;
  if (int s = make_tensor_map(&mq, ws + l.q_codes, 1, D / 2, S, (uint64_t)d.B * d.Hq, D / 2, S * (D / 2), D / 2, 128)) return s;
  if (int s = make_tensor_map(&mk, ws + l.k_codes, 1, D / 2, S, (uint64_t)d.B * d.Hkv, D / 2, S * (D / 2), D / 2, 128)) return s;
  if (int s = make_tensor_map(&mv, ws + l.v_fp8, 1, D, S, (uint64_t)d.B * d.Hkv, D, S * D, D, 128)) return s;
  FwdParams p{};
  p.B = d.B; p.Hq = d.Hq; p.Hkv = d.Hkv; p.S = d.S;
  p.scale_log2 = resolve_scale(d) * kLog2e;
  p.q_sf = ws + l.q_scales; p.k_sf = ws + l.k_scales;
  p.q_global = reinterpret_cast<const float*>(ws + l.q_global);
  p.k_global = reinterpret_cast<const float*>(ws + l.k_global);
  p.o = static_cast<__nv_bfloat16*>(a.o);
  p.o_sb = a.o_strides.batch; p.o_sh = a.o_strides.head; p.o_ss = a.o_strides.seq;
  p.lse = a.lse;
  p.status = reinterpret_cast<uint32_t*>(ws + l.status);
  FA4B_CUDA(cudaMemsetAsync(p.status, 0, 16, st));
  const int smem = (int)sizeof(FwdSmem<D>) + 1024;
  static std::mutex mu;
  static bool configured[64] = {};
  int dev = 0;
  FA4B_CUDA(cudaGetDevice(&dev));
  {
    std::lock_guard<std::mutex> lock(mu);
    if (dev < 64 && !configured[dev]) {
      FA4B_CUDA(cudaFuncSetAttribute(attn_fwd_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
      configured[dev] = true;
    }
  }
  const unsigned grid = (unsigned)(d.B * d.Hq * (d.S / 128));
  if (a.ev_before) FA4B_CUDA(cudaEventRecord(static_cast<cudaEvent_t>(a.ev_before), st));
  attn_fwd_kernel<D><<<grid, kFwdThreads, smem, st>>>(p, mq, mk, mv);
  FA4B_CUDA(cudaGetLastError());
  if (a.ev_after) FA4B_CUDA(cudaEventRecord(static_cast<cudaEvent_t>(a.ev_after), st));
  return FA4B_OK;
}

int launch_attn_fwd(const fa4b_attn_fwd_args& a, cudaStream_t st) {
  if (int s = check_dims(a.dims)) return s;
  FA4B_REQUIRE(a.dims.pv_format == FA4B_PV_FP8_E4M3, FA4B_UNSUPPORTED, "the MXFP4 P.V route is not built yet");
  FA4B_REQUIRE(a.o && a.lse && a.ws, FA4B_BAD_ARG, "o, lse and ws are required");
  FA4B_REQUIRE((reinterpret_cast<uintptr_t>(a.o) & 15) == 0 && a.o_strides.batch % 8 == 0 && a.o_strides.head % 8 == 0 &&
                   a.o_strides.seq % 8 == 0,
               FA4B_BAD_ALIGN, "o: base must be 16-byte aligned and strides multiples of 8 elements");
  if (!a.prepared) {
    fa4b_attn_prepare_args pa{a.dims, a.q, a.q_strides, a.k, a.k_strides, a.v, a.v_strides, a.ws};
    if (int s = launch_attn_prepare(pa, st)) return s;
  }
  return a.dims.D == 128 ? fwd_impl<128>(a, st) : fwd_impl<64>(a, st);
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

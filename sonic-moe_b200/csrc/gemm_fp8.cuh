// FP8 (E4M3) grouped GEMM with fp32 block scales on CTA pairs: activations carry one scale per row and 128
// reduction elements (1 x 128), weights one scale per 128 x 128 block, scale = amax / 448.  The hardware's own
// block scaling (1 x 32, power-of-two scales) does not match these, so every 128-deep k-block is multiplied
// into a fresh accumulator in tensor memory (tcgen05.mma kind::f8f6f4, cta_group::2, M 256 x N 256 x K 32, four
// per k-block) and "promotion" warps add it, times  a_scale[row, kb] * b_scale[nblock, kb],  to fp32
// accumulators in registers while the tensor cores already work on the next k-block in the other half of
// tensor memory.  One pipeline stage = one k-block = 128 rows x 128 bytes per operand, so the staging,
// swizzle and descriptors are those of the bf16 kernel with 1-byte elements.
//
// Ragged-M only (forward and activation-gradient GEMMs); the weight-gradient GEMMs stay in bf16.
// Warps (16): 0 TMA producer · 1 MMA issuer (leader CTA) · 2,3 idle · 4..11 promotion + epilogue (two per
// TMEM lane quadrant, 128 columns each) · 12..15 row gather with TMA tile::gather4 (8 issuing threads per warp).
// Registers are moved from the light warps to the promotion warps with setmaxnreg.
#pragma once
#include "epilogue.cuh"
#include "ptx.cuh"

namespace smoe {
namespace fp8 {

constexpr int BM = 128;
constexpr int BN = 256;
constexpr int BN_CTA = 128;
constexpr int BK = 128;            // fp8 elements = bytes per row of a stage = one scale block
constexpr int STAGES = 6;
constexpr int UMMA_K = 32;
constexpr int A_STAGE_BYTES = BM * BK;      // 16 KiB
constexpr int B_STAGE_BYTES = BN_CTA * BK;  // 16 KiB
constexpr int MAX_EXPERTS = 1024;
constexpr int THREADS = 512;
constexpr int FIRST_PROMO_WARP = 4;
constexpr int FIRST_GATHER_WARP = 12;
constexpr int PROMO_WARPS = 8;

struct Scales {
  const float* a;        // (rows of the A source, K/128)
  long long a_ld;        // K / 128
  const float* b;        // per expert, per 128-row n-block, per k-block
  long long b_expert_stride, b_n_stride, b_k_stride;
};

struct SharedStorage {
  uint64_t full[STAGES];
  uint64_t empty[STAGES];
  uint64_t part_full[2];
  uint64_t part_empty[2];
  uint32_t tmem_base;
  int abort_flag;
  int m_tile_prefix[MAX_EXPERTS + 1];
};

constexpr int SMEM_BYTES = 1024 + STAGES * (A_STAGE_BYTES + B_STAGE_BYTES) + sizeof(SharedStorage);

struct Tile {
  int e, row0, row_end, n0, num_kb;
};

template <class Storage>
__device__ __forceinline__ bool decode_tile(const GemmParams& p, const Storage& ss, long long t, int num_n,
                                            uint32_t rank, Tile& tile) {
  const int total_m = ss.m_tile_prefix[p.E];
  if (t >= static_cast<long long>(total_m) * num_n) return false;
  const int mi = static_cast<int>(t / num_n);
  const int ni = static_cast<int>(t % num_n);
  int lo = 0, hi = p.E;
  while (hi - lo > 1) {
    const int mid = (lo + hi) >> 1;
    if (ss.m_tile_prefix[mid] <= mi) lo = mid; else hi = mid;
  }
  tile.e = lo;
  tile.row0 = p.off[lo] + (mi - ss.m_tile_prefix[lo]) * (2 * BM) + static_cast<int>(rank) * BM;
  tile.row_end = p.off[lo + 1];
  tile.n0 = ni * BN;
  tile.num_kb = p.K / BK;
  return true;
}

__host__ __device__ constexpr uint32_t make_idesc_e4m3(int M, int N, bool a_mn_major, bool b_mn_major) {
  return (1u << 4)                                    // D: f32
         | (0u << 7) | (0u << 10)                     // A, B: E4M3
         | (static_cast<uint32_t>(a_mn_major) << 15) | (static_cast<uint32_t>(b_mn_major) << 16)
         | (static_cast<uint32_t>(N >> 3) << 17) | (static_cast<uint32_t>(M >> 4) << 24);
}

__device__ __forceinline__ void umma_e4m3_pair(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                               uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t"
      "}\n"
      ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
      : "memory");
}

// Power-of-two scale: the smallest 2^e >= amax / 448, as the UE8M0 byte e + 127 and the exact factor 2^-e.
__device__ __forceinline__ uint8_t pow2_scale(float amax, float& inv_scale) {
  int e = 0;
  if (amax > 0.f) {
    const float m = frexpf(amax / 448.f, &e);  // amax / 448 = m 2^e, m in [0.5, 1)
    if (m == 0.5f) --e;
    e = max(e, -127);
  }
  inv_scale = __int_as_float((127 - e) << 23);  // e <= 121 for finite bf16 inputs
  return static_cast<uint8_t>(e + 127);
}

template <int N>
__device__ __forceinline__ void reg_dec() { asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(N)); }
template <int N>
__device__ __forceinline__ void reg_inc() { asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(N)); }

// A: K-major, gathered (TMA gather4) or plain.  B: K-major (forward) or MN-major (activation gradients).
template <bool A_GATHER, bool B_MN, int EPI>
__global__ void __launch_bounds__(THREADS, 1)
grouped_gemm_fp8_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                        const GemmParams p, const Scales sc) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sA = smem;
  uint8_t* sB = smem + STAGES * A_STAGE_BYTES;
  SharedStorage& ss = *reinterpret_cast<SharedStorage*>(smem + STAGES * (A_STAGE_BYTES + B_STAGE_BYTES));

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const bool leader = rank == 0;
  const long long first_tile = blockIdx.x >> 1;
  const long long tile_step = gridDim.x >> 1;
  volatile int* abort_flag = &ss.abort_flag;
  const int num_n = (p.N + BN - 1) / BN;
  constexpr uint32_t kTmaBytesPerCta = A_STAGE_BYTES + B_STAGE_BYTES;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(smem_u32(&ss.full[s]), 1);
      mbar_init(smem_u32(&ss.empty[s]), 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(smem_u32(&ss.part_full[a]), 1);
      mbar_init(smem_u32(&ss.part_empty[a]), 2 * PROMO_WARPS);
    }
    ss.abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == 0 && lane == 0) {
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(&ss.tmem_base), 2 * BN);
    tmem_relinquish();
  }
  if (warp == 2) {
    int running = 0;
    for (int base = 0; base < p.E; base += 32) {
      const int e = base + lane;
      int v = 0;
      if (e < p.E) v = (p.off[e + 1] - p.off[e] + 2 * BM - 1) / (2 * BM);
      int incl = v;
#pragma unroll
      for (int d = 1; d < 32; d <<= 1) {
        const int o = __shfl_up_sync(0xffffffffu, incl, d);
        if (lane >= d) incl += o;
      }
      if (e < p.E) ss.m_tile_prefix[e] = running + incl - v;
      running += __shfl_sync(0xffffffffu, incl, 31);
    }
    if (lane == 0) ss.m_tile_prefix[p.E] = running;
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();
  tc_fence_after();
  const uint32_t tmem_base = ss.tmem_base;

  if (warp < FIRST_PROMO_WARP) {
    reg_dec<56>();
    // ---- TMA producer ------------------------------------------------------------------------
    if (warp == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      Tile tile;
      for (long long t = first_tile; ok && decode_tile(p, ss, t, num_n, rank, tile); t += tile_step) {
        for (int kb = 0; kb < tile.num_kb; ++kb) {
          if (!mbar_wait(smem_u32(&ss.empty[stage]), phase ^ 1u, abort_flag)) { ok = false; break; }
          const uint32_t bar = map_to_cta(smem_u32(&ss.full[stage]), 0);
          if (leader && lane == 0) mbar_arrive_expect_tx(smem_u32(&ss.full[stage]), 2 * kTmaBytesPerCta);
          __syncwarp();
          if (lane == 0) {
            const int k0 = kb * BK;
            if constexpr (!A_GATHER) tma_load_2d_pair(&tmA, bar, smem_u32(sA + stage * A_STAGE_BYTES), k0, tile.row0);
            const int nb = tile.n0 + static_cast<int>(rank) * BN_CTA;
            const uint32_t b_dst = smem_u32(sB + stage * B_STAGE_BYTES);
            if constexpr (!B_MN) tma_load_2d_pair(&tmB, bar, b_dst, k0, tile.e * p.b_rows_per_expert + nb);
            else tma_load_2d_pair(&tmB, bar, b_dst, nb, tile.e * p.b_rows_per_expert + k0);
          }
          if (++stage == STAGES) { stage = 0; phase ^= 1u; }
        }
      }
      if (!ok && lane == 0 && p.status) atomicCAS(p.status, ST_OK, ST_TIMEOUT_PRODUCER);
    }
    // ---- MMA issuer ----------------------------------------------------------------------------
    else if (warp == 1 && leader) {
      constexpr uint32_t idesc = make_idesc_e4m3(2 * BM, BN, false, B_MN);
      constexpr uint32_t b_lbo = B_MN ? B_STAGE_BYTES : 16;
      constexpr uint32_t b_kstep = B_MN ? (UMMA_K * 128) : UMMA_K;  // bytes per 32 reduction elements
      int stage = 0;
      uint32_t phase = 0;
      int buf = 0;
      uint32_t buf_phase = 0;
      bool ok = true;
      Tile tile;
      for (long long t = first_tile; ok && decode_tile(p, ss, t, num_n, rank, tile); t += tile_step) {
        for (int kb = 0; kb < tile.num_kb; ++kb) {
          if (!mbar_wait(smem_u32(&ss.part_empty[buf]), buf_phase ^ 1u, abort_flag)) { ok = false; break; }
          if (!mbar_wait(smem_u32(&ss.full[stage]), phase, abort_flag)) { ok = false; break; }
          tc_fence_after();
          if (lane == 0) {
            const uint64_t a_desc = make_smem_desc(smem_u32(sA + stage * A_STAGE_BYTES), 16, 1024);
            const uint64_t b_desc = make_smem_desc(smem_u32(sB + stage * B_STAGE_BYTES), b_lbo, 1024);
            const uint32_t d_tmem = tmem_base + buf * BN;
#pragma unroll
            for (int k4 = 0; k4 < BK / UMMA_K; ++k4)
              umma_e4m3_pair(d_tmem, a_desc + ((k4 * UMMA_K) >> 4), b_desc + ((k4 * b_kstep) >> 4), idesc,
                             k4 > 0 ? 1u : 0u);
            umma_commit_pair(smem_u32(&ss.empty[stage]), 3);
            umma_commit_pair(smem_u32(&ss.part_full[buf]), 3);
          }
          __syncwarp();
          if (++stage == STAGES) { stage = 0; phase ^= 1u; }
          if (++buf == 2) { buf = 0; buf_phase ^= 1u; }
        }
      }
      if (!ok && lane == 0 && p.status) atomicCAS(p.status, ST_OK, ST_TIMEOUT_MMA);
    }
  } else if (warp >= FIRST_GATHER_WARP) {
    reg_dec<56>();
    // ---- row gather with TMA gather4: 8 issuing threads per warp, 4 rows x 128 B each ----------
    if constexpr (A_GATHER) {
      const int gt = threadIdx.x - 32 * FIRST_GATHER_WARP;  // 0..127
      const bool issuer = (gt & 3) == 0;
      const int j = gt >> 2;  // 0..31
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      Tile tile;
      for (long long t = first_tile; ok && decode_tile(p, ss, t, num_n, rank, tile); t += tile_step) {
        int r4[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int r = tile.row0 + 4 * j + i;
          r4[i] = (r < p.total_rows) ? p.gather[r] : 0;
        }
        for (int kb = 0; kb < tile.num_kb; ++kb) {
          if (!mbar_wait(smem_u32(&ss.empty[stage]), phase ^ 1u, abort_flag)) { ok = false; break; }
          if (issuer)
            tma_gather4_pair(&tmA, map_to_cta(smem_u32(&ss.full[stage]), 0),
                             smem_u32(sA + stage * A_STAGE_BYTES) + j * 512, kb * BK, r4[0], r4[1], r4[2], r4[3]);
          if (++stage == STAGES) { stage = 0; phase ^= 1u; }
        }
      }
      if (!ok && (gt & 31) == 0 && p.status) atomicCAS(p.status, ST_OK, ST_TIMEOUT_PRODUCER);
    }
  } else {
    reg_inc<200>();
    // ---- promotion + epilogue -----------------------------------------------------------------
    const int quad = warp & 3;
    const int col_half = (warp - FIRST_PROMO_WARP) >> 2;  // which 128 columns = which 128-row block of B
    const int row_in_tile = quad * 32 + lane;
    int buf = 0;
    uint32_t buf_phase = 0;
    bool ok = true;
    Tile tile;
    for (long long t = first_tile; ok && decode_tile(p, ss, t, num_n, rank, tile); t += tile_step) {
      const int r = tile.row0 + row_in_tile;
      const bool row_ok = r < tile.row_end;
      const int ncol0 = tile.n0 + col_half * 128;
      const bool cols_ok = ncol0 < p.N;
      const int src_row = (r < p.total_rows) ? (A_GATHER ? p.gather[r] : r) : 0;
      const float* a_sc = sc.a + static_cast<long long>(src_row) * sc.a_ld;
      const float* b_sc = sc.b + tile.e * sc.b_expert_stride + static_cast<long long>(cols_ok ? ncol0 / 128 : 0) * sc.b_n_stride;
      float acc[128];
#pragma unroll
      for (int i = 0; i < 128; ++i) acc[i] = 0.f;
      float scale_next = a_sc[0] * b_sc[0];
      for (int kb = 0; kb < tile.num_kb; ++kb) {
        const float scale = scale_next;
        if (kb + 1 < tile.num_kb) scale_next = a_sc[kb + 1] * b_sc[(kb + 1) * sc.b_k_stride];
        if (!mbar_wait(smem_u32(&ss.part_full[buf]), buf_phase, abort_flag)) { ok = false; break; }
        tc_fence_after();
        const uint32_t t_addr = tmem_base + buf * BN + col_half * 128 + (static_cast<uint32_t>(quad * 32) << 16);
        // two register buffers: the load of the next 32 columns is in flight while this one is accumulated
        uint32_t va[32], vb[32];
        tmem_ld32(t_addr, va);
        tmem_ld_wait();
        tmem_ld32(t_addr + 32, vb);
#pragma unroll
        for (int i = 0; i < 32; ++i) acc[i] = fmaf(__uint_as_float(va[i]), scale, acc[i]);
        tmem_ld_wait();
        tmem_ld32(t_addr + 64, va);
#pragma unroll
        for (int i = 0; i < 32; ++i) acc[32 + i] = fmaf(__uint_as_float(vb[i]), scale, acc[32 + i]);
        tmem_ld_wait();
        tmem_ld32(t_addr + 96, vb);
#pragma unroll
        for (int i = 0; i < 32; ++i) acc[64 + i] = fmaf(__uint_as_float(va[i]), scale, acc[64 + i]);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 32; ++i) acc[96 + i] = fmaf(__uint_as_float(vb[i]), scale, acc[96 + i]);
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive_cluster_relaxed(map_to_cta(smem_u32(&ss.part_empty[buf]), 0));
        if (++buf == 2) { buf = 0; buf_phase ^= 1u; }
      }
      if (!ok) break;
      float score = 0.f;
      if constexpr (EPI == EPI_DSWIGLU || EPI == EPI_SCATTER) {
        if (row_ok) score = load_score(p.scores, p.scores_are_bf16, p.s_scatter[r]);
      }
      float ds_acc = 0.f;
      if (row_ok && cols_ok) {
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          uint32_t v[32];
#pragma unroll
          for (int i = 0; i < 32; ++i) v[i] = __float_as_uint(acc[c * 32 + i]);
          epilogue_chunk<EPI, false>(p, tile.e, r, ncol0 + c * 32, v, score, ds_acc);
        }
      }
      if constexpr (EPI == EPI_DSWIGLU) {
        // every partial row the reduction reads is written, also the one past the last column block (zero)
        if (row_ok)
          p.ds_partial[static_cast<long long>(2 * (tile.n0 / BN) + col_half) * p.total_rows + r] = ds_acc;
      }
    }
    if (!ok && lane == 0 && p.status) atomicCAS(p.status, ST_OK, ST_TIMEOUT_EPILOGUE);
  }

  if (*abort_flag != 0) {
    const uint64_t t0 = global_timer_ns();
    while (global_timer_ns() - t0 < 200000ull) __nanosleep(1000);
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 2 * BN);
  }
}

}  // namespace fp8
}  // namespace smoe

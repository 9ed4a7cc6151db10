// Grouped (per-expert) GEMM for the MoE layer on sm_100a: TMA -> shared-memory ring -> tcgen05.mma with
// the accumulator in tensor memory -> epilogue warps.  One persistent CTA per SM, three roles:
//   warp 0      producer: TMA tiled loads into a 4-stage ring (and, in the TMA-gather variant,
//               tile::gather4 row gathers)
//   warp 1      MMA issuer: owns tensor memory (2 accumulators of 128 x 256 fp32 = all 512 columns)
//   warps 2..5  epilogue: tcgen05.ld the finished accumulator, apply the fused epilogue, store
//   warps 6..9  (kernels with a gathered operand, LSU-gather variant) row gather with 16-byte
//               cp.async copies written straight into the 128-byte-swizzled stage
//
// Two problem shapes share the kernel:
//   ragged-M  out[off[e] + m, n] = sum_k A[row(off[e] + m), k] * B_e[n, k]       (forward, dH, dX)
//   ragged-K  out_e[m, n]        = sum_{t in expert e} A[t, m] * B[t, n]          (weight gradients)
// Operands may be K-major (rows of the tile hold 128 B of the reduction dim) or MN-major (rows hold
// 128 B of the M/N dim, one row per reduction index); either may be a row gather through an index
// vector, so no permuted copy of the activations is ever written.
#pragma once
#include "epilogue.cuh"
#include "ptx.cuh"

namespace smoe {

constexpr int BM = 128;     // accumulator rows  (TMEM lanes)
constexpr int BN = 256;     // accumulator cols  (TMEM columns per accumulator)
constexpr int BK = 64;      // reduction elements per pipeline stage (128 B of bf16)
constexpr int STAGES = 4;
constexpr int UMMA_K = 16;  // reduction elements per tcgen05.mma (bf16)
constexpr int A_STAGE_BYTES = BM * BK * 2;  // 16 KiB
constexpr int B_STAGE_BYTES = BN * BK * 2;  // 32 KiB
constexpr int CHUNK_BYTES = BK * 128;       // one 64-element MN chunk of an MN-major tile: BK rows x 128 B
constexpr int MAX_EXPERTS = 1024;
// Warp roles: warp 0 TMA producer, warp 1 MMA issuer, then EW epilogue warps (4 or 8), then GW
// cp.async gather warps (0, 4 or 8).
__host__ __device__ constexpr int gemm_threads(int epi_warps, int gather_warps) {
  return 32 * (2 + epi_warps + gather_warps);
}

struct SharedStorage {
  uint64_t full[STAGES];
  uint64_t empty[STAGES];
  uint64_t acc_full[2];
  uint64_t acc_empty[2];
  uint32_t tmem_base;
  int abort_flag;
  int m_tile_prefix[MAX_EXPERTS + 1];
};

constexpr int GEMM_SMEM_BYTES = 1024 /*alignment slack*/ + STAGES * (A_STAGE_BYTES + B_STAGE_BYTES) + sizeof(SharedStorage);

struct Tile {
  int e;        // expert
  int row0;     // ragged-M: first grouped row of the tile; ragged-K: first output row (m offset)
  int row_end;  // ragged-M: off[e+1]; ragged-K: M
  int n0;       // first output column
  int k_begin;  // ragged-K: first grouped row of the expert
  int k_end;    // ragged-K: off[e+1]
  int num_kb;   // pipeline stages this tile consumes
};

template <bool RAGGED_K>
__device__ __forceinline__ bool decode_tile(const GemmParams& p, const SharedStorage& ss, long long t, int num_n,
                                            Tile& tile) {
  if constexpr (!RAGGED_K) {
    const int total_m = ss.m_tile_prefix[p.E];
    if (t >= static_cast<long long>(total_m) * num_n) return false;
    const int mi = static_cast<int>(t / num_n);
    const int ni = static_cast<int>(t % num_n);
    int lo = 0, hi = p.E;  // largest e with prefix[e] <= mi
    while (hi - lo > 1) {
      const int mid = (lo + hi) >> 1;
      if (ss.m_tile_prefix[mid] <= mi) lo = mid; else hi = mid;
    }
    tile.e = lo;
    tile.row0 = p.off[lo] + (mi - ss.m_tile_prefix[lo]) * BM;
    tile.row_end = p.off[lo + 1];
    tile.n0 = ni * BN;
    tile.k_begin = 0;
    tile.k_end = p.K;
    tile.num_kb = p.K / BK;
    return true;
  } else {
    const int num_m = (p.M + BM - 1) / BM;
    const long long per_e = static_cast<long long>(num_m) * num_n;
    if (t >= per_e * p.E) return false;
    const int e = static_cast<int>(t / per_e);
    const int rem = static_cast<int>(t % per_e);
    tile.e = e;
    tile.row0 = (rem / num_n) * BM;
    tile.row_end = p.M;
    tile.n0 = (rem % num_n) * BN;
    tile.k_begin = p.off[e];
    tile.k_end = p.off[e + 1];
    tile.num_kb = (tile.k_end - tile.k_begin + BK - 1) / BK;
    return true;
  }
}

template <bool RAGGED_K, bool A_GATHER, bool A_MN, bool B_GATHER, bool B_MN, int EPI, int EW, int GW>
__global__ void __launch_bounds__(gemm_threads(EW, GW), 1)
grouped_gemm_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                    const GemmParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sA = smem;
  uint8_t* sB = smem + STAGES * A_STAGE_BYTES;
  SharedStorage& ss = *reinterpret_cast<SharedStorage*>(smem + STAGES * (A_STAGE_BYTES + B_STAGE_BYTES));

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  volatile int* abort_flag = &ss.abort_flag;
  const int num_n = (p.N + BN - 1) / BN;
  constexpr bool LSU_GATHER = GW > 0;
  constexpr int GATHER_THREADS = 32 * GW;
  constexpr int FIRST_GATHER_WARP = 2 + EW;
  static_assert(EW == 4 || EW == 8, "4 or 8 epilogue warps");
  static_assert(GW == 0 || GW == 4 || GW == 8, "0, 4 or 8 gather warps");
  constexpr bool kLsuA = LSU_GATHER && A_GATHER;   // A rows arrive through cp.async, not TMA
  constexpr bool kLsuB = LSU_GATHER && B_GATHER;
  constexpr bool kLsu = kLsuA || kLsuB;
  static_assert(!(A_GATHER && B_GATHER), "at most one operand is gathered");
  constexpr uint32_t kTmaBytes = (kLsuA ? 0 : A_STAGE_BYTES) + (kLsuB ? 0 : B_STAGE_BYTES);

  // ---- set-up -------------------------------------------------------------------------------
  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(smem_u32(&ss.full[s]), 1 + (kLsu ? GATHER_THREADS : 0));
      mbar_init(smem_u32(&ss.empty[s]), 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(smem_u32(&ss.acc_full[a]), 1);
      mbar_init(smem_u32(&ss.acc_empty[a]), EW);  // one arrival per epilogue warp
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
  if constexpr (!RAGGED_K) {
    // Exclusive prefix of ceil(count / BM) over experts, by warp 2.
    if (warp == 2) {
      int running = 0;
      for (int base = 0; base < p.E; base += 32) {
        const int e = base + lane;
        int v = 0;
        if (e < p.E) v = (p.off[e + 1] - p.off[e] + BM - 1) / BM;
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
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = ss.tmem_base;

  // ---- producer -----------------------------------------------------------------------------
  if (warp == 0) {
    int stage = 0;
    uint32_t phase = 0;
    bool ok = true;
    Tile tile;
    for (long long t = blockIdx.x; ok && decode_tile<RAGGED_K>(p, ss, t, num_n, tile); t += gridDim.x) {
      // ragged-M gathered A: the four source rows this lane fetches are the same for every k-block
      int ar[4] = {0, 0, 0, 0};
      if constexpr (A_GATHER && !RAGGED_K && !kLsuA) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const int r = tile.row0 + 4 * lane + j;
          ar[j] = (r < p.total_rows) ? p.gather[r] : 0;
        }
      }
      for (int kb = 0; kb < tile.num_kb; ++kb) {
        if (!mbar_wait(smem_u32(&ss.empty[stage]), phase ^ 1u, abort_flag)) { ok = false; break; }
        const uint32_t bar = smem_u32(&ss.full[stage]);
        const uint32_t a_dst = smem_u32(sA + stage * A_STAGE_BYTES);
        const uint32_t b_dst = smem_u32(sB + stage * B_STAGE_BYTES);
        if (lane == 0) mbar_arrive_expect_tx(bar, kTmaBytes);
        __syncwarp();
        const int k0 = RAGGED_K ? (tile.k_begin + kb * BK) : kb * BK;  // ragged-K: first grouped row of the stage

        // ---- A ----
        if constexpr (kLsuA) {
          // gathered by warps 6..9
        } else if constexpr (!A_MN) {
          if constexpr (A_GATHER) {
            tma_gather4(&tmA, bar, a_dst + lane * 512, k0, ar[0], ar[1], ar[2], ar[3]);
          } else {
            if (lane == 0) tma_load_2d(&tmA, bar, a_dst, k0, tile.row0);
          }
        } else {
          // MN-major: 2 chunks of 64 m-elements, BK reduction rows each
          if constexpr (A_GATHER) {
            const int c = lane >> 4, tq = lane & 15;
            int r[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const int tok = k0 + 4 * tq + j;
              r[j] = (tok < tile.k_end) ? p.gather[tok] : p.gather_rows;
            }
            tma_gather4(&tmA, bar, a_dst + c * CHUNK_BYTES + tq * 512, tile.row0 + 64 * c, r[0], r[1], r[2], r[3]);
          } else {
            if (lane < BM / 64) tma_load_2d(&tmA, bar, a_dst + lane * CHUNK_BYTES, tile.row0 + 64 * lane, k0);
          }
        }
        // ---- B ----
        if constexpr (kLsuB) {
          // gathered by warps 6..9
        } else if constexpr (!B_MN) {
          static_assert(!B_GATHER || B_MN, "a gathered B is only used MN-major");
          if (lane == 0) tma_load_2d(&tmB, bar, b_dst, k0, tile.e * p.b_rows_per_expert + tile.n0);
        } else {
          if constexpr (B_GATHER) {
#pragma unroll
            for (int rep = 0; rep < (BN / 64) * 16 / 32; ++rep) {
              const int q = lane + 32 * rep;
              const int c = q >> 4, tq = q & 15;
              int r[4];
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                const int tok = k0 + 4 * tq + j;
                r[j] = (tok < tile.k_end) ? p.gather[tok] : p.gather_rows;
              }
              tma_gather4(&tmB, bar, b_dst + c * CHUNK_BYTES + tq * 512, tile.n0 + 64 * c, r[0], r[1], r[2], r[3]);
            }
          } else {
            const int krow = RAGGED_K ? k0 : (tile.e * p.b_rows_per_expert + k0);
            if (lane < BN / 64) tma_load_2d(&tmB, bar, b_dst + lane * CHUNK_BYTES, tile.n0 + 64 * lane, krow);
          }
        }
        if (++stage == STAGES) { stage = 0; phase ^= 1u; }
      }
    }
    if (!ok && lane == 0 && p.status) atomicCAS(p.status, ST_OK, ST_TIMEOUT_PRODUCER);
  }
  // ---- MMA issuer ---------------------------------------------------------------------------
  else if (warp == 1) {
    constexpr uint32_t idesc = make_idesc_bf16(BM, BN, A_MN, B_MN);
    constexpr uint32_t a_lbo = A_MN ? CHUNK_BYTES : 16;
    constexpr uint32_t b_lbo = B_MN ? CHUNK_BYTES : 16;
    constexpr uint32_t a_kstep = A_MN ? (UMMA_K * 128) : (UMMA_K * 2);  // bytes per UMMA_K step
    constexpr uint32_t b_kstep = B_MN ? (UMMA_K * 128) : (UMMA_K * 2);
    int stage = 0;
    uint32_t phase = 0;
    int acc = 0;
    uint32_t acc_phase = 0;
    bool ok = true;
    Tile tile;
    for (long long t = blockIdx.x; ok && decode_tile<RAGGED_K>(p, ss, t, num_n, tile); t += gridDim.x) {
      if (tile.num_kb == 0) continue;  // empty expert: the epilogue writes zeros without an accumulator
      if (!mbar_wait(smem_u32(&ss.acc_empty[acc]), acc_phase ^ 1u, abort_flag)) { ok = false; break; }
      tc_fence_after();
      const uint32_t d_tmem = tmem_base + acc * BN;
      for (int kb = 0; kb < tile.num_kb; ++kb) {
        if (!mbar_wait(smem_u32(&ss.full[stage]), phase, abort_flag)) { ok = false; break; }
        tc_fence_after();
        if (lane == 0) {
          if constexpr (kLsu) fence_proxy_async_smem();  // stage bytes written by cp.async -> async proxy reads
          const uint64_t a_desc = make_smem_desc(smem_u32(sA + stage * A_STAGE_BYTES), a_lbo, 1024);
          const uint64_t b_desc = make_smem_desc(smem_u32(sB + stage * B_STAGE_BYTES), b_lbo, 1024);
#pragma unroll
          for (int k4 = 0; k4 < BK / UMMA_K; ++k4) {
            umma_bf16(d_tmem, a_desc + ((k4 * a_kstep) >> 4), b_desc + ((k4 * b_kstep) >> 4), idesc,
                      (kb > 0 || k4 > 0) ? 1u : 0u);
          }
          umma_commit(smem_u32(&ss.empty[stage]));  // frees the stage once these MMAs have read it
        }
        __syncwarp();
        if (++stage == STAGES) { stage = 0; phase ^= 1u; }
      }
      if (!ok) break;
      if (lane == 0) umma_commit(smem_u32(&ss.acc_full[acc]));
      __syncwarp();
      if (++acc == 2) { acc = 0; acc_phase ^= 1u; }
    }
    if (!ok && lane == 0 && p.status) atomicCAS(p.status, ST_OK, ST_TIMEOUT_MMA);
  }
  // ---- LSU gather producers ------------------------------------------------------------------
  else if (warp >= FIRST_GATHER_WARP) {
    if constexpr (kLsu) {
      const int gt = threadIdx.x - 32 * FIRST_GATHER_WARP;  // 0..GATHER_THREADS-1
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      Tile tile;
      for (long long t = blockIdx.x; ok && decode_tile<RAGGED_K>(p, ss, t, num_n, tile); t += gridDim.x) {
        if constexpr (!RAGGED_K) {
          // K-major A tile: 128 rows x 128 B.  8 consecutive threads fetch the 8 16-byte pieces of a row;
          // thread handles rows rb, rb+16, ...; the swizzle term (row & 7) is the same for all of them.
          static_assert(kLsuA && !A_MN, "ragged-M kernels gather a K-major A");
          constexpr int RPP = GATHER_THREADS / 8;  // rows per pass: 16 or 32 (a multiple of 8)
          constexpr int NPASS = BM / RPP;          // 8 or 4
          const int c = gt & 7, rb = gt >> 3;
          const uint32_t dst_off = rb * 128 + ((c ^ (rb & 7)) << 4);
          const __nv_bfloat16* src[NPASS];
#pragma unroll
          for (int i = 0; i < NPASS; ++i) {
            const int r = tile.row0 + rb + RPP * i;
            const int idx = (r < p.total_rows) ? p.gather[r] : 0;
            src[i] = p.gather_src + static_cast<long long>(idx) * p.gather_ld + c * 8;
          }
          for (int kb = 0; kb < tile.num_kb; ++kb) {
            if (!mbar_wait(smem_u32(&ss.empty[stage]), phase ^ 1u, abort_flag)) { ok = false; break; }
            const uint32_t dst = smem_u32(sA + stage * A_STAGE_BYTES) + dst_off;
#pragma unroll
            for (int i = 0; i < NPASS; ++i) cp_async16(dst + i * (RPP * 128), src[i] + kb * BK, 16);
            cp_async_arrive_noinc(smem_u32(&ss.full[stage]));
            if (++stage == STAGES) { stage = 0; phase ^= 1u; }
          }
        } else {
          // MN-major tile: one reduction index (token) per 128-byte row, 64 tokens per chunk, one chunk
          // per 64 elements of M (A: 2 chunks) or N (B: 4 chunks).  A token's elements are contiguous in
          // global memory: CPR 16-byte pieces per token, fetched by CPR consecutive threads.
          constexpr int CPR = kLsuA ? (BM / 8) : (BN / 8);           // 16 or 32 pieces per token
          constexpr int ROWS_PER_PASS = GATHER_THREADS / CPR;          // 8 or 4 tokens per pass
          constexpr int PASSES = BK / ROWS_PER_PASS;                   // 8 or 16
          const int cc = gt % CPR, rb = gt / CPR;
          const int chunk = cc >> 3, c = cc & 7;
          const int col0 = (kLsuA ? tile.row0 : tile.n0) + cc * 8;
          const bool col_ok = col0 < (kLsuA ? p.M : p.N);
          const __nv_bfloat16* src_col = p.gather_src + col0;
          uint8_t* stage_base = kLsuA ? sA : sB;
          constexpr int STAGE_BYTES = kLsuA ? A_STAGE_BYTES : B_STAGE_BYTES;
          // Source rows of three stages are kept in registers, loaded two stages before they are needed, so the
          // latency of the index loads never sits between "stage is free" and "copies issued".
          int idx0[PASSES], idx1[PASSES], idx2[PASSES];
          auto load_idx = [&](int kb, int (&dst_idx)[PASSES]) {
            const int k0 = tile.k_begin + kb * BK;
#pragma unroll
            for (int i = 0; i < PASSES; ++i) {
              const int tok = k0 + rb + ROWS_PER_PASS * i;
              dst_idx[i] = (kb < tile.num_kb && tok < tile.k_end && col_ok) ? p.gather[tok] : -1;
            }
          };
          load_idx(0, idx0);
          load_idx(1, idx1);
          load_idx(2, idx2);
          for (int kb = 0; kb < tile.num_kb; ++kb) {
            if (!mbar_wait(smem_u32(&ss.empty[stage]), phase ^ 1u, abort_flag)) { ok = false; break; }
            const uint32_t dst = smem_u32(stage_base + stage * STAGE_BYTES) + chunk * CHUNK_BYTES;
#pragma unroll
            for (int i = 0; i < PASSES; ++i) {
              const int r = rb + ROWS_PER_PASS * i;
              const bool valid = idx0[i] >= 0;
              const __nv_bfloat16* src = src_col + static_cast<long long>(valid ? idx0[i] : 0) * p.gather_ld;
              cp_async16(dst + r * 128 + ((c ^ (r & 7)) << 4), src, valid ? 16u : 0u);
            }
            cp_async_arrive_noinc(smem_u32(&ss.full[stage]));
#pragma unroll
            for (int i = 0; i < PASSES; ++i) { idx0[i] = idx1[i]; idx1[i] = idx2[i]; }
            load_idx(kb + 3, idx2);
            if (++stage == STAGES) { stage = 0; phase ^= 1u; }
          }
        }
      }
      cp_async_wait_all();
      if (!ok && (gt & 31) == 0 && p.status) atomicCAS(p.status, ST_OK, ST_TIMEOUT_PRODUCER);
    }
  }
  // ---- epilogue -----------------------------------------------------------------------------
  else {
    const int quad = warp & 3;            // TMEM lanes [32*quad, 32*quad + 32) belong to this warp
    constexpr int COL_SPLIT = EW / 4;     // warps sharing a lane quadrant split the accumulator's columns
    constexpr int COLS_PER_WARP = BN / COL_SPLIT;
    const int col_half = (warp - 2) >> 2; // 0 .. COL_SPLIT-1
    const int row_in_tile = quad * 32 + lane;
    int acc = 0;
    uint32_t acc_phase = 0;
    bool ok = true;
    Tile tile;
    for (long long t = blockIdx.x; ok && decode_tile<RAGGED_K>(p, ss, t, num_n, tile); t += gridDim.x) {
      const int r = tile.row0 + row_in_tile;
      const bool row_ok = r < tile.row_end;
      const bool have_acc = tile.num_kb > 0;
      if (have_acc) {
        if (!mbar_wait(smem_u32(&ss.acc_full[acc]), acc_phase, abort_flag)) { ok = false; break; }
        tc_fence_after();
      }
      float score = 0.f;
      int slot = 0;
      if constexpr (EPI == EPI_DSWIGLU || EPI == EPI_SCATTER || EPI == EPI_STORE_ROWS) {
        if (row_ok && (EPI != EPI_STORE_ROWS || p.scores != nullptr)) {
          slot = p.s_scatter[r];
          score = load_score(p.scores, p.scores_are_bf16, slot);
        }
      }
      float ds_acc = 0.f;
      const uint32_t t_addr = tmem_base + acc * BN + (static_cast<uint32_t>(quad * 32) << 16);
#pragma unroll 1
      for (int c = col_half * (COLS_PER_WARP / 32); c < (col_half + 1) * (COLS_PER_WARP / 32); ++c) {
        const int n = tile.n0 + c * 32;
        if (n >= p.N) break;  // N is a multiple of 32: a chunk is entirely inside or entirely outside
        uint32_t v[32];
        if (have_acc) {
          tmem_ld32(t_addr + c * 32, v);
          tmem_ld_wait();
        } else {
#pragma unroll
          for (int j = 0; j < 32; ++j) v[j] = 0u;
        }
        if (!row_ok) continue;
        epilogue_chunk<EPI, RAGGED_K>(p, tile.e, r, n, v, score, ds_acc);
      }
      if constexpr (EPI == EPI_DSWIGLU) {
        // two partial rows per 256-column tile; with 4 epilogue warps one warp covers both halves
        if (row_ok) {
          float* dsp = p.ds_partial + static_cast<long long>(2 * (tile.n0 / BN)) * p.total_rows + r;
          if constexpr (COL_SPLIT == 2) {
            dsp[static_cast<long long>(col_half) * p.total_rows] = ds_acc;
          } else {
            dsp[0] = ds_acc;
            dsp[p.total_rows] = 0.f;
          }
        }
      }
      if (have_acc) {
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(smem_u32(&ss.acc_empty[acc]));
        if (++acc == 2) { acc = 0; acc_phase ^= 1u; }
      }
    }
    if (!ok && lane == 0 && p.status) atomicCAS(p.status, ST_OK, ST_TIMEOUT_EPILOGUE);
  }

  // ---- tear-down ----------------------------------------------------------------------------
  // After a timeout some copies may still be in flight; give them time to land before the CTA's
  // shared memory and tensor memory are released.
  if (*abort_flag != 0) {
    const uint64_t t0 = global_timer_ns();
    while (global_timer_ns() - t0 < 200000ull) __nanosleep(1000);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 2 * BN);
  }
}

}  // namespace smoe

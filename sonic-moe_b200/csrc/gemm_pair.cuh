// Grouped GEMM on CTA pairs: a cluster of two CTAs (one SM pair) computes a 256 x 256 output tile with
// tcgen05.mma.cta_group::2.  Each CTA stages its own 128 rows of A and its own 128 of the tile's 256 B rows,
// so a stage costs 32 KiB of shared-memory fill per CTA instead of 48 KiB and six stages fit; the
// accumulator (this CTA's 128 rows x all 256 columns, fp32) lives in the CTA's own tensor memory, two
// of them so the epilogue of one tile overlaps the main loop of the next.
//
// DUAL mode (kernels with a gathered operand): one work unit is two tiles that share the gathered operand's
// stage -- 256 x 512 (DUAL_N: two B tiles) or 512 x 256 (DUAL_M: two A tiles) -- one per accumulator.  A stage
// is then 48 KiB (gathered tile + two plain tiles), four stages deep, and every gathered row feeds twice the
// MMA work, which is what bounds these kernels (row gathers are many small TMA operations); the price is that
// the two accumulators no longer alternate between consecutive units.
//
// Roles per CTA (warp index):
//   0        TMA producer for the operands that are not gathered (both CTAs; completion bytes are counted
//            on the leader CTA's "full" barrier)
//   1        leader CTA: MMA issuer.  other CTA: idle
//   2..      EW epilogue warps (4 or 8)
//   2+EW..   GW gather warps (0, 4 or 8): the routed rows of the gathered operand by TMA tile::gather4, issued
//            from 32 threads spread over these warps (gather4 operations issued by one warp are serialised)
//
// Barriers.  full[s]: leader only; one arrival (the leader's expect_tx), tx = TMA bytes of both CTAs,
// gathered rows included.  empty[s], acc_full[a]: per CTA, signalled by the leader's multicast
// tcgen05.commit.  acc_empty[a]: leader only, one arrival per epilogue warp of both CTAs.  Every wait is
// bounded (ptx.cuh).
#pragma once
#include "epilogue.cuh"
#include "ptx.cuh"

namespace smoe {
namespace pair {

constexpr int BM = 128;          // rows per CTA (TMEM lanes); the pair's tile has 2 * BM rows
constexpr int BN = 256;          // tile columns = accumulator columns
constexpr int BN_CTA = 128;      // B rows each CTA stages
constexpr int BK = 64;
constexpr int STAGES = 6;
constexpr int UMMA_K = 16;
constexpr int A_STAGE_BYTES = BM * BK * 2;       // 16 KiB
constexpr int B_STAGE_BYTES = BN_CTA * BK * 2;   // 16 KiB
constexpr int CHUNK_BYTES = BK * 128;            // 64-element MN chunk: BK rows x 128 B
constexpr int MAX_EXPERTS = 1024;

// DUAL kernels keep warps 2 and 3 idle so that every role fills whole warpgroups (setmaxnreg is a warpgroup-wide
// instruction): warps 0-3 producer / MMA, 4-11 epilogue, 12-15 gather.
__host__ __device__ constexpr int threads(int epi_warps, int gather_warps, bool dual = false) {
  return 32 * ((dual ? 4 : 2) + epi_warps + gather_warps);
}

struct SharedStorage {
  uint64_t full[STAGES];
  uint64_t empty[STAGES];
  uint64_t acc_full[2];
  uint64_t acc_empty[2];
  uint32_t tmem_base;
  int abort_flag;
  int m_tile_prefix[MAX_EXPERTS + 1];  // ragged-M: exclusive prefix of ceil(count / 256) per expert
};

// Output staging of the plain-store epilogues: each epilogue warp owns 32 rows x (payload + 16 B pad).  A thread
// writes its accumulator row there, the warp reads it back so that consecutive lanes hold consecutive 16-byte pieces
// of one row, and stores whole 64- or 128-byte row segments: 4 or 8 requests to L2 per store instruction instead of
// 32 (with one row per lane the epilogue sent about as many requests to L2 as the main loop's operand fetches and
// competed with them).  Single tiles (4 epilogue warps): 128-byte payload; dual tiles (8 warps): 64-byte payload.
constexpr int STAGE_OUT_PITCH_WIDE = 144;    // 128 B payload: row r starts 36 words after row r-1 -> conflict-free
constexpr int STAGE_OUT_PITCH_NARROW = 80;   // 64 B payload
constexpr int STAGE_OUT_BYTES = 8 * 32 * STAGE_OUT_PITCH_NARROW;  // 20480 >= 4 * 32 * 144
static_assert(4 * 32 * STAGE_OUT_PITCH_WIDE <= STAGE_OUT_BYTES, "staging area");
constexpr int SMEM_BYTES =
    1024 + STAGES * (A_STAGE_BYTES + B_STAGE_BYTES) + ((sizeof(SharedStorage) + 15) & ~15) + STAGE_OUT_BYTES;
static_assert(SMEM_BYTES <= 227 * 1024, "shared memory per CTA");

struct Tile {
  int e;
  int row0;     // ragged-M: first grouped row of THIS CTA's 128 rows; ragged-K: first output row of this CTA
  int row_end;  // ragged-M: off[e+1]; ragged-K: M
  int n0;       // first column of the pair's 256-column tile
  int k_begin, k_end;
  int num_kb;
};

enum { DUAL_NONE = 0, DUAL_N = 1, DUAL_M = 2 };

// num_n counts work units along N (DUAL_N: 512 columns each).
template <bool RAGGED_K, int DUAL = DUAL_NONE>
__device__ __forceinline__ bool decode_tile(const GemmParams& p, const SharedStorage& ss, long long t, int num_n,
                                            uint32_t rank, Tile& tile) {
  constexpr int UNIT_N = DUAL == DUAL_N ? 2 * BN : BN;
  constexpr int UNIT_M = DUAL == DUAL_M ? 4 * BM : 2 * BM;
  if constexpr (!RAGGED_K) {
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
    tile.n0 = ni * UNIT_N;
    tile.k_begin = 0;
    tile.k_end = p.K;
    tile.num_kb = p.K / BK;
    return true;
  } else {
    const int num_m = (p.M + UNIT_M - 1) / UNIT_M;
    const long long per_e = static_cast<long long>(num_m) * num_n;
    if (t >= per_e * p.E) return false;
    const int e = static_cast<int>(t / per_e);
    const int rem = static_cast<int>(t % per_e);
    tile.e = e;
    tile.row0 = (rem / num_n) * UNIT_M + static_cast<int>(rank) * BM;
    tile.row_end = p.M;
    tile.n0 = (rem % num_n) * UNIT_N;
    tile.k_begin = p.off[e];
    tile.k_end = p.off[e + 1];
    tile.num_kb = (tile.k_end - tile.k_begin + BK - 1) / BK;
    return true;
  }
}

// What the MMA issuer needs to know about work unit t: whether it exists and how many k-blocks it has.  The full
// decode_tile (a 64-bit division, a binary search and two dependent global loads) would sit between the last MMA of
// one tile and the first of the next; for ragged-M the k-block count is a constant, for ragged-K the expert's token
// range is fetched one unit ahead by the caller.
template <bool RAGGED_K, int DUAL>
__device__ __forceinline__ long long num_units(const GemmParams& p, const SharedStorage& ss, int num_n) {
  if constexpr (!RAGGED_K) {
    return static_cast<long long>(ss.m_tile_prefix[p.E]) * num_n;
  } else {
    constexpr int UNIT_M = DUAL == DUAL_M ? 4 * BM : 2 * BM;
    const int num_m = (p.M + UNIT_M - 1) / UNIT_M;
    return static_cast<long long>(num_m) * num_n * p.E;
  }
}

template <bool RAGGED_K, int DUAL>
__device__ __forceinline__ int unit_num_kb(const GemmParams& p, long long t, long long total, int num_n) {
  if (t >= total) return 0;
  if constexpr (!RAGGED_K) {
    return p.K / BK;
  } else {
    constexpr int UNIT_M = DUAL == DUAL_M ? 4 * BM : 2 * BM;
    const int num_m = (p.M + UNIT_M - 1) / UNIT_M;
    const int e = static_cast<int>(t / (static_cast<long long>(num_m) * num_n));
    return (p.off[e + 1] - p.off[e] + BK - 1) / BK;
  }
}

template <bool RAGGED_K, bool A_GATHER, bool A_MN, bool B_GATHER, bool B_MN, int EPI, int EW, int GW,
          int DUAL = DUAL_NONE>
__global__ void __launch_bounds__(threads(EW, GW, DUAL != 0), 1)
grouped_gemm_pair_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                         const GemmParams p) {
  // DUAL: four stages of three 16 KiB tiles (A, B and the second plain tile X) instead of six stages of two
  constexpr int NSTAGES = DUAL != DUAL_NONE ? 4 : STAGES;
  constexpr int X_STAGE_BYTES = DUAL != DUAL_NONE ? A_STAGE_BYTES : 0;
  static_assert(DUAL != DUAL_N || !B_GATHER, "DUAL_N doubles the plain B tile");
  static_assert(DUAL != DUAL_M || (!A_GATHER && A_MN && RAGGED_K), "DUAL_M doubles the plain MN-major A tile of a ragged-K kernel");
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sA = smem;
  uint8_t* sB = smem + NSTAGES * A_STAGE_BYTES;
  uint8_t* sX = sB + NSTAGES * B_STAGE_BYTES;
  SharedStorage& ss = *reinterpret_cast<SharedStorage*>(smem + NSTAGES * (A_STAGE_BYTES + B_STAGE_BYTES + X_STAGE_BYTES));
  uint8_t* stage_out = reinterpret_cast<uint8_t*>(&ss) + ((sizeof(SharedStorage) + 15) & ~15);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();  // 0 = leader
  const bool leader = rank == 0;
  const long long first_tile = blockIdx.x >> 1;
  const long long tile_step = gridDim.x >> 1;
  volatile int* abort_flag = &ss.abort_flag;
  constexpr int UNIT_N = DUAL == DUAL_N ? 2 * BN : BN;
  const int num_n = (p.N + UNIT_N - 1) / UNIT_N;

  constexpr bool kGather = A_GATHER || B_GATHER;
  static_assert(!(A_GATHER && B_GATHER), "at most one operand is gathered");
  static_assert(!kGather || GW > 0, "a gathered operand needs gather warps");
  static_assert(EW == 4 || EW == 8, "4 or 8 epilogue warps");
  static_assert(GW == 0 || GW == 4 || GW == 8 || GW == 16, "0, 4, 8 or 16 gather warps");
  constexpr int GATHER_THREADS = 32 * GW;
  constexpr int FIRST_EPI_WARP = DUAL != DUAL_NONE ? 4 : 2;
  constexpr int FIRST_GATHER_WARP = FIRST_EPI_WARP + EW;
  static_assert(DUAL == DUAL_NONE || (EW == 8 && GW == 4), "dual tiles: 8 epilogue warps, 4 gather warps (512 threads)");
  constexpr uint32_t kTmaBytesPerCta = A_STAGE_BYTES + B_STAGE_BYTES + X_STAGE_BYTES;  // gathered rows included

  // ---- set-up -------------------------------------------------------------------------------
  if (threadIdx.x == 0) {
    for (int s = 0; s < NSTAGES; ++s) {
      mbar_init(smem_u32(&ss.full[s]), 1);
      mbar_init(smem_u32(&ss.empty[s]), 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(smem_u32(&ss.acc_full[a]), 1);
      mbar_init(smem_u32(&ss.acc_empty[a]), 2 * EW);
    }
    ss.abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == 0 && lane == 0) {
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(&ss.tmem_base), 2 * BN);  // all 512 columns: both CTAs get the same base
    tmem_relinquish();
  }
  if constexpr (!RAGGED_K) {
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
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();  // the other CTA's barriers are initialised before anything can arrive on them
  tc_fence_after();
  const uint32_t tmem_base = ss.tmem_base;

  // DUAL: the epilogue warps hold 128 accumulator values per thread; registers move to them from the other roles
  // (512 threads x 128 registers at launch; two warpgroups give up 72 registers per thread, two take 72).  Each
  // role branch starts with its own setmaxnreg so that the register limit is known along the whole branch.
  if (warp < FIRST_EPI_WARP) {
  if constexpr (DUAL != DUAL_NONE) asm volatile("setmaxnreg.dec.sync.aligned.u32 56;");
  // ---- TMA producer -------------------------------------------------------------------------
  if (warp == 0) {
    if constexpr (kTmaBytesPerCta > 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      Tile tile;
      for (long long t = first_tile; ok && decode_tile<RAGGED_K, DUAL>(p, ss, t, num_n, rank, tile); t += tile_step) {
        for (int kb = 0; kb < tile.num_kb; ++kb) {
          if (!mbar_wait(smem_u32(&ss.empty[stage]), phase ^ 1u, abort_flag)) { ok = false; break; }
          const uint32_t bar = map_to_cta(smem_u32(&ss.full[stage]), 0);  // the leader's barrier
          const uint32_t a_dst = smem_u32(sA + stage * A_STAGE_BYTES);
          const uint32_t b_dst = smem_u32(sB + stage * B_STAGE_BYTES);
          if (leader && lane == 0) mbar_arrive_expect_tx(smem_u32(&ss.full[stage]), 2 * kTmaBytesPerCta);
          __syncwarp();
          const int k0 = RAGGED_K ? (tile.k_begin + kb * BK) : kb * BK;
          if constexpr (!A_GATHER) {
            if constexpr (!A_MN) {
              if (lane == 0) tma_load_2d_pair(&tmA, bar, a_dst, k0, tile.row0);
            } else {
              if (lane < BM / 64) tma_load_2d_pair(&tmA, bar, a_dst + lane * CHUNK_BYTES, tile.row0 + 64 * lane, k0);
            }
          }
          if constexpr (!B_GATHER) {
            const int nb = tile.n0 + static_cast<int>(rank) * BN_CTA;  // this CTA's half of the B rows
            if constexpr (!B_MN) {
              if (lane == 0) tma_load_2d_pair(&tmB, bar, b_dst, k0, tile.e * p.b_rows_per_expert + nb);
            } else {
              const int krow = RAGGED_K ? k0 : (tile.e * p.b_rows_per_expert + k0);
              if (lane < BN_CTA / 64) tma_load_2d_pair(&tmB, bar, b_dst + lane * CHUNK_BYTES, nb + 64 * lane, krow);
            }
          }
          if constexpr (DUAL == DUAL_N) {  // the unit's second B tile: columns n0 + 256 ...
            const uint32_t x_dst = smem_u32(sX + stage * X_STAGE_BYTES);
            const int nb = tile.n0 + BN + static_cast<int>(rank) * BN_CTA;
            if constexpr (!B_MN) {
              if (lane == 0) tma_load_2d_pair(&tmB, bar, x_dst, k0, tile.e * p.b_rows_per_expert + nb);
            } else {
              const int krow = RAGGED_K ? k0 : (tile.e * p.b_rows_per_expert + k0);
              if (lane < BN_CTA / 64) tma_load_2d_pair(&tmB, bar, x_dst + lane * CHUNK_BYTES, nb + 64 * lane, krow);
            }
          }
          if constexpr (DUAL == DUAL_M) {  // the unit's second A tile: rows row0 + 256 ...
            const uint32_t x_dst = smem_u32(sX + stage * X_STAGE_BYTES);
            if (lane < BM / 64)
              tma_load_2d_pair(&tmA, bar, x_dst + lane * CHUNK_BYTES, tile.row0 + 2 * BM + 64 * lane, k0);
          }
          if (++stage == NSTAGES) { stage = 0; phase ^= 1u; }
        }
      }
      if (!ok && lane == 0 && p.status) atomicCAS(p.status, ST_OK, ST_TIMEOUT_PRODUCER);
    }
  }
  // ---- MMA issuer (leader) / gather relay (other CTA) ----------------------------------------
  else if (warp == 1) {
    if (leader) {
      constexpr uint32_t idesc = make_idesc_bf16(2 * BM, BN, A_MN, B_MN);
      constexpr uint32_t a_lbo = A_MN ? CHUNK_BYTES : 16;
      constexpr uint32_t b_lbo = B_MN ? CHUNK_BYTES : 16;
      constexpr uint32_t a_kstep = A_MN ? (UMMA_K * 128) : (UMMA_K * 2);
      constexpr uint32_t b_kstep = B_MN ? (UMMA_K * 128) : (UMMA_K * 2);
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      const long long total_units = num_units<RAGGED_K, DUAL>(p, ss, num_n);
      int next_kb = unit_num_kb<RAGGED_K, DUAL>(p, first_tile, total_units, num_n);
      for (long long t = first_tile; ok && t < total_units; t += tile_step) {
        const int num_kb = next_kb;
        next_kb = unit_num_kb<RAGGED_K, DUAL>(p, t + tile_step, total_units, num_n);  // loads overlap this unit's MMAs
        if (num_kb == 0) continue;
        if constexpr (DUAL == DUAL_NONE) {
          if (!mbar_wait(smem_u32(&ss.acc_empty[acc]), acc_phase ^ 1u, abort_flag)) { ok = false; break; }
        } else {
          // both accumulators belong to this unit; the first group may start as soon as the epilogue has copied the
          // previous unit's first accumulator out, the second group waits for the second one (below)
          if (!mbar_wait(smem_u32(&ss.acc_empty[0]), acc_phase ^ 1u, abort_flag)) { ok = false; break; }
        }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + (DUAL == DUAL_NONE ? acc * BN : 0);
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(smem_u32(&ss.full[stage]), phase, abort_flag)) { ok = false; break; }
          tc_fence_after();
          const uint64_t a_desc = make_smem_desc(smem_u32(sA + stage * A_STAGE_BYTES), a_lbo, 1024);
          const uint64_t b_desc = make_smem_desc(smem_u32(sB + stage * B_STAGE_BYTES), b_lbo, 1024);
          if (lane == 0) {
#pragma unroll
            for (int k4 = 0; k4 < BK / UMMA_K; ++k4) {
              umma_bf16_pair(d_tmem, a_desc + ((k4 * a_kstep) >> 4), b_desc + ((k4 * b_kstep) >> 4), idesc,
                             (kb > 0 || k4 > 0) ? 1u : 0u);
            }
          }
          if constexpr (DUAL != DUAL_NONE) {
            if (kb == 0) {  // the second accumulator of the previous unit has been copied out
              __syncwarp();
              if (!mbar_wait(smem_u32(&ss.acc_empty[1]), acc_phase ^ 1u, abort_flag)) { ok = false; break; }
              tc_fence_after();
            }
          }
          if (lane == 0) {
            if constexpr (DUAL == DUAL_N) {
              const uint64_t x_desc = make_smem_desc(smem_u32(sX + stage * X_STAGE_BYTES), b_lbo, 1024);
#pragma unroll
              for (int k4 = 0; k4 < BK / UMMA_K; ++k4) {
                umma_bf16_pair(d_tmem + BN, a_desc + ((k4 * a_kstep) >> 4), x_desc + ((k4 * b_kstep) >> 4), idesc,
                               (kb > 0 || k4 > 0) ? 1u : 0u);
              }
            }
            if constexpr (DUAL == DUAL_M) {
              const uint64_t x_desc = make_smem_desc(smem_u32(sX + stage * X_STAGE_BYTES), a_lbo, 1024);
#pragma unroll
              for (int k4 = 0; k4 < BK / UMMA_K; ++k4) {
                umma_bf16_pair(d_tmem + BN, x_desc + ((k4 * a_kstep) >> 4), b_desc + ((k4 * b_kstep) >> 4), idesc,
                               (kb > 0 || k4 > 0) ? 1u : 0u);
              }
            }
            umma_commit_pair(smem_u32(&ss.empty[stage]), 3);  // frees the stage in both CTAs
          }
          __syncwarp();
          if (++stage == NSTAGES) { stage = 0; phase ^= 1u; }
        }
        if (!ok) break;
        if constexpr (DUAL == DUAL_NONE) {
          if (lane == 0) umma_commit_pair(smem_u32(&ss.acc_full[acc]), 3);
          __syncwarp();
          if (++acc == 2) { acc = 0; acc_phase ^= 1u; }
        } else {
          if (lane == 0) {
            umma_commit_pair(smem_u32(&ss.acc_full[0]), 3);
            umma_commit_pair(smem_u32(&ss.acc_full[1]), 3);
          }
          __syncwarp();
          acc_phase ^= 1u;
        }
      }
      if (!ok && lane == 0 && p.status) atomicCAS(p.status, ST_OK, ST_TIMEOUT_MMA);
    }
  }
  }  // warps below FIRST_EPI_WARP (DUAL: warps 2 and 3 idle)
  // ---- gather producers ----------------------------------------------------------------------
  else if (warp >= FIRST_GATHER_WARP) {
    if constexpr (DUAL != DUAL_NONE) asm volatile("setmaxnreg.dec.sync.aligned.u32 56;");
    if constexpr (kGather) {
      const int gt = threadIdx.x - 32 * FIRST_GATHER_WARP;
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      Tile tile;
      {
        // 32 issuing threads (every GATHER_THREADS/32-th thread, so they spread over all gather warps), each
        // fetching 4 rows x 128 B per stage with one gather4.
        constexpr int STRIDE = GATHER_THREADS / 32;
        const bool issuer = (gt % STRIDE) == 0;
        const int j = gt / STRIDE;  // 0..31
        const CUtensorMap* tm = A_GATHER ? &tmA : &tmB;
        uint8_t* stage_base = A_GATHER ? sA : sB;
        constexpr int STAGE_BYTES = A_GATHER ? A_STAGE_BYTES : B_STAGE_BYTES;
        for (long long t = first_tile; ok && decode_tile<RAGGED_K, DUAL>(p, ss, t, num_n, rank, tile); t += tile_step) {
          if constexpr (!RAGGED_K) {
            int r4[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              const int r = tile.row0 + 4 * j + i;
              r4[i] = (r < p.total_rows) ? p.gather[r] : 0;
            }
            for (int kb = 0; kb < tile.num_kb; ++kb) {
              if (!mbar_wait(smem_u32(&ss.empty[stage]), phase ^ 1u, abort_flag)) { ok = false; break; }
              if (issuer)
                tma_gather4_pair(tm, map_to_cta(smem_u32(&ss.full[stage]), 0),
                                 smem_u32(stage_base + stage * STAGE_BYTES) + j * 512, kb * BK, r4[0], r4[1], r4[2],
                                 r4[3]);
              if (++stage == NSTAGES) { stage = 0; phase ^= 1u; }
            }
          } else {
            const int chunk = j >> 4, tq = j & 15;  // 2 chunks of 64 columns, 16 groups of 4 tokens
            const int col0 = (A_GATHER ? tile.row0 : tile.n0 + static_cast<int>(rank) * BN_CTA) + 64 * chunk;
            int cur[4], nxt[4];
            auto load_idx = [&](int kb, int (&dst_idx)[4]) {
#pragma unroll
              for (int i = 0; i < 4; ++i) {
                const int tok = tile.k_begin + kb * BK + 4 * tq + i;
                dst_idx[i] = (kb < tile.num_kb && tok < tile.k_end) ? p.gather[tok] : p.gather_rows;  // out of range: zeros
              }
            };
            load_idx(0, cur);
            load_idx(1, nxt);
            for (int kb = 0; kb < tile.num_kb; ++kb) {
              if (!mbar_wait(smem_u32(&ss.empty[stage]), phase ^ 1u, abort_flag)) { ok = false; break; }
              if (issuer)
                tma_gather4_pair(tm, map_to_cta(smem_u32(&ss.full[stage]), 0),
                                 smem_u32(stage_base + stage * STAGE_BYTES) + chunk * CHUNK_BYTES + tq * 512, col0,
                                 cur[0], cur[1], cur[2], cur[3]);
#pragma unroll
              for (int i = 0; i < 4; ++i) cur[i] = nxt[i];
              load_idx(kb + 2, nxt);
              if (++stage == NSTAGES) { stage = 0; phase ^= 1u; }
            }
          }
        }
      }
      if (!ok && (gt & 31) == 0 && p.status) atomicCAS(p.status, ST_OK, ST_TIMEOUT_PRODUCER);
    }
  }
  // ---- epilogue -----------------------------------------------------------------------------
  else {
    if constexpr (DUAL != DUAL_NONE) asm volatile("setmaxnreg.inc.sync.aligned.u32 200;");
    const int quad = warp & 3;
    constexpr int COL_SPLIT = EW / 4;
    constexpr int COLS_PER_WARP = BN / COL_SPLIT;
    const int col_half = (warp - FIRST_EPI_WARP) >> 2;
    const int row_in_tile = quad * 32 + lane;
    int acc = 0;
    uint32_t acc_phase = 0;
    bool ok = true;
    Tile tile;
    for (long long t = first_tile; ok && decode_tile<RAGGED_K, DUAL>(p, ss, t, num_n, rank, tile); t += tile_step) {
      const bool have_acc = tile.num_kb > 0;
      constexpr int SUBTILES = DUAL == DUAL_NONE ? 1 : 2;
      if constexpr (DUAL != DUAL_NONE && EPI == EPI_STORE) {
        // Plain stores: both accumulators are copied out, rounded to bf16 (two values per register, 64 registers
        // per accumulator) and handed back before anything is stored, so the next unit's MMAs wait for two
        // tensor-memory reads and not for this unit's stores.
        constexpr int CHUNKS = COLS_PER_WARP / 32;  // 4
        static_assert(COLS_PER_WARP == 128, "dual tiles use 8 epilogue warps");
        uint32_t packed[2][CHUNKS * 16];
#pragma unroll
        for (int sub = 0; sub < 2; ++sub) {
          if (have_acc) {
            if (!mbar_wait(smem_u32(&ss.acc_full[sub]), acc_phase, abort_flag)) { ok = false; break; }
            tc_fence_after();
            const uint32_t t_addr = tmem_base + sub * BN + (static_cast<uint32_t>(quad * 32) << 16);
#pragma unroll
            for (int h = 0; h < CHUNKS / 2; ++h) {
              uint32_t v0[32], v1[32];
              tmem_ld32(t_addr + (col_half * CHUNKS + 2 * h) * 32, v0);
              tmem_ld32(t_addr + (col_half * CHUNKS + 2 * h + 1) * 32, v1);
              tmem_ld_wait();
              if (h == CHUNKS / 2 - 1) {  // last read of this accumulator: give it back before converting
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive_cluster_relaxed(map_to_cta(smem_u32(&ss.acc_empty[sub]), 0));
              }
#pragma unroll
              for (int j = 0; j < 16; ++j) {
                packed[sub][(2 * h) * 16 + j] = pack_bf16(__uint_as_float(v0[2 * j]), __uint_as_float(v0[2 * j + 1]));
                packed[sub][(2 * h + 1) * 16 + j] = pack_bf16(__uint_as_float(v1[2 * j]), __uint_as_float(v1[2 * j + 1]));
              }
            }
          } else {
#pragma unroll
            for (int j = 0; j < CHUNKS * 16; ++j) packed[sub][j] = 0u;
          }
        }
        if (!ok) break;
        {
          // stores: 64-byte row segments through this warp's staging rows (8 rows per store instruction)
          const uint32_t my_stage = smem_u32(stage_out) + (warp - FIRST_EPI_WARP) * (32 * STAGE_OUT_PITCH_NARROW);
#pragma unroll
          for (int sub = 0; sub < 2; ++sub) {
            const int row_base = tile.row0 + (DUAL == DUAL_M ? sub * 2 * BM : 0) + quad * 32;
            const int n0 = tile.n0 + (DUAL == DUAL_N ? sub * BN : 0);
            __nv_bfloat16* out = p.out0 + (RAGGED_K ? tile.e * p.out0_expert_stride : 0ll);
#pragma unroll
            for (int c = 0; c < CHUNKS; ++c) {
              const int n = n0 + (col_half * CHUNKS + c) * 32;
              if (n >= p.N) break;
#pragma unroll
              for (int q = 0; q < 4; ++q)
                st_shared_v4(my_stage + lane * STAGE_OUT_PITCH_NARROW + 16 * q, packed[sub][c * 16 + 4 * q],
                             packed[sub][c * 16 + 4 * q + 1], packed[sub][c * 16 + 4 * q + 2],
                             packed[sub][c * 16 + 4 * q + 3]);
              __syncwarp();
#pragma unroll
              for (int i = 0; i < 4; ++i) {
                const int rr = 8 * i + (lane >> 2);
                const uint4 w = ld_shared_v4(my_stage + rr * STAGE_OUT_PITCH_NARROW + 16 * (lane & 3));
                const int r = row_base + rr;
                if (r < tile.row_end) {
                  uint4* dst = reinterpret_cast<uint4*>(out + r * p.ld0 + n + 8 * (lane & 3));
                  *dst = p.accumulate ? add_bf16x8(w, dst) : w;
                }
              }
              __syncwarp();
            }
          }
        }
        if (have_acc) acc_phase ^= 1u;
        continue;
      }
#pragma unroll 1
      for (int sub = 0; sub < SUBTILES && ok; ++sub) {
        if constexpr (DUAL != DUAL_NONE) acc = sub;
        const int r = tile.row0 + (DUAL == DUAL_M ? sub * 2 * BM : 0) + row_in_tile;
        const int n0 = tile.n0 + (DUAL == DUAL_N ? sub * BN : 0);
        const bool row_ok = r < tile.row_end;
        float score = 0.f;
        if constexpr (EPI == EPI_DSWIGLU || EPI == EPI_DACT || EPI == EPI_SCATTER || EPI == EPI_STORE_ROWS) {
          if (row_ok && (EPI != EPI_STORE_ROWS || p.scores != nullptr))
            score = load_score(p.scores, p.scores_are_bf16, p.s_scatter[r]);
        }
        if constexpr (EPI == EPI_DSWIGLU || EPI == EPI_DACT) {
          // the epilogue reads this thread's piece of the saved pre-activation row: have the L2 fetch it while the
          // unit's MMAs are still running
          if (row_ok && n0 + col_half * COLS_PER_WARP < p.N) {
            const int zw = (EPI == EPI_DACT && !act_is_gated(p.act)) ? 1 : 2;  // z columns per accumulator column
            prefetch_l2_lines(p.z + static_cast<long long>(r) * (zw * p.N) + zw * (n0 + col_half * COLS_PER_WARP),
                              zw * COLS_PER_WARP * 2 / 128);
          }
        }
        if (have_acc) {
          if (!mbar_wait(smem_u32(&ss.acc_full[acc]), acc_phase, abort_flag)) { ok = false; break; }
          tc_fence_after();
        }
        float ds_acc = 0.f;
        const uint32_t t_addr = tmem_base + acc * BN + (static_cast<uint32_t>(quad * 32) << 16);
        if constexpr (DUAL != DUAL_NONE) {
          // Copy this warp's columns of the accumulator into registers and hand the accumulator back at once: the
          // next unit's MMAs need both accumulators, so the epilogue arithmetic and stores must not hold them.
          static_assert(DUAL == DUAL_NONE || COLS_PER_WARP == 128, "dual tiles use 8 epilogue warps");
          constexpr int CHUNKS = COLS_PER_WARP / 32;
          uint32_t v[CHUNKS][32];
          if (have_acc) {
#pragma unroll
            for (int c = 0; c < CHUNKS; ++c) tmem_ld32(t_addr + (col_half * CHUNKS + c) * 32, v[c]);
            tmem_ld_wait();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster_relaxed(map_to_cta(smem_u32(&ss.acc_empty[acc]), 0));
          } else {
#pragma unroll
            for (int c = 0; c < CHUNKS; ++c)
#pragma unroll
              for (int j = 0; j < 32; ++j) v[c][j] = 0u;
          }
          if constexpr (EPI == EPI_SWIGLU) {
            // z (unless not wanted) and y1 = silu(gate) * up leave through the warp's staging rows as 64-byte row
            // segments: one per 32 accumulator columns for z, one per 64 for y1 (N = 2I is a multiple of 128, so
            // chunks come in pairs)
            const uint32_t my_stage = smem_u32(stage_out) + (warp - FIRST_EPI_WARP) * (32 * STAGE_OUT_PITCH_NARROW);
            const int row_base = r - lane;
            uint32_t yp[16];
#pragma unroll
            for (int c = 0; c < CHUNKS; ++c) {
              const int n = n0 + (col_half * CHUNKS + c) * 32;
              if (n >= p.N) break;
              uint32_t zp[16];
#pragma unroll
              for (int j = 0; j < 16; ++j) {
                const float g = __uint_as_float(v[c][2 * j]);
                const float u = __uint_as_float(v[c][2 * j + 1]);
                zp[j] = pack_bf16(g, u);
                v[c][j] = __float_as_uint(g * sigmoid_f(g) * u);  // the chunk's 16 products, kept in place
              }
#pragma unroll
              for (int j = 0; j < 8; ++j)
                yp[(c & 1) * 8 + j] = pack_bf16(__uint_as_float(v[c][2 * j]), __uint_as_float(v[c][2 * j + 1]));
              if (p.out0 != nullptr)
                warp_store_rows64<STAGE_OUT_PITCH_NARROW>(my_stage, lane, zp, p.out0, p.ld0, row_base, tile.row_end, n);
              if (c & 1)
                warp_store_rows64<STAGE_OUT_PITCH_NARROW>(my_stage, lane, yp, p.out1, p.ld1, row_base, tile.row_end,
                                                          (n - 32) >> 1);
            }
          } else if (row_ok) {
#pragma unroll
            for (int c = 0; c < CHUNKS; ++c) {
              const int n = n0 + (col_half * CHUNKS + c) * 32;
              if (n < p.N) epilogue_chunk<EPI, RAGGED_K>(p, tile.e, r, n, v[c], score, ds_acc);
            }
          }
        } else if constexpr (EPI == EPI_DSWIGLU && EW == 4) {
          // dSwiGLU of single tiles, 32 accumulator columns at a time: the 128-byte piece of the saved pre-activation
          // row comes in, and the dz (128 B) and y1*s (64 B) pieces go out, through this warp's staging rows with
          // whole-row-segment accesses; the arithmetic stays one row per thread.
          const uint32_t my_stage = smem_u32(stage_out) + (warp - FIRST_EPI_WARP) * (32 * STAGE_OUT_PITCH_WIDE);
          const int row_base = tile.row0 + quad * 32;
#pragma unroll 1
          for (int c = 0; c < COLS_PER_WARP / 32; ++c) {
            const int n = n0 + c * 32;
            if (n >= p.N) break;
            uint32_t v[32], zw[32];
            if (have_acc) tmem_ld32(t_addr + c * 32, v);
            warp_load_rows128<STAGE_OUT_PITCH_WIDE>(my_stage, lane, zw, p.z, 2ll * p.N, row_base, tile.row_end, 2 * n);
            if (have_acc) {
              tmem_ld_wait();
            } else {
#pragma unroll
              for (int j = 0; j < 32; ++j) v[j] = 0u;
            }
            uint32_t ys[16];
#pragma unroll
            for (int i = 0; i < 32; ++i) {
              const __nv_bfloat162 gu = *reinterpret_cast<const __nv_bfloat162*>(&zw[i]);
              const float g = __low2float(gu), u = __high2float(gu);
              const float dy = __uint_as_float(v[i]);
              const float sig = sigmoid_f(g);
              const float silu = g * sig;
              const float y1 = silu * u;
              ds_acc += dy * y1;
              const float dg = dy * u * (sig * (1.f + g * (1.f - sig))) * score;
              const float du = dy * silu * score;
              zw[i] = pack_bf16(dg, du);
              v[i] = __float_as_uint(y1 * score);
            }
#pragma unroll
            for (int j = 0; j < 16; ++j) ys[j] = pack_bf16(__uint_as_float(v[2 * j]), __uint_as_float(v[2 * j + 1]));
            warp_store_rows128<STAGE_OUT_PITCH_WIDE>(my_stage, lane, zw, p.out0, p.ld0, row_base, tile.row_end, 2 * n);
            warp_store_rows64<STAGE_OUT_PITCH_WIDE>(my_stage, lane, ys, p.out1, p.ld1, row_base, tile.row_end, n);
          }
        } else if constexpr (EPI == EPI_STORE && EW == 4) {
          // plain stores of single tiles: two 32-column chunks (a 128-byte row segment) at a time through this warp's
          // staging rows, 4 full rows per store instruction
          const uint32_t my_stage = smem_u32(stage_out) + (warp - FIRST_EPI_WARP) * (32 * STAGE_OUT_PITCH_WIDE);
          const int row_base = tile.row0 + quad * 32;
          __nv_bfloat16* out = p.out0 + (RAGGED_K ? tile.e * p.out0_expert_stride : 0ll);
#pragma unroll 1
          for (int c = 0; c < COLS_PER_WARP / 32; c += 2) {
            const int n = n0 + c * 32;
            if (n >= p.N) break;  // N is a multiple of 64: both chunks exist or neither
            uint32_t v0[32], v1[32];
            if (have_acc) {
              tmem_ld32(t_addr + c * 32, v0);
              tmem_ld32(t_addr + (c + 1) * 32, v1);
              tmem_ld_wait();
            } else {
#pragma unroll
              for (int j = 0; j < 32; ++j) v0[j] = v1[j] = 0u;
            }
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              st_shared_v4(my_stage + lane * STAGE_OUT_PITCH_WIDE + 16 * q,
                           pack_bf16(__uint_as_float(v0[8 * q]), __uint_as_float(v0[8 * q + 1])),
                           pack_bf16(__uint_as_float(v0[8 * q + 2]), __uint_as_float(v0[8 * q + 3])),
                           pack_bf16(__uint_as_float(v0[8 * q + 4]), __uint_as_float(v0[8 * q + 5])),
                           pack_bf16(__uint_as_float(v0[8 * q + 6]), __uint_as_float(v0[8 * q + 7])));
              st_shared_v4(my_stage + lane * STAGE_OUT_PITCH_WIDE + 64 + 16 * q,
                           pack_bf16(__uint_as_float(v1[8 * q]), __uint_as_float(v1[8 * q + 1])),
                           pack_bf16(__uint_as_float(v1[8 * q + 2]), __uint_as_float(v1[8 * q + 3])),
                           pack_bf16(__uint_as_float(v1[8 * q + 4]), __uint_as_float(v1[8 * q + 5])),
                           pack_bf16(__uint_as_float(v1[8 * q + 6]), __uint_as_float(v1[8 * q + 7])));
            }
            __syncwarp();
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              const int rr = 4 * i + (lane >> 3);
              const uint4 w = ld_shared_v4(my_stage + rr * STAGE_OUT_PITCH_WIDE + 16 * (lane & 7));
              const int rw = row_base + rr;
              if (rw < tile.row_end) {
                uint4* dst = reinterpret_cast<uint4*>(out + rw * p.ld0 + n + 8 * (lane & 7));
                *dst = p.accumulate ? add_bf16x8(w, dst) : w;
              }
            }
            __syncwarp();
          }
        } else {
#pragma unroll 1
          for (int c = col_half * (COLS_PER_WARP / 32); c < (col_half + 1) * (COLS_PER_WARP / 32); ++c) {
            const int n = n0 + c * 32;
            if (n >= p.N) break;
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
        }
        if constexpr (EPI == EPI_DSWIGLU || EPI == EPI_DACT) {
          if (row_ok && n0 < p.N) {
            float* dsp = p.ds_partial + static_cast<long long>(2 * (n0 / BN)) * p.total_rows + r;
            if constexpr (COL_SPLIT == 2) {
              dsp[static_cast<long long>(col_half) * p.total_rows] = ds_acc;
            } else {
              dsp[0] = ds_acc;
              dsp[p.total_rows] = 0.f;
            }
          }
        }
        if constexpr (DUAL == DUAL_NONE) {
          if (have_acc) {
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(map_to_cta(smem_u32(&ss.acc_empty[acc]), 0));
            if (++acc == 2) { acc = 0; acc_phase ^= 1u; }
          }
        }
      }
      if constexpr (DUAL != DUAL_NONE) {
        if (have_acc) acc_phase ^= 1u;
      }
    }
    if (!ok && lane == 0 && p.status) atomicCAS(p.status, ST_OK, ST_TIMEOUT_EPILOGUE);
  }

  // ---- tear-down ----------------------------------------------------------------------------
  if (*abort_flag != 0) {
    const uint64_t t0 = global_timer_ns();
    while (global_timer_ns() - t0 < 200000ull) __nanosleep(1000);
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();  // neither CTA leaves while the other may still signal its barriers or read its smem
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 2 * BN);
  }
}

}  // namespace pair
}  // namespace smoe

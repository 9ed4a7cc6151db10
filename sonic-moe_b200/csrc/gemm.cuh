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

enum Epilogue : int {
  EPI_STORE = 0,    // out0[r, n] = bf16(acc)
  EPI_SWIGLU = 1,   // out0[r, n] = bf16(acc) (unless out0 == nullptr); out1[r, n/2] = silu(acc[2j]) * acc[2j+1]
  EPI_DSWIGLU = 2,  // acc = dy1; reads z, score; writes dz (out0), y1*s (out1), per-row partial of ds
  EPI_SCATTER = 3,  // red.add fp32: acc_out[token(r), n] += score(r) * acc
};

// Status codes written to GemmParams::status (first failure wins).
enum Status : int { ST_OK = 0, ST_TIMEOUT_PRODUCER = 1, ST_TIMEOUT_MMA = 2, ST_TIMEOUT_EPILOGUE = 3 };

struct GemmParams {
  int E;            // experts
  int M;            // ragged-K: rows of each expert's output; ragged-M: unused
  int N;            // output columns (per expert)
  int K;            // ragged-M: reduction length; ragged-K: unused
  int total_rows;   // rows of the grouped (expert-sorted) layout
  int gather_rows;  // rows of the tensor a gather reads from (an index >= gather_rows reads zeros)
  int b_rows_per_expert;  // ragged-M: rows one expert occupies in B's flattened 2D tensor map
  const int* off;         // (E+1) first grouped row of every expert
  const int* gather;      // (total_rows) source row of every grouped row, or nullptr
  const __nv_bfloat16* gather_src;  // the tensor the gather reads (LSU-gather variant)
  long long gather_ld;              // its row pitch in elements
  __nv_bfloat16* out0;
  long long ld0;
  long long out0_expert_stride;  // ragged-K only
  __nv_bfloat16* out1;
  long long ld1;
  // EPI_DSWIGLU / EPI_SCATTER
  const __nv_bfloat16* z;   // (total_rows, 2N) pre-activation saved by the forward pass
  const void* scores;       // flat routing scores, fp32 or bf16
  int scores_are_bf16;
  const int* s_scatter;     // (total_rows) flat score slot of every grouped row
  float* ds_partial;        // (2 * ceil(N/BN), total_rows) fp32: one row of partials per 128 accumulator columns
  float* acc_out;           // EPI_SCATTER: (gather_rows, N) fp32
  int* status;              // device word, 0 = ok
};

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

__device__ __forceinline__ float load_score(const void* scores, int is_bf16, int slot) {
  return is_bf16 ? __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(scores)[slot])
                 : reinterpret_cast<const float*>(scores)[slot];
}

__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

__device__ __forceinline__ float sigmoid_f(float x) { return __fdividef(1.0f, 1.0f + __expf(-x)); }

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
        if (!mbar_wait_warp(smem_u32(&ss.empty[stage]), phase ^ 1u, abort_flag)) { ok = false; break; }
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
      if (!mbar_wait_warp(smem_u32(&ss.acc_empty[acc]), acc_phase ^ 1u, abort_flag)) { ok = false; break; }
      tc_fence_after();
      const uint32_t d_tmem = tmem_base + acc * BN;
      for (int kb = 0; kb < tile.num_kb; ++kb) {
        if (!mbar_wait_warp(smem_u32(&ss.full[stage]), phase, abort_flag)) { ok = false; break; }
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
            if (!mbar_wait_warp(smem_u32(&ss.empty[stage]), phase ^ 1u, abort_flag)) { ok = false; break; }
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
          int idx[PASSES];
          auto load_idx = [&](int kb) {
            const int k0 = tile.k_begin + kb * BK;
#pragma unroll
            for (int i = 0; i < PASSES; ++i) {
              const int tok = k0 + rb + ROWS_PER_PASS * i;
              idx[i] = (tok < tile.k_end && col_ok) ? p.gather[tok] : -1;
            }
          };
          if (tile.num_kb > 0) load_idx(0);
          for (int kb = 0; kb < tile.num_kb; ++kb) {
            if (!mbar_wait_warp(smem_u32(&ss.empty[stage]), phase ^ 1u, abort_flag)) { ok = false; break; }
            const uint32_t dst = smem_u32(stage_base + stage * STAGE_BYTES) + chunk * CHUNK_BYTES;
#pragma unroll
            for (int i = 0; i < PASSES; ++i) {
              const int r = rb + ROWS_PER_PASS * i;
              const bool valid = idx[i] >= 0;
              const __nv_bfloat16* src = src_col + static_cast<long long>(valid ? idx[i] : 0) * p.gather_ld;
              cp_async16(dst + r * 128 + ((c ^ (r & 7)) << 4), src, valid ? 16u : 0u);
            }
            cp_async_arrive_noinc(smem_u32(&ss.full[stage]));
            if (kb + 1 < tile.num_kb) load_idx(kb + 1);  // in flight while the next stage is awaited
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
        if (!mbar_wait_warp(smem_u32(&ss.acc_full[acc]), acc_phase, abort_flag)) { ok = false; break; }
        tc_fence_after();
      }
      float score = 0.f;
      int slot = 0;
      if constexpr (EPI == EPI_DSWIGLU || EPI == EPI_SCATTER) {
        if (row_ok) {
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
        if constexpr (EPI == EPI_STORE) {
          __nv_bfloat16* dst = p.out0 + (RAGGED_K ? tile.e * p.out0_expert_stride : 0ll) + r * p.ld0 + n;
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            uint4 w;
            w.x = pack_bf16(__uint_as_float(v[8 * j + 0]), __uint_as_float(v[8 * j + 1]));
            w.y = pack_bf16(__uint_as_float(v[8 * j + 2]), __uint_as_float(v[8 * j + 3]));
            w.z = pack_bf16(__uint_as_float(v[8 * j + 4]), __uint_as_float(v[8 * j + 5]));
            w.w = pack_bf16(__uint_as_float(v[8 * j + 6]), __uint_as_float(v[8 * j + 7]));
            reinterpret_cast<uint4*>(dst)[j] = w;
          }
        } else if constexpr (EPI == EPI_SWIGLU) {
          if (p.out0 != nullptr) {
            __nv_bfloat16* dst = p.out0 + r * p.ld0 + n;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              uint4 w;
              w.x = pack_bf16(__uint_as_float(v[8 * j + 0]), __uint_as_float(v[8 * j + 1]));
              w.y = pack_bf16(__uint_as_float(v[8 * j + 2]), __uint_as_float(v[8 * j + 3]));
              w.z = pack_bf16(__uint_as_float(v[8 * j + 4]), __uint_as_float(v[8 * j + 5]));
              w.w = pack_bf16(__uint_as_float(v[8 * j + 6]), __uint_as_float(v[8 * j + 7]));
              reinterpret_cast<uint4*>(dst)[j] = w;
            }
          }
          // gate = even column, up = odd column
          float y[16];
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            const float g = __uint_as_float(v[2 * j]);
            const float u = __uint_as_float(v[2 * j + 1]);
            y[j] = g * sigmoid_f(g) * u;
          }
          __nv_bfloat16* dst1 = p.out1 + r * p.ld1 + (n >> 1);
#pragma unroll
          for (int j = 0; j < 2; ++j) {
            uint4 w;
            w.x = pack_bf16(y[8 * j + 0], y[8 * j + 1]);
            w.y = pack_bf16(y[8 * j + 2], y[8 * j + 3]);
            w.z = pack_bf16(y[8 * j + 4], y[8 * j + 5]);
            w.w = pack_bf16(y[8 * j + 6], y[8 * j + 7]);
            reinterpret_cast<uint4*>(dst1)[j] = w;
          }
        } else if constexpr (EPI == EPI_DSWIGLU) {
          // acc[., i] = dy1[r, i]; z[r, 2i] = gate, z[r, 2i+1] = up
          const uint4* zsrc = reinterpret_cast<const uint4*>(p.z + static_cast<long long>(r) * (2ll * p.N) + 2 * n);
          __nv_bfloat16* dz_dst = p.out0 + r * p.ld0 + 2 * n;
          __nv_bfloat16* ys_dst = p.out1 + r * p.ld1 + n;
#pragma unroll
          for (int j = 0; j < 4; ++j) {  // 8 accumulator columns per step
            const uint4 za = zsrc[2 * j], zb = zsrc[2 * j + 1];
            const uint32_t zw[8] = {za.x, za.y, za.z, za.w, zb.x, zb.y, zb.z, zb.w};
            uint32_t dzw[8];
            float ys[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              const __nv_bfloat162 gu = *reinterpret_cast<const __nv_bfloat162*>(&zw[i]);
              const float g = __low2float(gu), u = __high2float(gu);
              const float dy = __uint_as_float(v[8 * j + i]);
              const float sig = sigmoid_f(g);
              const float silu = g * sig;
              const float y1 = silu * u;
              ds_acc += dy * y1;
              const float dg = dy * u * (sig * (1.f + g * (1.f - sig))) * score;
              const float du = dy * silu * score;
              dzw[i] = pack_bf16(dg, du);
              ys[i] = y1 * score;
            }
            reinterpret_cast<uint4*>(dz_dst)[2 * j] = make_uint4(dzw[0], dzw[1], dzw[2], dzw[3]);
            reinterpret_cast<uint4*>(dz_dst)[2 * j + 1] = make_uint4(dzw[4], dzw[5], dzw[6], dzw[7]);
            reinterpret_cast<uint4*>(ys_dst)[j] = make_uint4(pack_bf16(ys[0], ys[1]), pack_bf16(ys[2], ys[3]),
                                                             pack_bf16(ys[4], ys[5]), pack_bf16(ys[6], ys[7]));
          }
        } else if constexpr (EPI == EPI_SCATTER) {
          float* dst = p.acc_out + static_cast<long long>(p.gather[r]) * p.N + n;
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(dst + 4 * j),
                         "f"(score * __uint_as_float(v[4 * j + 0])), "f"(score * __uint_as_float(v[4 * j + 1])),
                         "f"(score * __uint_as_float(v[4 * j + 2])), "f"(score * __uint_as_float(v[4 * j + 3]))
                         : "memory");
          }
        }
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

// FP8 (E4M3) grouped GEMM with power-of-two block scales applied by the tensor cores themselves:
// tcgen05.mma.kind::mxf8f6f4.block_scale on CTA pairs (M 256 x N 256 x K 32), scale factors in UE8M0
// (one byte = a biased exponent) read from tensor memory.  The hardware takes one scale per row (A) and per
// column (B) for every 32 reduction elements; the layer's coarser blocks -- one activation scale per row and
// 128 reduction elements, one weight scale per 128 x 128 block -- are fed by giving the four MMAs of a
// 128-deep k-block the same scale byte and all 128 columns of a weight block the same byte.  The whole
// reduction accumulates in tensor memory (no per-k-block promotion in registers), so the kernel is the bf16
// pair kernel with 1-byte operands plus a scale-factor pipeline:
//
//   warp 0   TMA producer (A unless gathered, B), 6 stages of 128 rows x 128 bytes per operand and CTA
//   warp 1   MMA issuer (leader CTA): per group of four k-blocks  tcgen05.cp  of the group's scale words from
//            shared to tensor memory, then 16 MMAs whose instruction descriptors select byte kb & 3
//   warp 2   A scale words: row r's four bytes (k-blocks 4g..4g+3) -> shared memory in the layout tcgen05.cp
//            expects (row r at 16 (r % 32) + 4 (r / 32)); follows the row gather
//   warp 3   B scale words, same layout over the 256 columns of the tile
//   warps 4..11  epilogue: drain the 128 x 256 fp32 accumulator into registers (128 per thread), hand tensor
//            memory back to the MMA issuer at once, then run the fused epilogue from registers
//   warps 12..15 row gather with TMA tile::gather4
//
// Tensor memory: columns 0..255 accumulator, 256.. four sets of scale factors (4 columns A + 8 columns B each).
// Ragged-M only; every wait is bounded.
#pragma once
#include <cuda_fp8.h>

#include "gemm_fp8.cuh"

namespace smoe {
namespace mx8 {

using fp8::A_STAGE_BYTES;
using fp8::B_STAGE_BYTES;
using fp8::BK;
using fp8::BM;
using fp8::BN;
using fp8::BN_CTA;
using fp8::FIRST_GATHER_WARP;
using fp8::MAX_EXPERTS;
using fp8::STAGES;
using fp8::THREADS;
using fp8::Tile;
using fp8::UMMA_K;

constexpr int FIRST_EPI_WARP = 4;
constexpr int EPI_WARPS = 8;
constexpr int KB_PER_GROUP = 4;          // k-blocks whose scale bytes share one 32-bit word
constexpr int SFA_BYTES = 512;           // 128 rows x 4 bytes
constexpr int SFB_BYTES = 1024;          // 256 columns x 4 bytes
constexpr int SF_SET_BYTES = SFA_BYTES + SFB_BYTES;
constexpr int SF_SETS = 4;             // groups the scale-factor warps may run ahead of the MMA issuer
constexpr uint32_t TMEM_COLS = 512;
constexpr uint32_t TMEM_SF_COL = 256;    // first scale-factor column
constexpr uint32_t TMEM_SF_SET_COLS = 32;
constexpr uint32_t TMEM_SFB_OFFSET = 16;

struct ScaleBytes {
  const uint32_t* a;     // (rows of the A source, a_ld) words: byte j of word g = UE8M0 scale of k-block 4g + j
  long long a_ld;        // words per row = ceil(K / 128 / 4)
  const uint8_t* b;      // per expert, per 128-wide n-block, per k-block: one byte
  long long b_expert_stride, b_n_stride, b_k_stride;
};

struct SharedStorage {
  uint64_t full[STAGES];
  uint64_t empty[STAGES];
  uint64_t sf_full[SF_SETS];
  uint64_t sf_empty[SF_SETS];
  uint64_t acc_full;
  uint64_t acc_empty;
  uint32_t tmem_base;
  int abort_flag;
  float row_amax[2][BM];  // EPI_SWIGLU with quantised y1: the two column halves of a row exchange their max |y1|
  int m_tile_prefix[MAX_EXPERTS + 1];
};

// Output staging: 32 rows x 80 bytes per epilogue warp, so that bf16 outputs leave as 64-byte row segments (8 rows
// per store instruction) instead of one row per lane (see warp_store_rows64 in epilogue.cuh).
constexpr int STAGE_OUT_PITCH = 80;
constexpr int STAGE_OUT_BYTES = EPI_WARPS * 32 * STAGE_OUT_PITCH;  // 20 KiB
constexpr int SMEM_BYTES = 1024 + STAGES * (A_STAGE_BYTES + B_STAGE_BYTES) + SF_SETS * SF_SET_BYTES +
                           ((sizeof(SharedStorage) + 15) & ~15) + STAGE_OUT_BYTES;
static_assert(SMEM_BYTES <= 227 * 1024, "shared memory per CTA");

// Instruction descriptor of the block-scaled kinds: no accumulator-format field (always fp32); scale-factor
// byte selectors for B (bits 4-5) and A (bits 29-30); bit 23 = scale factors are UE8M0.
__host__ __device__ constexpr uint32_t make_idesc_mx(int M, int N, bool b_mn_major, uint32_t sf_id) {
  return (sf_id << 4) | (0u << 7) | (0u << 10)                // A, B: E4M3
         | (0u << 15) | (static_cast<uint32_t>(b_mn_major) << 16)
         | (static_cast<uint32_t>(N >> 3) << 17) | (1u << 23) | (static_cast<uint32_t>(M >> 4) << 24)
         | (sf_id << 29);
}

__device__ __forceinline__ void umma_mx_pair(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                             uint32_t tmem_sfa, uint32_t tmem_sfb, uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %6, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::mxf8f6f4.block_scale [%0], %1, %2, %3, [%4], [%5], p;\n\t"
      "}\n"
      ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(tmem_sfa), "r"(tmem_sfb), "r"(accumulate)
      : "memory");
}

// 32 rows x 16 bytes of shared memory -> 4 columns of tensor memory, the same 32 rows repeated in all four
// lane quadrants; executed in both CTAs of the pair, each from its own shared memory.
__device__ __forceinline__ void tmem_cp_sf_pair(uint32_t taddr, uint64_t sdesc) {
  asm volatile("tcgen05.cp.cta_group::2.32x128b.warpx4 [%0], %1;" ::"r"(taddr), "l"(sdesc) : "memory");
}

// Unswizzled K-major descriptor for the scale-factor words: 8-row groups of 16-byte rows, 128 bytes apart.
__device__ __forceinline__ uint64_t make_sf_desc(uint32_t saddr) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((saddr >> 4) & 0x3FFFu);
  d |= static_cast<uint64_t>((128u >> 4) & 0x3FFFu) << 32;
  d |= 1ull << 46;
  return d;
}

template <bool A_GATHER, bool B_MN, int EPI>
__global__ void __launch_bounds__(THREADS, 1)
grouped_gemm_mxfp8_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                          const GemmParams p, const ScaleBytes sc) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sA = smem;
  uint8_t* sB = smem + STAGES * A_STAGE_BYTES;
  uint8_t* sSF = smem + STAGES * (A_STAGE_BYTES + B_STAGE_BYTES);
  SharedStorage& ss = *reinterpret_cast<SharedStorage*>(sSF + SF_SETS * SF_SET_BYTES);
  uint8_t* stage_out = reinterpret_cast<uint8_t*>(&ss) + ((sizeof(SharedStorage) + 15) & ~15);

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
    for (int s = 0; s < SF_SETS; ++s) {
      mbar_init(smem_u32(&ss.sf_full[s]), 4);   // two producer warps in each CTA
      mbar_init(smem_u32(&ss.sf_empty[s]), 1);
    }
    mbar_init(smem_u32(&ss.acc_full), 1);
    mbar_init(smem_u32(&ss.acc_empty), 2 * EPI_WARPS);
    ss.abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == 0 && lane == 0) {
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(&ss.tmem_base), TMEM_COLS);
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

  if (warp < FIRST_EPI_WARP) {
    fp8::reg_dec<56>();
    // ---- TMA producer ------------------------------------------------------------------------
    if (warp == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      Tile tile;
      for (long long t = first_tile; ok && fp8::decode_tile(p, ss, t, num_n, rank, tile); t += tile_step) {
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
      constexpr uint32_t b_lbo = B_MN ? B_STAGE_BYTES : 16;
      constexpr uint32_t b_kstep = B_MN ? (UMMA_K * 128) : UMMA_K;  // bytes per 32 reduction elements
      int stage = 0;
      uint32_t phase = 0;
      int set = 0;
      uint32_t set_phase = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      // the issuer only needs the number of work units and of k-blocks (a constant): no per-tile decode on its path
      const long long total_units = static_cast<long long>(ss.m_tile_prefix[p.E]) * num_n;
      const int num_kb = p.K / BK;
      for (long long t = first_tile; ok && t < total_units; t += tile_step) {
        // the epilogue warps of both CTAs have copied the previous tile out of tensor memory
        if (!mbar_wait(smem_u32(&ss.acc_empty), acc_phase ^ 1u, abort_flag)) { ok = false; break; }
        acc_phase ^= 1u;
        uint32_t tsfa = 0, tsfb = 0;
        for (int kb = 0; kb < num_kb; ++kb) {
          if ((kb & (KB_PER_GROUP - 1)) == 0) {
            if (!mbar_wait(smem_u32(&ss.sf_full[set]), set_phase, abort_flag)) { ok = false; break; }
            tc_fence_after();
            tsfa = tmem_base + TMEM_SF_COL + set * TMEM_SF_SET_COLS;
            tsfb = tsfa + TMEM_SFB_OFFSET;
            if (lane == 0) {
              const uint32_t s_sf = smem_u32(sSF + set * SF_SET_BYTES);
              tmem_cp_sf_pair(tsfa, make_sf_desc(s_sf));
              tmem_cp_sf_pair(tsfb, make_sf_desc(s_sf + SFA_BYTES));
              tmem_cp_sf_pair(tsfb + 4, make_sf_desc(s_sf + SFA_BYTES + 512));
              umma_commit_pair(smem_u32(&ss.sf_empty[set]), 3);  // the words have left shared memory
            }
            __syncwarp();
            if (++set == SF_SETS) { set = 0; set_phase ^= 1u; }
          }
          if (!mbar_wait(smem_u32(&ss.full[stage]), phase, abort_flag)) { ok = false; break; }
          tc_fence_after();
          if (lane == 0) {
            const uint32_t idesc = make_idesc_mx(2 * BM, BN, B_MN, static_cast<uint32_t>(kb & (KB_PER_GROUP - 1)));
            const uint64_t a_desc = make_smem_desc(smem_u32(sA + stage * A_STAGE_BYTES), 16, 1024);
            const uint64_t b_desc = make_smem_desc(smem_u32(sB + stage * B_STAGE_BYTES), b_lbo, 1024);
#pragma unroll
            for (int k4 = 0; k4 < BK / UMMA_K; ++k4)
              umma_mx_pair(tmem_base, a_desc + ((k4 * UMMA_K) >> 4), b_desc + ((k4 * b_kstep) >> 4), idesc, tsfa,
                           tsfb, (kb > 0 || k4 > 0) ? 1u : 0u);
            umma_commit_pair(smem_u32(&ss.empty[stage]), 3);
            if (kb == num_kb - 1) umma_commit_pair(smem_u32(&ss.acc_full), 3);
          }
          __syncwarp();
          if (++stage == STAGES) { stage = 0; phase ^= 1u; }
        }
      }
      if (!ok && lane == 0 && p.status) atomicCAS(p.status, ST_OK, ST_TIMEOUT_MMA);
    }
    // ---- scale-factor words of A (warp 2) and B (warp 3) ----------------------------------------
    else if (warp >= 2) {
      int set = 0;
      uint32_t set_phase = 0;
      bool ok = true;
      Tile tile;
      for (long long t = first_tile; ok && fp8::decode_tile(p, ss, t, num_n, rank, tile); t += tile_step) {
        const int groups = (tile.num_kb + KB_PER_GROUP - 1) / KB_PER_GROUP;
        const uint32_t* a_src[4];
        const uint8_t* b_src[2];
        if (warp == 2) {
#pragma unroll
          for (int j = 0; j < 4; ++j) {  // lane owns rows lane, lane + 32, lane + 64, lane + 96 of the CTA's 128
            const int r = tile.row0 + lane + 32 * j;
            a_src[j] = nullptr;
            if (r < tile.row_end) a_src[j] = sc.a + static_cast<long long>(A_GATHER ? p.gather[r] : r) * sc.a_ld;
          }
        } else {
          const int nblocks = (p.N + 127) / 128;
#pragma unroll
          for (int h = 0; h < 2; ++h)
            b_src[h] = sc.b + tile.e * sc.b_expert_stride +
                       static_cast<long long>(min(tile.n0 / 128 + h, nblocks - 1)) * sc.b_n_stride;
        }
        // words of group g: A rows (warp 2) or the tile's two weight blocks (warp 3); loaded one group ahead
        auto load_words = [&](int g, uint4& w0, uint4& w1) {
          if (warp == 2) {
            // 0x7F = 2^0: rows past the expert's end are computed and never stored
            w0.x = a_src[0] ? a_src[0][g] : 0x7F7F7F7Fu;
            w0.y = a_src[1] ? a_src[1][g] : 0x7F7F7F7Fu;
            w0.z = a_src[2] ? a_src[2][g] : 0x7F7F7F7Fu;
            w0.w = a_src[3] ? a_src[3][g] : 0x7F7F7F7Fu;
          } else {
            uint32_t w[2];
#pragma unroll
            for (int h = 0; h < 2; ++h) {
              w[h] = 0u;
#pragma unroll
              for (int j = 0; j < KB_PER_GROUP; ++j) {
                const int kb = g * KB_PER_GROUP + j;
                const uint32_t byte = kb < tile.num_kb ? b_src[h][kb * sc.b_k_stride] : 0x7Fu;
                w[h] |= byte << (8 * j);
              }
            }
            w0 = make_uint4(w[0], w[0], w[0], w[0]);
            w1 = make_uint4(w[1], w[1], w[1], w[1]);
          }
        };
        uint4 w0, w1 = make_uint4(0, 0, 0, 0);
        load_words(0, w0, w1);
        for (int g = 0; g < groups; ++g) {
          uint4 n0 = w0, n1 = w1;
          if (g + 1 < groups) load_words(g + 1, n0, n1);
          if (!mbar_wait(smem_u32(&ss.sf_empty[set]), set_phase ^ 1u, abort_flag)) { ok = false; break; }
          uint8_t* dst = sSF + set * SF_SET_BYTES;
          if (warp == 2) {
            reinterpret_cast<uint4*>(dst)[lane] = w0;
          } else {
            reinterpret_cast<uint4*>(dst + SFA_BYTES)[lane] = w0;        // columns 0..127 of the tile
            reinterpret_cast<uint4*>(dst + SFA_BYTES + 512)[lane] = w1;  // columns 128..255
          }
          // the words are in shared memory (and visible to the tensor cores' proxy) long before the arrive,
          // which crosses to the leader CTA, lets the MMA warp issue the copy
          fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0) mbar_arrive_cluster_relaxed(map_to_cta(smem_u32(&ss.sf_full[set]), 0));
          if (++set == SF_SETS) { set = 0; set_phase ^= 1u; }
          w0 = n0;
          w1 = n1;
        }
      }
      if (!ok && lane == 0 && p.status) atomicCAS(p.status, ST_OK, ST_TIMEOUT_PRODUCER);
    }
  } else if (warp >= FIRST_GATHER_WARP) {
    fp8::reg_dec<56>();
    // ---- row gather with TMA gather4: 8 issuing threads per warp, 4 rows x 128 B each ----------
    if constexpr (A_GATHER) {
      const int gt = threadIdx.x - 32 * FIRST_GATHER_WARP;  // 0..127
      const bool issuer = (gt & 3) == 0;
      const int j = gt >> 2;  // 0..31
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      Tile tile;
      for (long long t = first_tile; ok && fp8::decode_tile(p, ss, t, num_n, rank, tile); t += tile_step) {
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
    fp8::reg_inc<200>();
    // ---- epilogue ---------------------------------------------------------------------------------
    const int quad = warp & 3;
    const int col_half = (warp - FIRST_EPI_WARP) >> 2;
    const int row_in_tile = quad * 32 + lane;
    const uint32_t my_stage = smem_u32(stage_out) + (warp - FIRST_EPI_WARP) * (32 * STAGE_OUT_PITCH);
    uint32_t acc_phase = 0;
    bool ok = true;
    Tile tile;
    for (long long t = first_tile; ok && fp8::decode_tile(p, ss, t, num_n, rank, tile); t += tile_step) {
      const int r = tile.row0 + row_in_tile;
      const bool row_ok = r < tile.row_end;
      const int ncol0 = tile.n0 + col_half * 128;
      const bool cols_ok = ncol0 < p.N;
      float score = 0.f;
      if constexpr (EPI == EPI_DSWIGLU || EPI == EPI_SCATTER || EPI == EPI_STORE_ROWS) {
        if (row_ok && (EPI != EPI_STORE_ROWS || p.scores != nullptr))
          score = load_score(p.scores, p.scores_are_bf16, p.s_scatter[r]);
      }
      if (!mbar_wait(smem_u32(&ss.acc_full), acc_phase, abort_flag)) { ok = false; break; }
      acc_phase ^= 1u;
      tc_fence_after();
      const uint32_t t_addr = tmem_base + col_half * 128 + (static_cast<uint32_t>(quad * 32) << 16);
      uint32_t v0[32], v1[32], v2[32], v3[32];
      tmem_ld32(t_addr, v0);
      tmem_ld32(t_addr + 32, v1);
      tmem_ld32(t_addr + 64, v2);
      tmem_ld32(t_addr + 96, v3);
      tmem_ld_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster_relaxed(map_to_cta(smem_u32(&ss.acc_empty), 0));
      float ds_acc = 0.f;
      bool done = false;
      if constexpr (EPI == EPI_DSWIGLU) {
        if (p.q_out != nullptr) {
          // dz also leaves quantised: this thread's 128 accumulator columns are 256 columns of dz = two scale blocks
          // of its row, so amax, scale and conversion are thread-local (same arithmetic as the row quantiser on the
          // bf16 dz: bit-identical bytes)
          done = true;
          if (cols_ok) {  // warp-uniform; rows past the expert's end read zeros and store nothing
            auto quantise_block = [&](uint32_t (&a)[32], uint32_t (&b)[32], int n) {
              float amax = 0.f;
              dswiglu_chunk_staged<true, STAGE_OUT_PITCH>(p, my_stage, lane, r - lane, tile.row_end, n, a, score, ds_acc,
                                                          amax);
              dswiglu_chunk_staged<true, STAGE_OUT_PITCH>(p, my_stage, lane, r - lane, tile.row_end, n + 32, b, score,
                                                          ds_acc, amax);
              if (!row_ok) return;
              float inv;
              const uint8_t byte = fp8::pow2_scale(amax, inv);
              uint8_t* dst = p.q_out + static_cast<long long>(r) * (2ll * p.N) + 2 * n;
              auto cvt4 = [&](uint32_t w0, uint32_t w1) {  // two packed bf16 pairs -> four E4M3 bytes
                const uint32_t lo = __nv_cvt_float2_to_fp8x2(
                    make_float2(__uint_as_float(w0 << 16) * inv, __uint_as_float(w0 & 0xFFFF0000u) * inv),
                    __NV_SATFINITE, __NV_E4M3);
                const uint32_t hi = __nv_cvt_float2_to_fp8x2(
                    make_float2(__uint_as_float(w1 << 16) * inv, __uint_as_float(w1 & 0xFFFF0000u) * inv),
                    __NV_SATFINITE, __NV_E4M3);
                return lo | (hi << 16);
              };
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                reinterpret_cast<uint4*>(dst)[j] = make_uint4(cvt4(a[8 * j], a[8 * j + 1]), cvt4(a[8 * j + 2], a[8 * j + 3]),
                                                              cvt4(a[8 * j + 4], a[8 * j + 5]), cvt4(a[8 * j + 6], a[8 * j + 7]));
                reinterpret_cast<uint4*>(dst + 64)[j] = make_uint4(cvt4(b[8 * j], b[8 * j + 1]), cvt4(b[8 * j + 2], b[8 * j + 3]),
                                                                   cvt4(b[8 * j + 4], b[8 * j + 5]), cvt4(b[8 * j + 6], b[8 * j + 7]));
              }
              p.q_scale[static_cast<long long>(r) * p.q_scale_ld + (2 * n) / 128] = byte;
            };
            quantise_block(v0, v1, ncol0);
            if (ncol0 + 64 < p.N) quantise_block(v2, v3, ncol0 + 64);
          }
        }
      }
      if constexpr (EPI == EPI_SWIGLU) {
        if (p.q_out != nullptr) {
          // y1 leaves quantised.  A scale block of y1 (128 columns) is the tile's whole width of z (256 columns): the
          // two epilogue warps of a lane quadrant each hold half of it for the same rows and exchange their max |y1|
          // through shared memory (a 64-thread named barrier per quadrant; both warps walk the same tiles).
          done = true;
          uint32_t yw[32];  // 64 y1 values of this row as packed bf16 pairs
          float amax = 0.f;
          auto swiglu_keep = [&](uint32_t (&a)[32], int c) {
            const int n = ncol0 + 32 * c;
            if (cols_ok && p.out0 != nullptr) {  // warp-uniform: z leaves as 64-byte row segments
              uint32_t zp[16];
#pragma unroll
              for (int j = 0; j < 16; ++j) zp[j] = pack_bf16(__uint_as_float(a[2 * j]), __uint_as_float(a[2 * j + 1]));
              warp_store_rows64<STAGE_OUT_PITCH>(my_stage, lane, zp, p.out0, p.ld0, r - lane, tile.row_end, n);
            }
#pragma unroll
            for (int j = 0; j < 8; ++j) {  // gate = even column, up = odd column
              const float g0 = __uint_as_float(a[4 * j]), u0 = __uint_as_float(a[4 * j + 1]);
              const float g1 = __uint_as_float(a[4 * j + 2]), u1 = __uint_as_float(a[4 * j + 3]);
              const uint32_t w = pack_bf16(g0 * sigmoid_f(g0) * u0, g1 * sigmoid_f(g1) * u1);
              yw[8 * c + j] = w;
              amax = fmaxf(amax, fmaxf(fabsf(__uint_as_float(w << 16)), fabsf(__uint_as_float(w & 0xFFFF0000u))));
            }
          };
          swiglu_keep(v0, 0);
          swiglu_keep(v1, 1);
          swiglu_keep(v2, 2);
          swiglu_keep(v3, 3);
          ss.row_amax[col_half][row_in_tile] = (row_ok && cols_ok) ? amax : 0.f;
          asm volatile("bar.sync %0, 64;" ::"r"(1 + quad) : "memory");
          amax = fmaxf(amax, ss.row_amax[col_half ^ 1][row_in_tile]);
          asm volatile("bar.sync %0, 64;" ::"r"(1 + quad) : "memory");  // the slots may be rewritten for the next tile
          if (row_ok && cols_ok) {
            float inv;
            const uint8_t byte = fp8::pow2_scale(amax, inv);
            auto cvt4 = [&](uint32_t w0, uint32_t w1) {
              const uint32_t lo = __nv_cvt_float2_to_fp8x2(
                  make_float2(__uint_as_float(w0 << 16) * inv, __uint_as_float(w0 & 0xFFFF0000u) * inv),
                  __NV_SATFINITE, __NV_E4M3);
              const uint32_t hi = __nv_cvt_float2_to_fp8x2(
                  make_float2(__uint_as_float(w1 << 16) * inv, __uint_as_float(w1 & 0xFFFF0000u) * inv),
                  __NV_SATFINITE, __NV_E4M3);
              return lo | (hi << 16);
            };
            uint8_t* dst = p.q_out + static_cast<long long>(r) * (p.N / 2) + (ncol0 >> 1);
#pragma unroll
            for (int j = 0; j < 4; ++j)
              reinterpret_cast<uint4*>(dst)[j] = make_uint4(cvt4(yw[8 * j], yw[8 * j + 1]), cvt4(yw[8 * j + 2], yw[8 * j + 3]),
                                                            cvt4(yw[8 * j + 4], yw[8 * j + 5]), cvt4(yw[8 * j + 6], yw[8 * j + 7]));
            if (col_half == 0) p.q_scale[static_cast<long long>(r) * p.q_scale_ld + tile.n0 / BN] = byte;
          }
        }
      }
      if constexpr (EPI == EPI_DSWIGLU) {
        if (!done && cols_ok) {
          done = true;
          float unused = 0.f;
          dswiglu_chunk_staged<false, STAGE_OUT_PITCH>(p, my_stage, lane, r - lane, tile.row_end, ncol0, v0, score, ds_acc, unused);
          dswiglu_chunk_staged<false, STAGE_OUT_PITCH>(p, my_stage, lane, r - lane, tile.row_end, ncol0 + 32, v1, score, ds_acc, unused);
          if (ncol0 + 64 < p.N) {
            dswiglu_chunk_staged<false, STAGE_OUT_PITCH>(p, my_stage, lane, r - lane, tile.row_end, ncol0 + 64, v2, score, ds_acc, unused);
            dswiglu_chunk_staged<false, STAGE_OUT_PITCH>(p, my_stage, lane, r - lane, tile.row_end, ncol0 + 96, v3, score, ds_acc, unused);
          }
        }
      }
      if constexpr (EPI == EPI_STORE) {
        if (cols_ok) {  // warp-uniform
          done = true;
          auto store32 = [&](uint32_t (&a)[32], int n) {
            uint32_t w[16];
#pragma unroll
            for (int j = 0; j < 16; ++j) w[j] = pack_bf16(__uint_as_float(a[2 * j]), __uint_as_float(a[2 * j + 1]));
            warp_store_rows64<STAGE_OUT_PITCH>(my_stage, lane, w, p.out0, p.ld0, r - lane, tile.row_end, n);
          };
          store32(v0, ncol0);
          store32(v1, ncol0 + 32);
          store32(v2, ncol0 + 64);
          store32(v3, ncol0 + 96);
        }
      }
      if (!done && row_ok && cols_ok) {
        epilogue_chunk<EPI, false>(p, tile.e, r, ncol0, v0, score, ds_acc);
        epilogue_chunk<EPI, false>(p, tile.e, r, ncol0 + 32, v1, score, ds_acc);
        epilogue_chunk<EPI, false>(p, tile.e, r, ncol0 + 64, v2, score, ds_acc);
        epilogue_chunk<EPI, false>(p, tile.e, r, ncol0 + 96, v3, score, ds_acc);
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
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

}  // namespace mx8
}  // namespace smoe

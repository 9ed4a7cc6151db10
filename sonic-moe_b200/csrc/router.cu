// Fused routing front end: router GEMM (tokens x H x E on tcgen05, the accumulator row of a token never leaves the
// SM) -> logits rounded to bf16 and written out -> top-K and softmax over the K winners straight from the
// accumulator row -> per-expert token counts and the column sums of the full softmax (what the load-balancing loss
// needs), all in one pass over x.  The layer otherwise spends a library GEMM, a top-k kernel, a (T, E) fp32
// softmax and its column sum on the same 8 MiB of logits.
//
// One persistent CTA per SM, 128 tokens per tile, N = E (<= 256) accumulator columns:
//   warp 0      TMA producer: x tile 128 x 64 and router-weight tile E x 64 per stage (128-byte swizzle)
//   warp 1      MMA issuer: tcgen05.mma M 128 x N E x K 16 into one of two tensor-memory accumulators
//   warps 2-5   epilogue: thread = token.  Pass 1 over the row: round to bf16, store the logits, keep the K best
//               (value, then lower column) in a sorted register list, running max / sum of exponentials.
//               Pass 2 (the row is read from tensor memory again): probabilities, reduced over the warp's 32 tokens
//               with a 31-shuffle butterfly and added to the warp's running column sums; the 4 warps' and then the
//               CTAs' sums are added up in a fixed order, so the column sums are bit-reproducible.
// The routing decision is taken on the bf16-rounded logits the kernel writes, so it can be checked bit for bit
// against a stable sort of that output.  Every wait is bounded (ptx.cuh).
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <math.h>
#include <stdint.h>

#include <mutex>

#include "../../include/sonicmoe_b200.h"
#include "device_cache.cuh"
#include "ptx.cuh"

namespace smoe {
namespace router {

constexpr int BM = 128;
constexpr int BK = 64;
constexpr int UMMA_K = 16;
constexpr int A_STAGE_BYTES = BM * BK * 2;  // 16 KiB
constexpr int MAX_E = 256;
constexpr int THREADS = 192;
constexpr int MAX_STAGES = 6;

struct Shared {
  uint64_t full[MAX_STAGES];
  uint64_t empty[MAX_STAGES];
  uint64_t acc_full[2];
  uint64_t acc_empty[2];
  uint32_t tmem_base;
  int abort_flag;
  float colsum_warp[4][MAX_E];  // [epilogue warp][column]: each warp's running sums over its tokens of all tiles
  int hist[MAX_E];
};

struct Params {
  int T, H, E, K;
  int stages;
  int acc_cols;  // tensor-memory columns per accumulator (power of two >= E)
  __nv_bfloat16* logits;  // (T, E)
  float* scores;          // (T, K)
  int* indices;           // (T, K)
  float* colsum_partial;  // (grid, E)
  int* hist_partial;      // (grid, E)
  int* status;
};

__device__ __forceinline__ uint32_t order_key(float v) {  // larger key = better; NaN first, -0 == +0
  if (v != v) return 0xFFFFFFFFu;
  v = v + 0.0f;
  const uint32_t b = __float_as_uint(v);
  return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}
__device__ __forceinline__ float key_value(uint32_t k) {
  const uint32_t b = (k & 0x80000000u) ? (k & 0x7FFFFFFFu) : ~k;
  return __uint_as_float(b);
}

template <int KC>
__global__ void __launch_bounds__(THREADS, 1)
router_forward_kernel(const __grid_constant__ CUtensorMap tmX, const __grid_constant__ CUtensorMap tmW, const Params p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const int b_stage_bytes = p.E * BK * 2;
  const int stage_bytes = A_STAGE_BYTES + b_stage_bytes;  // E is a multiple of 32: stages stay 1024-byte aligned
  Shared& ss = *reinterpret_cast<Shared*>(smem + p.stages * stage_bytes);
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  volatile int* abort_flag = &ss.abort_flag;
  const int num_tiles = (p.T + BM - 1) / BM;
  const int num_kb = p.H / BK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < p.stages; ++s) {
      mbar_init(smem_u32(&ss.full[s]), 1);
      mbar_init(smem_u32(&ss.empty[s]), 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(smem_u32(&ss.acc_full[a]), 1);
      mbar_init(smem_u32(&ss.acc_empty[a]), 4);
    }
    ss.abort_flag = 0;
    fence_mbar_init();
    tma_prefetch_desc(&tmX);
    tma_prefetch_desc(&tmW);
  }
  for (int e = threadIdx.x; e < MAX_E; e += THREADS) {
#pragma unroll
    for (int w = 0; w < 4; ++w) ss.colsum_warp[w][e] = 0.f;
    ss.hist[e] = 0;
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(&ss.tmem_base), 2 * p.acc_cols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = ss.tmem_base;

  if (warp == 0) {
    // ---- TMA producer -------------------------------------------------------------------------------------
    int stage = 0;
    uint32_t phase = 0;
    bool ok = true;
    for (int tile = blockIdx.x; ok && tile < num_tiles; tile += gridDim.x) {
      for (int kb = 0; kb < num_kb; ++kb) {
        if (!mbar_wait(smem_u32(&ss.empty[stage]), phase ^ 1u, abort_flag)) { ok = false; break; }
        if (lane == 0) {
          const uint32_t bar = smem_u32(&ss.full[stage]);
          const uint32_t a_dst = smem_u32(smem + stage * stage_bytes);
          mbar_arrive_expect_tx(bar, stage_bytes);
          tma_load_2d(&tmX, bar, a_dst, kb * BK, tile * BM);
          tma_load_2d(&tmW, bar, a_dst + A_STAGE_BYTES, kb * BK, 0);
        }
        __syncwarp();
        if (++stage == p.stages) { stage = 0; phase ^= 1u; }
      }
    }
    if (!ok && lane == 0 && p.status) atomicCAS(p.status, SMOE_ST_OK, SMOE_ST_TIMEOUT_PRODUCER);
  } else if (warp == 1) {
    // ---- MMA issuer ---------------------------------------------------------------------------------------
    const uint32_t idesc = make_idesc_bf16(BM, p.E, false, false);
    int stage = 0;
    uint32_t phase = 0;
    int acc = 0;
    uint32_t acc_phase = 0;
    bool ok = true;
    for (int tile = blockIdx.x; ok && tile < num_tiles; tile += gridDim.x) {
      if (!mbar_wait(smem_u32(&ss.acc_empty[acc]), acc_phase ^ 1u, abort_flag)) { ok = false; break; }
      tc_fence_after();
      const uint32_t d_tmem = tmem_base + acc * p.acc_cols;
      for (int kb = 0; kb < num_kb; ++kb) {
        if (!mbar_wait(smem_u32(&ss.full[stage]), phase, abort_flag)) { ok = false; break; }
        tc_fence_after();
        if (lane == 0) {
          const uint32_t a_addr = smem_u32(smem + stage * stage_bytes);
          const uint64_t a_desc = make_smem_desc(a_addr, 16, 1024);
          const uint64_t b_desc = make_smem_desc(a_addr + A_STAGE_BYTES, 16, 1024);
#pragma unroll
          for (int k4 = 0; k4 < BK / UMMA_K; ++k4)
            umma_bf16(d_tmem, a_desc + ((k4 * UMMA_K * 2) >> 4), b_desc + ((k4 * UMMA_K * 2) >> 4), idesc,
                      (kb > 0 || k4 > 0) ? 1u : 0u);
          umma_commit(smem_u32(&ss.empty[stage]));
        }
        __syncwarp();
        if (++stage == p.stages) { stage = 0; phase ^= 1u; }
      }
      if (!ok) break;
      if (lane == 0) umma_commit(smem_u32(&ss.acc_full[acc]));
      __syncwarp();
      if (++acc == 2) { acc = 0; acc_phase ^= 1u; }
    }
    if (!ok && lane == 0 && p.status) atomicCAS(p.status, SMOE_ST_OK, SMOE_ST_TIMEOUT_MMA);
  } else {
    // ---- epilogue: thread = token -------------------------------------------------------------------------
    const int quad = warp & 3;         // the 32 tensor-memory lanes this warp may read
    const int ew = warp - 2;           // 0..3, slot in colsum_warp
    const int chunks = p.E >> 5;
    int acc = 0;
    uint32_t acc_phase = 0;
    bool ok = true;
    for (int tile = blockIdx.x; ok && tile < num_tiles; tile += gridDim.x) {
      if (!mbar_wait(smem_u32(&ss.acc_full[acc]), acc_phase, abort_flag)) { ok = false; break; }
      tc_fence_after();
      const int row = tile * BM + quad * 32 + lane;
      const bool valid = row < p.T;
      const uint32_t t_addr = tmem_base + acc * p.acc_cols + (static_cast<uint32_t>(quad * 32) << 16);
      uint64_t top[KC];
#pragma unroll
      for (int j = 0; j < KC; ++j) top[j] = 0ull;
      float m = -INFINITY, s = 0.f;
      // pass 1: logits out, top-K list, running max / sum of exponentials
      for (int c = 0; c < chunks; ++c) {
        uint32_t v[32];
        tmem_ld32(t_addr + c * 32, v);
        tmem_ld_wait();
        float f[32];
        uint32_t packed[16];
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          const __nv_bfloat162 h = __floats2bfloat162_rn(__uint_as_float(v[2 * j]), __uint_as_float(v[2 * j + 1]));
          packed[j] = *reinterpret_cast<const uint32_t*>(&h);
          f[2 * j] = __low2float(h);
          f[2 * j + 1] = __high2float(h);
        }
        if (valid) {
          uint4* dst = reinterpret_cast<uint4*>(p.logits + static_cast<long long>(row) * p.E + c * 32);
#pragma unroll
          for (int q = 0; q < 4; ++q)
            dst[q] = make_uint4(packed[4 * q], packed[4 * q + 1], packed[4 * q + 2], packed[4 * q + 3]);
        }
        float cm = f[0];
#pragma unroll
        for (int j = 1; j < 32; ++j) cm = fmaxf(cm, f[j]);
        const float m_new = fmaxf(m, cm);
        float add = 0.f;
#pragma unroll
        for (int j = 0; j < 32; ++j) add += __expf(f[j] - m_new);
        s = s * __expf(m - m_new) + add;
        m = m_new;
#pragma unroll
        for (int j = 0; j < 32; ++j) {
          const uint64_t key = (static_cast<uint64_t>(order_key(f[j])) << 32) | (0xFFFFFFFFu - (c * 32 + j));
          if (key > top[KC - 1]) {
#pragma unroll
            for (int i = KC - 1; i >= 0; --i) {
              const bool gt_prev = (i > 0) && key > top[i > 0 ? i - 1 : 0];
              const bool gt_here = key > top[i];
              top[i] = gt_prev ? top[i > 0 ? i - 1 : 0] : (gt_here ? key : top[i]);
            }
          }
        }
      }
      // scores over the K winners, indices, histogram
      if (valid) {
        const float vmax = key_value(static_cast<uint32_t>(top[0] >> 32));
        float ex[KC];
        float sum = 0.f;
#pragma unroll
        for (int k = 0; k < KC; ++k) {
          ex[k] = (k < p.K) ? expf(key_value(static_cast<uint32_t>(top[k] >> 32)) - vmax) : 0.f;
          sum += ex[k];
        }
#pragma unroll
        for (int k = 0; k < KC; ++k) {
          if (k < p.K) {
            const int col = static_cast<int>(0xFFFFFFFFu - static_cast<uint32_t>(top[k]));
            p.scores[static_cast<long long>(row) * p.K + k] = ex[k] / sum;
            p.indices[static_cast<long long>(row) * p.K + k] = col;
            atomicAdd(&ss.hist[col], 1);
          }
        }
      }
      // pass 2: probabilities of the full softmax, summed over the warp's 32 tokens column by column
      const float inv_s = valid ? 1.f / s : 0.f;
      for (int c = 0; c < chunks; ++c) {
        uint32_t v[32];
        tmem_ld32(t_addr + c * 32, v);
        tmem_ld_wait();
        float q[32];
#pragma unroll
        for (int j = 0; j < 32; ++j)
          q[j] = valid ? __expf(__bfloat162float(__float2bfloat16_rn(__uint_as_float(v[j]))) - m) * inv_s : 0.f;
        // butterfly: after the step with distance d a lane holds d partial columns; lane l ends with column l
#pragma unroll
        for (int d = 16; d > 0; d >>= 1) {
          const bool upper = (lane & d) != 0;
#pragma unroll
          for (int j = 0; j < d; ++j) {
            const float send = upper ? q[j] : q[j + d];
            const float keep = upper ? q[j + d] : q[j];
            q[j] = keep + __shfl_xor_sync(0xffffffffu, send, d);
          }
        }
        ss.colsum_warp[ew][c * 32 + lane] += q[0];  // this lane is the only writer of this word
      }
      // the accumulator is free again
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&ss.acc_empty[acc]));
      if (++acc == 2) { acc = 0; acc_phase ^= 1u; }
    }
    if (!ok && lane == 0 && p.status) atomicCAS(p.status, SMOE_ST_OK, SMOE_ST_TIMEOUT_EPILOGUE);
  }

  if (*abort_flag != 0) {
    const uint64_t t0 = global_timer_ns();
    while (global_timer_ns() - t0 < 200000ull) __nanosleep(1000);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 2 * p.acc_cols);
  }
  // this CTA's partial results: the four warps' column sums in a fixed order, and the token counts
  for (int col = threadIdx.x; col < p.E; col += THREADS) {
    p.colsum_partial[static_cast<long long>(blockIdx.x) * p.E + col] =
        ((ss.colsum_warp[0][col] + ss.colsum_warp[1][col]) + ss.colsum_warp[2][col]) + ss.colsum_warp[3][col];
    p.hist_partial[static_cast<long long>(blockIdx.x) * p.E + col] = ss.hist[col];
  }
}

// count[e] and colsum[e]: the CTAs' partials added up in CTA order.
__global__ void __launch_bounds__(256) router_finish_kernel(const float* __restrict__ colsum_partial,
                                                            const int* __restrict__ hist_partial, int blocks, int E,
                                                            float* __restrict__ colsum, int* __restrict__ count) {
  const int e = threadIdx.x;
  if (e >= E) return;
  float s = 0.f;
  int c = 0;
  for (int b = 0; b < blocks; ++b) {
    s += colsum_partial[static_cast<long long>(b) * E + e];
    c += hist_partial[static_cast<long long>(b) * E + e];
  }
  colsum[e] = s;
  count[e] = c;
}

// dlogits[t, e] = g_logits[t, e]                                      (optional)
//              + s_k (g_k - sum_j g_j s_j) for e = idx[t, k]           (gradient through the K winners' softmax)
//              + p[t, e] (c_e - sum_j p[t, j] c_j)                     (optional: gradient c of the column sums of
//                                                                       the full softmax p of the row)
// One warp per row; the row's probabilities are recomputed from the saved bf16 logits.
template <int PER_LANE>
__global__ void __launch_bounds__(256) router_backward_kernel(__nv_bfloat16* __restrict__ dlogits,
                                                              const __nv_bfloat16* __restrict__ logits,
                                                              const float* __restrict__ dscore,
                                                              const float* __restrict__ score,
                                                              const int* __restrict__ indices,
                                                              const float* __restrict__ g_colsum,
                                                              const __nv_bfloat16* __restrict__ g_logits, int rows,
                                                              int E, int K) {
  const int lane = threadIdx.x & 31;
  const long long row = static_cast<long long>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= rows) return;
  float out[PER_LANE];
#pragma unroll
  for (int j = 0; j < PER_LANE; ++j) {
    const int col = lane + 32 * j;
    out[j] = (g_logits != nullptr && col < E) ? __bfloat162float(g_logits[row * E + col]) : 0.f;
  }
  if (g_colsum != nullptr) {
    float l[PER_LANE];
    float m = -INFINITY;
#pragma unroll
    for (int j = 0; j < PER_LANE; ++j) {
      const int col = lane + 32 * j;
      l[j] = col < E ? __bfloat162float(logits[row * E + col]) : -INFINITY;
      m = fmaxf(m, l[j]);
    }
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, d));
    float s = 0.f, dot = 0.f;
#pragma unroll
    for (int j = 0; j < PER_LANE; ++j) {
      const int col = lane + 32 * j;
      l[j] = col < E ? __expf(l[j] - m) : 0.f;
      s += l[j];
      dot += col < E ? l[j] * g_colsum[col] : 0.f;
    }
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) {
      s += __shfl_xor_sync(0xffffffffu, s, d);
      dot += __shfl_xor_sync(0xffffffffu, dot, d);
    }
    const float inv = 1.f / s;
    dot *= inv;
#pragma unroll
    for (int j = 0; j < PER_LANE; ++j) {
      const int col = lane + 32 * j;
      if (col < E) out[j] += l[j] * inv * (g_colsum[col] - dot);
    }
  }
  if (dscore != nullptr) {
    float dot = 0.f;
    for (int k = lane; k < K; k += 32) dot += dscore[row * K + k] * score[row * K + k];
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, d);
    for (int k = 0; k < K; ++k) {  // every lane walks the K winners; the owner of the column adds the term
      const int col = indices[row * K + k];
      const float term = score[row * K + k] * (dscore[row * K + k] - dot);
#pragma unroll
      for (int j = 0; j < PER_LANE; ++j)
        if (col == lane + 32 * j) out[j] += term;
    }
  }
#pragma unroll
  for (int j = 0; j < PER_LANE; ++j) {
    const int col = lane + 32 * j;
    if (col < E) dlogits[row * E + col] = __float2bfloat16_rn(out[j]);
  }
}

using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(ptr);
  });
  return fn;
}

static int encode_rows(CUtensorMap* map, const void* base, uint64_t rows, uint64_t cols, uint32_t box_rows) {
  EncodeTiledFn fn = encode_fn();
  if (fn == nullptr) return SMOE_ERR_DRIVER;
  static thread_local bool context_bound = false;
  if (!context_bound) {
    if (cudaFree(nullptr) != cudaSuccess) return SMOE_ERR_DRIVER;
    context_bound = true;
  }
  if ((reinterpret_cast<uintptr_t>(base) & 15u) != 0) return SMOE_ERR_ALIGNMENT;
  const cuuint64_t dims[2] = {cols, rows};
  const cuuint64_t strides[1] = {cols * 2};
  const cuuint32_t box[2] = {BK, box_rows};
  const cuuint32_t estr[2] = {1, 1};
  const CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? SMOE_OK : SMOE_ERR_TENSORMAP;
}

static bool unsupported(int T, int H, int E, int K) {
  return T < 0 || H <= 0 || (H % BK) != 0 || E < 32 || E > MAX_E || (E % 32) != 0 || K <= 0 || K > 16 || K > E;
}

}  // namespace router
}  // namespace smoe

using namespace smoe;
using namespace smoe::router;

extern "C" {

int smoe_router_forward_supported(int H, int E, int K) { return unsupported(1, H, E, K) ? 0 : 1; }

size_t smoe_router_forward_workspace_bytes(int E) {
  const int sms = num_sms();
  return static_cast<size_t>(sms > 0 ? sms : 256) * static_cast<size_t>(E > 0 ? E : 1) * 8;
}

int smoe_router_forward(const void* x, const void* router_w, void* logits, float* scores, int* indices,
                        int* expert_count, float* prob_colsum, void* workspace, int T, int H, int E, int K,
                        int* status, void* stream) {
  if (unsupported(T, H, E, K)) return SMOE_ERR_SHAPE;
  if (workspace == nullptr) return SMOE_ERR_WORKSPACE;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int sms = num_sms();
  if (sms <= 0) return SMOE_ERR_DRIVER;
  const int tiles = (T + BM - 1) / BM;
  const int grid = tiles < sms ? tiles : sms;
  float* colsum_partial = static_cast<float*>(workspace);
  int* hist_partial = reinterpret_cast<int*>(colsum_partial + static_cast<size_t>(sms) * E);
  if (T > 0) {
    CUtensorMap tmX, tmW;
    int rc = encode_rows(&tmX, x, T, H, BM);
    if (rc != SMOE_OK) return rc;
    rc = encode_rows(&tmW, router_w, E, H, E);
    if (rc != SMOE_OK) return rc;
    Params p = {};
    p.T = T; p.H = H; p.E = E; p.K = K;
    p.stages = E <= 128 ? 6 : 4;
    p.acc_cols = E <= 32 ? 32 : E <= 64 ? 64 : E <= 128 ? 128 : 256;
    p.logits = static_cast<__nv_bfloat16*>(logits);
    p.scores = scores; p.indices = indices;
    p.colsum_partial = colsum_partial; p.hist_partial = hist_partial;
    p.status = status;
    const int smem = 1024 + p.stages * (A_STAGE_BYTES + E * BK * 2) + static_cast<int>(sizeof(Shared));
    const int dev = current_device();
    if (dev < 0) return SMOE_ERR_DRIVER;
    static PerDeviceFlag configured8, configured16;
    if (K <= 8) {
      if (!configured8.test(dev)) {
        if (cudaFuncSetAttribute(router_forward_kernel<8>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024) !=
            cudaSuccess)
          return SMOE_ERR_LAUNCH;
        configured8.set(dev);
      }
      router_forward_kernel<8><<<grid, THREADS, smem, st>>>(tmX, tmW, p);
    } else {
      if (!configured16.test(dev)) {
        if (cudaFuncSetAttribute(router_forward_kernel<16>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024) !=
            cudaSuccess)
          return SMOE_ERR_LAUNCH;
        configured16.set(dev);
      }
      router_forward_kernel<16><<<grid, THREADS, smem, st>>>(tmX, tmW, p);
    }
    if (cudaGetLastError() != cudaSuccess) return SMOE_ERR_LAUNCH;
  }
  router_finish_kernel<<<1, 256, 0, st>>>(colsum_partial, hist_partial, T > 0 ? grid : 0, E, prob_colsum, expert_count);
  return cudaGetLastError() == cudaSuccess ? SMOE_OK : SMOE_ERR_LAUNCH;
}

int smoe_router_backward(void* dlogits, const void* logits, const float* dscores, const float* scores,
                         const int* indices, const float* g_colsum, const void* g_logits, int T, int E, int K,
                         void* stream) {
  if (T < 0 || E <= 0 || E > MAX_E || K <= 0 || K > E) return SMOE_ERR_SHAPE;
  if (dscores != nullptr && (scores == nullptr || indices == nullptr)) return SMOE_ERR_SHAPE;
  if (g_colsum != nullptr && logits == nullptr) return SMOE_ERR_SHAPE;
  if (T == 0) return SMOE_OK;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const unsigned grid = (T + 7) / 8;
  __nv_bfloat16* d = static_cast<__nv_bfloat16*>(dlogits);
  const __nv_bfloat16* l = static_cast<const __nv_bfloat16*>(logits);
  const __nv_bfloat16* g = static_cast<const __nv_bfloat16*>(g_logits);
  const int per_lane = (E + 31) / 32;
  if (per_lane <= 2)
    router_backward_kernel<2><<<grid, 256, 0, st>>>(d, l, dscores, scores, indices, g_colsum, g, T, E, K);
  else if (per_lane <= 4)
    router_backward_kernel<4><<<grid, 256, 0, st>>>(d, l, dscores, scores, indices, g_colsum, g, T, E, K);
  else
    router_backward_kernel<8><<<grid, 256, 0, st>>>(d, l, dscores, scores, indices, g_colsum, g, T, E, K);
  return cudaGetLastError() == cudaSuccess ? SMOE_OK : SMOE_ERR_LAUNCH;
}

}  // extern "C"

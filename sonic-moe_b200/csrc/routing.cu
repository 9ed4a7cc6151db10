// Routing-side kernels of the MoE layer: top-k + softmax, its backward, the expert histogram and
// prefix sum, the stable counting sort that builds the grouped-row index vectors, and the
// gather-and-sum over each token's routed rows.  All of them are HBM- or latency-bound integer /
// elementwise work: coalesced 16-byte accesses, warp shuffles, shared-memory histograms.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <math.h>
#include <stdint.h>

#include <mutex>

#include "../../include/sonicmoe_b200.h"
#include "device_cache.cuh"

namespace smoe {

constexpr int kSortThreads = 256;
constexpr int kSortWarps = kSortThreads / 32;
constexpr int kMaxSortBlocks = 128;       // chunks the flat index vector is cut into
constexpr int kMaxSmemExperts = 4096;     // histogram bins kept in shared memory

static inline cudaStream_t S(void* s) { return static_cast<cudaStream_t>(s); }
static inline int launch_rc() { return cudaGetLastError() == cudaSuccess ? SMOE_OK : SMOE_ERR_LAUNCH; }

// ----------------------------------------------------------------------------------------------
// top-k + softmax over the K winners
// ----------------------------------------------------------------------------------------------
// Order: larger value first; equal values: lower column first (-0.0 == +0.0, NaN sorts first).
__device__ __forceinline__ uint32_t order_key(float v) {
  if (v != v) return 0xFFFFFFFFu;
  v = v + 0.0f;  // -0.0 -> +0.0
  const uint32_t b = __float_as_uint(v);
  return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}

__device__ __forceinline__ float key_value(uint32_t k) {
  const uint32_t b = (k & 0x80000000u) ? (k & 0x7FFFFFFFu) : ~k;
  return __uint_as_float(b);
}

template <typename T>
__device__ __forceinline__ float to_f32(T v);
template <>
__device__ __forceinline__ float to_f32<float>(float v) { return v; }
template <>
__device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

// One warp per row; lane l keeps columns l, l+32, ... in registers (PER_LANE of them).
template <typename T, int PER_LANE>
__global__ void __launch_bounds__(256) topk_softmax_kernel(const T* __restrict__ logits, float* __restrict__ scores,
                                                           int* __restrict__ indices, int rows, int E, int K) {
  const int lane = threadIdx.x & 31;
  const long long row = static_cast<long long>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= rows) return;
  const T* src = logits + row * E;
  uint64_t key[PER_LANE];
#pragma unroll
  for (int j = 0; j < PER_LANE; ++j) {
    const int col = lane + 32 * j;
    key[j] = 0ull;  // below every real key (real keys have a non-zero low half or high half)
    if (col < E) key[j] = (static_cast<uint64_t>(order_key(to_f32(src[col]))) << 32) | (0xFFFFFFFFu - col);
  }
  uint64_t mine = 0ull;  // lane j keeps the j-th winner
  for (int k = 0; k < K; ++k) {
    uint64_t best = key[0];
#pragma unroll
    for (int j = 1; j < PER_LANE; ++j) best = key[j] > best ? key[j] : best;
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) {
      const uint64_t o = __shfl_xor_sync(0xffffffffu, best, d);
      best = o > best ? o : best;
    }
#pragma unroll
    for (int j = 0; j < PER_LANE; ++j)
      if (key[j] == best) key[j] = 0ull;  // keys are unique (they embed the column)
    if (lane == k) mine = best;
  }
  const bool active = lane < K;
  const float v = active ? key_value(static_cast<uint32_t>(mine >> 32)) : 0.f;
  const int col = active ? static_cast<int>(0xFFFFFFFFu - static_cast<uint32_t>(mine)) : 0;
  const float vmax = __shfl_sync(0xffffffffu, v, 0);
  float ex = active ? expf(v - vmax) : 0.f;
  float sum = ex;
#pragma unroll
  for (int d = 16; d > 0; d >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, d);
  if (active) {
    scores[row * K + lane] = ex / sum;
    indices[row * K + lane] = col;
  }
}

// Any E: K passes over the row, each finding the best key below the previous winner.
template <typename T>
__global__ void __launch_bounds__(256) topk_softmax_generic_kernel(const T* __restrict__ logits,
                                                                   float* __restrict__ scores,
                                                                   int* __restrict__ indices, int rows, int E,
                                                                   int K) {
  const int lane = threadIdx.x & 31;
  const long long row = static_cast<long long>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= rows) return;
  const T* src = logits + row * E;
  uint64_t prev = ~0ull;
  float vmax = 0.f, sum = 0.f;
  for (int k = 0; k < K; ++k) {
    uint64_t best = 0ull;
    for (int col = lane; col < E; col += 32) {
      const uint64_t kk = (static_cast<uint64_t>(order_key(to_f32(src[col]))) << 32) | (0xFFFFFFFFu - col);
      if (kk < prev && kk > best) best = kk;
    }
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) {
      const uint64_t o = __shfl_xor_sync(0xffffffffu, best, d);
      best = o > best ? o : best;
    }
    prev = best;
    const float v = key_value(static_cast<uint32_t>(best >> 32));
    if (k == 0) vmax = v;
    const float ex = expf(v - vmax);
    sum += ex;
    if (lane == 0) {
      scores[row * K + k] = ex;  // normalised below
      indices[row * K + k] = static_cast<int>(0xFFFFFFFFu - static_cast<uint32_t>(best));
    }
  }
  __syncwarp();
  if (lane == 0)
    for (int k = 0; k < K; ++k) scores[row * K + k] = scores[row * K + k] / sum;
}

template <typename T>
static int launch_topk(const void* logits, float* scores, int* indices, int rows, int E, int K, cudaStream_t st) {
  const T* src = static_cast<const T*>(logits);
  const int warps = 8;
  const unsigned grid = (rows + warps - 1) / warps;
  const int per_lane = (E + 31) / 32;
  if (K > 32) {
    topk_softmax_generic_kernel<T><<<grid, warps * 32, 0, st>>>(src, scores, indices, rows, E, K);
  } else if (per_lane <= 1) {
    topk_softmax_kernel<T, 1><<<grid, warps * 32, 0, st>>>(src, scores, indices, rows, E, K);
  } else if (per_lane <= 2) {
    topk_softmax_kernel<T, 2><<<grid, warps * 32, 0, st>>>(src, scores, indices, rows, E, K);
  } else if (per_lane <= 4) {
    topk_softmax_kernel<T, 4><<<grid, warps * 32, 0, st>>>(src, scores, indices, rows, E, K);
  } else if (per_lane <= 8) {
    topk_softmax_kernel<T, 8><<<grid, warps * 32, 0, st>>>(src, scores, indices, rows, E, K);
  } else if (per_lane <= 16) {
    topk_softmax_kernel<T, 16><<<grid, warps * 32, 0, st>>>(src, scores, indices, rows, E, K);
  } else if (per_lane <= 32) {
    topk_softmax_kernel<T, 32><<<grid, warps * 32, 0, st>>>(src, scores, indices, rows, E, K);
  } else {
    topk_softmax_generic_kernel<T><<<grid, warps * 32, 0, st>>>(src, scores, indices, rows, E, K);
  }
  return launch_rc();
}

// dlogits[t, idx[t,k]] = s_k * (g_k - sum_j g_j s_j); every other column of the row is written as zero.
template <typename T>
__global__ void __launch_bounds__(256) softmax_topk_bwd_kernel(T* __restrict__ dlogits,
                                                               const float* __restrict__ dscore,
                                                               const float* __restrict__ score,
                                                               const int* __restrict__ indices, int rows, int E,
                                                               int K) {
  const int lane = threadIdx.x & 31;
  const long long row = static_cast<long long>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= rows) return;
  T* dst = dlogits + row * E;
  for (int col = lane; col < E; col += 32) dst[col] = static_cast<T>(0.f);
  float dot = 0.f;
  for (int k = lane; k < K; k += 32) dot += dscore[row * K + k] * score[row * K + k];
#pragma unroll
  for (int d = 16; d > 0; d >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, d);
  __syncwarp();
  for (int k = lane; k < K; k += 32) {
    const float s = score[row * K + k];
    dst[indices[row * K + k]] = static_cast<T>(s * (dscore[row * K + k] - dot));
  }
}

// ----------------------------------------------------------------------------------------------
// histogram + prefix sum
// ----------------------------------------------------------------------------------------------
template <typename IdxT>
__global__ void __launch_bounds__(kSortThreads) chunk_histogram_kernel(const IdxT* __restrict__ idx, long long n,
                                                                       int E, int* __restrict__ block_hist) {
  extern __shared__ int hist[];
  for (int e = threadIdx.x; e < E; e += blockDim.x) hist[e] = 0;
  __syncthreads();
  const long long chunk = (n + gridDim.x - 1) / gridDim.x;
  const long long begin = chunk * blockIdx.x;
  const long long end = begin + chunk < n ? begin + chunk : n;
  for (long long p = begin + threadIdx.x; p < end; p += blockDim.x) {
    const long long e = static_cast<long long>(idx[p]);
    if (e >= 0 && e < E) atomicAdd(&hist[e], 1);
  }
  __syncthreads();
  for (int e = threadIdx.x; e < E; e += blockDim.x) block_hist[static_cast<long long>(blockIdx.x) * E + e] = hist[e];
}

// Large E (bins do not fit in shared memory): global atomics into a zeroed count vector.
template <typename IdxT>
__global__ void __launch_bounds__(256) global_histogram_kernel(const IdxT* __restrict__ idx, long long n, int E,
                                                               int* __restrict__ count) {
  for (long long p = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; p < n;
       p += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long e = static_cast<long long>(idx[p]);
    if (e >= 0 && e < E) atomicAdd(&count[e], 1);
  }
}

// One CTA.  For every bin: turn the per-chunk counts into exclusive per-chunk bases (in place) and
// produce the bin total; then an inclusive scan over the bins.
//   count[e]   = total of bin e               (optional)
//   cumsum[e]  = count[0] + ... + count[e]    (optional)
//   offset[e]  = exclusive scan, E+1 entries  (optional)
__global__ void __launch_bounds__(1024) scan_bins_kernel(int* __restrict__ block_hist, int num_blocks, int E,
                                                         const int* __restrict__ count_in, int* __restrict__ count,
                                                         int* __restrict__ cumsum, int* __restrict__ offset) {
  __shared__ int warp_sums[32];
  __shared__ int carry;
  if (threadIdx.x == 0) carry = 0;
  if (offset != nullptr && threadIdx.x == 0) offset[0] = 0;
  __syncthreads();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  for (int base = 0; base < E; base += blockDim.x) {
    const int e = base + threadIdx.x;
    int total = 0;
    if (e < E) {
      if (block_hist != nullptr) {
        for (int b = 0; b < num_blocks; ++b) {
          const int c = block_hist[static_cast<long long>(b) * E + e];
          block_hist[static_cast<long long>(b) * E + e] = total;
          total += c;
        }
      } else {
        total = count_in[e];
      }
      if (count != nullptr) count[e] = total;
    }
    int incl = total;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
      const int o = __shfl_up_sync(0xffffffffu, incl, d);
      if (lane >= d) incl += o;
    }
    if (lane == 31) warp_sums[warp] = incl;
    __syncthreads();
    if (warp == 0) {
      int w = warp_sums[lane];
#pragma unroll
      for (int d = 1; d < 32; d <<= 1) {
        const int o = __shfl_up_sync(0xffffffffu, w, d);
        if (lane >= d) w += o;
      }
      warp_sums[lane] = w;  // inclusive over warps
    }
    __syncthreads();
    const int before = carry + (warp > 0 ? warp_sums[warp - 1] : 0);
    if (e < E) {
      if (cumsum != nullptr) cumsum[e] = before + incl;
      if (offset != nullptr) offset[e + 1] = before + incl;
    }
    __syncthreads();
    if (threadIdx.x == 0) carry += warp_sums[31];
    __syncthreads();
  }
}

// Stable counting-sort scatter.  Chunk b owns flat slots [b*chunk, (b+1)*chunk); block_hist[b][e]
// already holds how many slots of bin e precede the chunk.  Grouped row of slot p:
//   r = offset[e] + block_hist[b][e] + (slots of bin e earlier in the chunk)
// Outputs: s_scatter[r] = p, s_reverse[p] = r, x_gather[r] = token of slot p
// (p / K for a fixed K per token, token_idx[p] when the caller lists the pairs).
__global__ void __launch_bounds__(kSortThreads) sort_scatter_kernel(const int* __restrict__ idx, long long n, int E,
                                                                    const int* __restrict__ block_hist,
                                                                    const int* __restrict__ offset, int K,
                                                                    const int* __restrict__ token_idx,
                                                                    int* __restrict__ s_scatter,
                                                                    int* __restrict__ s_reverse,
                                                                    int* __restrict__ x_gather) {
  extern __shared__ int sm[];
  int* running = sm;                 // [E] slots of each bin already placed by this chunk (plus bases)
  int* warp_cnt = sm + E;            // [kSortWarps][E]
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  for (int e = threadIdx.x; e < E; e += blockDim.x) {
    running[e] = offset[e] + block_hist[static_cast<long long>(blockIdx.x) * E + e];
#pragma unroll
    for (int w = 0; w < kSortWarps; ++w) warp_cnt[w * E + e] = 0;
  }
  __syncthreads();
  const long long chunk = (n + gridDim.x - 1) / gridDim.x;
  const long long begin = chunk * blockIdx.x;
  const long long end = begin + chunk < n ? begin + chunk : n;
  for (long long step = begin; step < end; step += blockDim.x) {
    const long long p = step + threadIdx.x;
    const bool valid = p < end;
    int e = valid ? idx[p] : -1;
    if (e < 0 || e >= E) e = -1;  // out-of-range ids are dropped (the histogram skipped them too)
    const unsigned peers = __match_any_sync(0xffffffffu, e);
    const int rank_in_warp = __popc(peers & ((1u << lane) - 1u));
    const bool leader = (e >= 0) && (rank_in_warp == 0);
    if (leader) warp_cnt[warp * E + e] = __popc(peers);
    __syncthreads();
    if (e >= 0) {
      int before = running[e];
      for (int w = 0; w < warp; ++w) before += warp_cnt[w * E + e];
      const int r = before + rank_in_warp;
      s_scatter[r] = static_cast<int>(p);
      s_reverse[p] = r;
      x_gather[r] = token_idx != nullptr ? token_idx[p] : static_cast<int>(p / K);
    }
    __syncthreads();
    if (leader) {
      atomicAdd(&running[e], __popc(peers));
      warp_cnt[warp * E + e] = 0;
    }
    __syncthreads();
  }
}

// offsets[t] = first position p with sorted_idx[p] >= t, for t = 0..T (offsets[T] = n).
__global__ void sorted_offsets_kernel(const int* __restrict__ sorted_idx, long long n, int T,
                                      int* __restrict__ offsets) {
  const int t = blockIdx.x * blockDim.x + threadIdx.x;
  if (t > T) return;
  long long lo = 0, hi = n;
  while (lo < hi) {
    const long long mid = (lo + hi) >> 1;
    if (sorted_idx[mid] < t) lo = mid + 1; else hi = mid;
  }
  offsets[t] = static_cast<int>(lo);
}

// ----------------------------------------------------------------------------------------------
// gather-and-sum over each token's routed rows
// ----------------------------------------------------------------------------------------------
// out[t, :] = sum_{p in [tok_off[t], tok_off[t+1])} w[p] * src[rev[p], :]   (w == nullptr: plain sum)
// tok_off == nullptr means a fixed K rows per token: p in [t*K, (t+1)*K).
// One thread per 8 consecutive columns of one token, fp32 accumulation.
template <typename W, bool ADD_FP32>
__global__ void __launch_bounds__(256) gather_sum_kernel(const __nv_bfloat16* __restrict__ src,
                                                         __nv_bfloat16* __restrict__ out, const W* __restrict__ w,
                                                         const int* __restrict__ rev, const int* __restrict__ tok_off,
                                                         const float* __restrict__ add, int T, int H, int K) {
  const int vec_per_row = H >> 3;
  const long long g = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (g >= static_cast<long long>(T) * vec_per_row) return;
  const int t = static_cast<int>(g / vec_per_row);
  const int c = static_cast<int>(g % vec_per_row);
  int p0, p1;
  if (tok_off != nullptr) { p0 = tok_off[t]; p1 = tok_off[t + 1]; } else { p0 = t * K; p1 = p0 + K; }
  float acc[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) acc[j] = 0.f;
  if constexpr (ADD_FP32) {
    const float4 a0 = reinterpret_cast<const float4*>(add + static_cast<long long>(t) * H)[2 * c];
    const float4 a1 = reinterpret_cast<const float4*>(add + static_cast<long long>(t) * H)[2 * c + 1];
    acc[0] = a0.x; acc[1] = a0.y; acc[2] = a0.z; acc[3] = a0.w;
    acc[4] = a1.x; acc[5] = a1.y; acc[6] = a1.z; acc[7] = a1.w;
  }
#pragma unroll 4
  for (int p = p0; p < p1; ++p) {
    const int r = rev[p];
    const float wt = (w != nullptr) ? static_cast<float>(w[p]) : 1.f;
    const uint4 v = reinterpret_cast<const uint4*>(src + static_cast<long long>(r) * H)[c];
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 f = __bfloat1622float2(h[j]);
      acc[2 * j] += wt * f.x;
      acc[2 * j + 1] += wt * f.y;
    }
  }
  uint4 o;
  __nv_bfloat162* oh = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
  for (int j = 0; j < 4; ++j) oh[j] = __floats2bfloat162_rn(acc[2 * j], acc[2 * j + 1]);
  reinterpret_cast<uint4*>(out + static_cast<long long>(t) * H)[c] = o;
}

// fp32 (T,H) -> bf16 (T,H)
__global__ void __launch_bounds__(256) cast_f32_bf16_kernel(const float* __restrict__ src,
                                                            __nv_bfloat16* __restrict__ dst, long long n8) {
  const long long g = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (g >= n8) return;
  const float4 a = reinterpret_cast<const float4*>(src)[2 * g];
  const float4 b = reinterpret_cast<const float4*>(src)[2 * g + 1];
  uint4 o;
  __nv_bfloat162* oh = reinterpret_cast<__nv_bfloat162*>(&o);
  oh[0] = __floats2bfloat162_rn(a.x, a.y);
  oh[1] = __floats2bfloat162_rn(a.z, a.w);
  oh[2] = __floats2bfloat162_rn(b.x, b.y);
  oh[3] = __floats2bfloat162_rn(b.z, b.w);
  reinterpret_cast<uint4*>(dst)[g] = o;
}

// ds[s_scatter[r]] = sum_c ds_partial[c, r]
template <typename OutT>
__global__ void __launch_bounds__(256) ds_reduce_kernel(const float* __restrict__ ds_partial,
                                                        const int* __restrict__ s_scatter, OutT* __restrict__ ds,
                                                        int TK, int ncols) {
  const int r = blockIdx.x * blockDim.x + threadIdx.x;
  if (r >= TK) return;
  float acc = 0.f;
  for (int c = 0; c < ncols; ++c) acc += ds_partial[static_cast<long long>(c) * TK + r];
  ds[s_scatter[r]] = static_cast<OutT>(acc);
}

// Scratch of the allocation-free entry point: kMaxSortBlocks x kNoAllocMaxExperts per-chunk bins
// (512 KiB), resident on every GPU that loads the library until the process exits.
constexpr int kNoAllocMaxExperts = 1024;
static __device__ __align__(256) int g_noalloc_hist[kMaxSortBlocks * kNoAllocMaxExperts];

// Device address of g_noalloc_hist on the current device.  In host code the symbol itself is only a
// host-side handle, never a device pointer, so the address is looked up once per device.
static int noalloc_scratch(int** out) {
  static std::mutex mu;
  static int* cached[kMaxDevices] = {};
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return SMOE_ERR_DRIVER;
  std::lock_guard<std::mutex> lock(mu);
  if (cached[dev] == nullptr) {
    void* ptr = nullptr;
    if (cudaGetSymbolAddress(&ptr, g_noalloc_hist) != cudaSuccess || ptr == nullptr) return SMOE_ERR_DRIVER;
    cached[dev] = static_cast<int*>(ptr);
  }
  *out = cached[dev];
  return SMOE_OK;
}

// out[e, n] = sum over the grouped rows r of expert e of w_r * src[row(r), n]   (bias gradients)
//   row(r) = gather[r] or r;  w_r = scores[s_scatter[r]] or 1.  One CTA per (expert, 256 columns):
//   warp w takes rows w, w+8, ...; a lane covers 8 columns; partial sums meet in shared memory.
template <typename ScoreT>
__global__ void __launch_bounds__(256) expert_column_sum_kernel(const __nv_bfloat16* __restrict__ src, long long ld,
                                                                const int* __restrict__ gather,
                                                                const ScoreT* __restrict__ scores,
                                                                const int* __restrict__ s_scatter,
                                                                const int* __restrict__ off,
                                                                __nv_bfloat16* __restrict__ out, int N) {
  __shared__ float part[8][256];
  const int e = blockIdx.x;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int col = blockIdx.y * 256 + lane * 8;
  float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
  if (col < N) {
    for (int r = off[e] + warp; r < off[e + 1]; r += 8) {
      const long long row = gather != nullptr ? gather[r] : r;
      const float w = scores != nullptr ? static_cast<float>(scores[s_scatter[r]]) : 1.f;
      const uint4 v = *reinterpret_cast<const uint4*>(src + row * ld + col);
      const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 f = __bfloat1622float2(h[j]);
        acc[2 * j] += w * f.x;
        acc[2 * j + 1] += w * f.y;
      }
    }
  }
#pragma unroll
  for (int j = 0; j < 8; ++j) part[warp][lane * 8 + j] = acc[j];
  __syncthreads();
  const int c = threadIdx.x;
  if (blockIdx.y * 256 + c < N) {
    float s = 0.f;
#pragma unroll
    for (int w = 0; w < 8; ++w) s += part[w][c];
    out[static_cast<long long>(e) * N + blockIdx.y * 256 + c] = __float2bfloat16(s);
  }
}

// ds[s_scatter[r]] += <dout[gather[r], :], b2[e(r), :]>: the part of the score gradient that comes from the
// down-projection bias.  One warp per grouped row; the expert of a row by binary search in the offsets.
template <typename DsT>
__global__ void __launch_bounds__(256) ds_bias_term_kernel(const __nv_bfloat16* __restrict__ dout,
                                                           const __nv_bfloat16* __restrict__ b2,
                                                           const int* __restrict__ off, const int* __restrict__ gather,
                                                           const int* __restrict__ s_scatter, DsT* __restrict__ ds,
                                                           int E, int H, int TK) {
  const int lane = threadIdx.x & 31;
  const int r = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (r >= TK) return;
  int lo = 0, hi = E;
  while (hi - lo > 1) {
    const int mid = (lo + hi) >> 1;
    if (off[mid] <= r) lo = mid; else hi = mid;
  }
  const __nv_bfloat16* a = dout + static_cast<long long>(gather[r]) * H;
  const __nv_bfloat16* b = b2 + static_cast<long long>(lo) * H;
  float acc = 0.f;
  for (int c = lane * 8; c < H; c += 256) {
    const uint4 va = *reinterpret_cast<const uint4*>(a + c), vb = *reinterpret_cast<const uint4*>(b + c);
    const __nv_bfloat162* ha = reinterpret_cast<const __nv_bfloat162*>(&va);
    const __nv_bfloat162* hb = reinterpret_cast<const __nv_bfloat162*>(&vb);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 fa = __bfloat1622float2(ha[j]), fb = __bfloat1622float2(hb[j]);
      acc += fa.x * fb.x + fa.y * fb.y;
    }
  }
#pragma unroll
  for (int d = 16; d > 0; d >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, d);
  if (lane == 0) {
    const int slot = s_scatter[r];
    ds[slot] = static_cast<DsT>(static_cast<float>(ds[slot]) + acc);
  }
}

static int sort_blocks(long long n) {
  long long b = (n + 4 * kSortThreads - 1) / (4 * kSortThreads);
  if (b < 1) b = 1;
  if (b > kMaxSortBlocks) b = kMaxSortBlocks;
  return static_cast<int>(b);
}

}  // namespace smoe

using namespace smoe;

extern "C" {

int smoe_abi_version(void) { return 1; }

int smoe_topk_softmax(const void* logits, int logits_dtype, float* scores, int* indices, int T, int E, int K,
                      void* stream) {
  if (T < 0 || E <= 0 || K <= 0 || K > E) return SMOE_ERR_SHAPE;
  if (T == 0) return SMOE_OK;
  if (logits_dtype == SMOE_F32) return launch_topk<float>(logits, scores, indices, T, E, K, S(stream));
  if (logits_dtype == SMOE_BF16) return launch_topk<__nv_bfloat16>(logits, scores, indices, T, E, K, S(stream));
  return SMOE_ERR_DTYPE;
}

int smoe_softmax_topk_backward(void* dlogits, int dlogits_dtype, const float* dscore, const float* score,
                               const int* indices, int T, int E, int K, void* stream) {
  if (T < 0 || E <= 0 || K <= 0 || K > E) return SMOE_ERR_SHAPE;
  if (T == 0) return SMOE_OK;
  const unsigned grid = (T + 7) / 8;
  if (dlogits_dtype == SMOE_F32) {
    softmax_topk_bwd_kernel<float><<<grid, 256, 0, S(stream)>>>(static_cast<float*>(dlogits), dscore, score, indices,
                                                                 T, E, K);
  } else if (dlogits_dtype == SMOE_BF16) {
    softmax_topk_bwd_kernel<__nv_bfloat16><<<grid, 256, 0, S(stream)>>>(static_cast<__nv_bfloat16*>(dlogits), dscore,
                                                                         score, indices, T, E, K);
  } else {
    return SMOE_ERR_DTYPE;
  }
  return launch_rc();
}

size_t smoe_count_cumsum_workspace_bytes(int E) {
  return static_cast<size_t>(kMaxSortBlocks) * static_cast<size_t>(E > 0 ? E : 1) * sizeof(int);
}

int smoe_count_cumsum(const void* x, int x_dtype, long long n, int E, int* count, int* cumsum, void* workspace,
                      void* stream) {
  if (n < 0 || E <= 0 || count == nullptr) return SMOE_ERR_SHAPE;
  if (x_dtype != SMOE_I32 && x_dtype != SMOE_I64) return SMOE_ERR_DTYPE;
  cudaStream_t st = S(stream);
  if (E <= kMaxSmemExperts) {
    if (workspace == nullptr) return SMOE_ERR_WORKSPACE;
    int* hist = static_cast<int*>(workspace);
    const int blocks = sort_blocks(n);
    if (x_dtype == SMOE_I32)
      chunk_histogram_kernel<int><<<blocks, kSortThreads, E * sizeof(int), st>>>(static_cast<const int*>(x), n, E, hist);
    else
      chunk_histogram_kernel<long long><<<blocks, kSortThreads, E * sizeof(int), st>>>(
          static_cast<const long long*>(x), n, E, hist);
    scan_bins_kernel<<<1, 1024, 0, st>>>(hist, blocks, E, nullptr, count, cumsum, nullptr);
  } else {
    if (cudaMemsetAsync(count, 0, sizeof(int) * E, st) != cudaSuccess) return SMOE_ERR_LAUNCH;
    const int blocks = static_cast<int>(n / 1024 + 1 < 1184 ? n / 1024 + 1 : 1184);
    if (x_dtype == SMOE_I32)
      global_histogram_kernel<int><<<blocks, 256, 0, st>>>(static_cast<const int*>(x), n, E, count);
    else
      global_histogram_kernel<long long><<<blocks, 256, 0, st>>>(static_cast<const long long*>(x), n, E, count);
    if (cumsum != nullptr) scan_bins_kernel<<<1, 1024, 0, st>>>(nullptr, 0, E, count, nullptr, cumsum, nullptr);
  }
  return launch_rc();
}

size_t smoe_route_metadata_workspace_bytes(int E) { return smoe_count_cumsum_workspace_bytes(E); }

int smoe_count_cumsum_noalloc_max_experts(void) { return kNoAllocMaxExperts; }

// Same result as smoe_count_cumsum, for hosts that can give the library no workspace: the per-chunk
// histograms live in the file-scope device array g_noalloc_hist instead.  Nothing is allocated or freed
// here, and no allocating runtime or library routine is called.
//   * E is limited to kNoAllocMaxExperts (1024) bins; a larger E returns SMOE_ERR_NOALLOC_LIMIT.
//   * The first call on each device looks the array's device address up (cudaGetSymbolAddress, with that
//     device current) and caches it; make that first call before any stream capture begins.
//   * All calls on a device share the one array.  It keeps whatever the previous call left in it, which is
//     harmless: the histogram kernel stores every entry the scan kernel later reads, so nothing has to
//     start at zero.  Two calls whose kernels overlap on the GPU (different streams) race on it: keep calls
//     on one device stream-ordered with respect to each other.
int smoe_count_cumsum_noalloc(const void* x, int x_dtype, long long n, int E, int* count, int* cumsum,
                              void* stream) {
  if (n < 0 || E <= 0 || count == nullptr) return SMOE_ERR_SHAPE;
  if (E > kNoAllocMaxExperts) return SMOE_ERR_NOALLOC_LIMIT;
  if (x_dtype != SMOE_I32 && x_dtype != SMOE_I64) return SMOE_ERR_DTYPE;
  int* hist = nullptr;
  const int rc = noalloc_scratch(&hist);
  if (rc != SMOE_OK) return rc;
  cudaStream_t st = S(stream);
  const int blocks = sort_blocks(n);
  if (x_dtype == SMOE_I32)
    chunk_histogram_kernel<int><<<blocks, kSortThreads, E * sizeof(int), st>>>(static_cast<const int*>(x), n, E, hist);
  else
    chunk_histogram_kernel<long long><<<blocks, kSortThreads, E * sizeof(int), st>>>(
        static_cast<const long long*>(x), n, E, hist);
  scan_bins_kernel<<<1, 1024, 0, st>>>(hist, blocks, E, nullptr, count, cumsum, nullptr);
  return launch_rc();
}

int smoe_route_metadata(const int* expert_idx, const int* token_idx, long long n, int E, int K, int* expert_count,
                        int* expert_offset, int* s_scatter_idx, int* s_reverse_scatter_idx, int* x_gather_idx,
                        void* workspace, void* stream) {
  if (n < 0 || E <= 0 || E > kMaxSmemExperts || n > 0x7FFFFFFFll) return SMOE_ERR_SHAPE;
  if (token_idx == nullptr && K <= 0) return SMOE_ERR_SHAPE;
  if (workspace == nullptr) return SMOE_ERR_WORKSPACE;
  cudaStream_t st = S(stream);
  int* hist = static_cast<int*>(workspace);
  const int blocks = sort_blocks(n);
  chunk_histogram_kernel<int><<<blocks, kSortThreads, E * sizeof(int), st>>>(expert_idx, n, E, hist);
  scan_bins_kernel<<<1, 1024, 0, st>>>(hist, blocks, E, nullptr, expert_count, nullptr, expert_offset);
  if (n > 0) {
    const size_t smem = static_cast<size_t>(E) * (1 + kSortWarps) * sizeof(int);
    static PerDeviceFlag configured;
    const int dev = current_device();
    if (dev < 0) return SMOE_ERR_DRIVER;
    if (!configured.test(dev)) {
      if (cudaFuncSetAttribute(sort_scatter_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                               kMaxSmemExperts * (1 + kSortWarps) * (int)sizeof(int)) != cudaSuccess)
        return SMOE_ERR_LAUNCH;
      configured.set(dev);
    }
    sort_scatter_kernel<<<blocks, kSortThreads, smem, st>>>(expert_idx, n, E, hist, expert_offset, K, token_idx,
                                                            s_scatter_idx, s_reverse_scatter_idx, x_gather_idx);
  }
  return launch_rc();
}

int smoe_sorted_offsets(const int* sorted_idx, long long n, int T, int* offsets, void* stream) {
  if (n < 0 || T < 0) return SMOE_ERR_SHAPE;
  sorted_offsets_kernel<<<(T + 1 + 255) / 256, 256, 0, S(stream)>>>(sorted_idx, n, T, offsets);
  return launch_rc();
}

int smoe_gather_sum(const void* src, void* out, const void* weights, int weights_dtype, const int* reverse_idx,
                    const int* token_offset, int T, int H, int K, void* stream) {
  if (T < 0 || H <= 0 || (H % 8) != 0) return SMOE_ERR_SHAPE;
  if (token_offset == nullptr && K <= 0) return SMOE_ERR_SHAPE;
  if (T == 0) return SMOE_OK;
  const long long total = static_cast<long long>(T) * (H / 8);
  const unsigned grid = static_cast<unsigned>((total + 255) / 256);
  const __nv_bfloat16* s = static_cast<const __nv_bfloat16*>(src);
  __nv_bfloat16* o = static_cast<__nv_bfloat16*>(out);
  if (weights == nullptr || weights_dtype == SMOE_F32) {
    gather_sum_kernel<float, false><<<grid, 256, 0, S(stream)>>>(s, o, static_cast<const float*>(weights), reverse_idx,
                                                                 token_offset, nullptr, T, H, K);
  } else if (weights_dtype == SMOE_BF16) {
    gather_sum_kernel<__nv_bfloat16, false><<<grid, 256, 0, S(stream)>>>(
        s, o, static_cast<const __nv_bfloat16*>(weights), reverse_idx, token_offset, nullptr, T, H, K);
  } else {
    return SMOE_ERR_DTYPE;
  }
  return launch_rc();
}

int smoe_cast_f32_to_bf16(const float* src, void* dst, long long n, void* stream) {
  if (n < 0 || (n % 8) != 0) return SMOE_ERR_SHAPE;
  if (n == 0) return SMOE_OK;
  const long long n8 = n / 8;
  cast_f32_bf16_kernel<<<static_cast<unsigned>((n8 + 255) / 256), 256, 0, S(stream)>>>(
      src, static_cast<__nv_bfloat16*>(dst), n8);
  return launch_rc();
}

int smoe_expert_column_sum(const void* src, long long ld, const int* gather_idx, const void* scores,
                           int scores_dtype, const int* s_scatter_idx, const int* expert_offset, void* out, int E,
                           int N, void* stream) {
  if (E <= 0 || N <= 0 || (N % 8) != 0 || (ld % 8) != 0) return SMOE_ERR_SHAPE;
  const dim3 grid(E, (N + 255) / 256);
  const __nv_bfloat16* s = static_cast<const __nv_bfloat16*>(src);
  __nv_bfloat16* o = static_cast<__nv_bfloat16*>(out);
  if (scores == nullptr || scores_dtype == SMOE_F32)
    expert_column_sum_kernel<float><<<grid, 256, 0, S(stream)>>>(s, ld, gather_idx, static_cast<const float*>(scores),
                                                                 s_scatter_idx, expert_offset, o, N);
  else if (scores_dtype == SMOE_BF16)
    expert_column_sum_kernel<__nv_bfloat16><<<grid, 256, 0, S(stream)>>>(
        s, ld, gather_idx, static_cast<const __nv_bfloat16*>(scores), s_scatter_idx, expert_offset, o, N);
  else
    return SMOE_ERR_DTYPE;
  return launch_rc();
}

int smoe_ds_add_bias_term(const void* dout, const void* b2, const int* expert_offset, const int* x_gather_idx,
                          const int* s_scatter_idx, void* ds, int ds_dtype, int E, int H, int TK, void* stream) {
  if (E <= 0 || H <= 0 || (H % 8) != 0 || TK < 0) return SMOE_ERR_SHAPE;
  if (TK == 0) return SMOE_OK;
  const unsigned grid = (TK + 7) / 8;
  const __nv_bfloat16* d = static_cast<const __nv_bfloat16*>(dout);
  const __nv_bfloat16* b = static_cast<const __nv_bfloat16*>(b2);
  if (ds_dtype == SMOE_F32)
    ds_bias_term_kernel<float><<<grid, 256, 0, S(stream)>>>(d, b, expert_offset, x_gather_idx, s_scatter_idx,
                                                            static_cast<float*>(ds), E, H, TK);
  else if (ds_dtype == SMOE_BF16)
    ds_bias_term_kernel<__nv_bfloat16><<<grid, 256, 0, S(stream)>>>(d, b, expert_offset, x_gather_idx, s_scatter_idx,
                                                                    static_cast<__nv_bfloat16*>(ds), E, H, TK);
  else
    return SMOE_ERR_DTYPE;
  return launch_rc();
}

int smoe_ds_reduce(const float* ds_partial, const int* s_scatter_idx, void* ds, int ds_dtype, int TK, int ncols,
                   void* stream) {
  if (TK < 0 || ncols <= 0) return SMOE_ERR_SHAPE;
  if (TK == 0) return SMOE_OK;
  const unsigned grid = (TK + 255) / 256;
  if (ds_dtype == SMOE_F32)
    ds_reduce_kernel<float><<<grid, 256, 0, S(stream)>>>(ds_partial, s_scatter_idx, static_cast<float*>(ds), TK, ncols);
  else if (ds_dtype == SMOE_BF16)
    ds_reduce_kernel<__nv_bfloat16><<<grid, 256, 0, S(stream)>>>(ds_partial, s_scatter_idx,
                                                                 static_cast<__nv_bfloat16*>(ds), TK, ncols);
  else
    return SMOE_ERR_DTYPE;
  return launch_rc();
}

}  // extern "C"

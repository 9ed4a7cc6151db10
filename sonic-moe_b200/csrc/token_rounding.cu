// Token-rounding selection: after the top-K choice every expert's token count is rounded to a multiple of
// the GEMM tile, by dropping its lowest-ranked top-K tokens or admitting its best-ranked other tokens.
//
// Ranking of the tokens of one expert (best first): tokens that chose the expert, by their renormalised
// score; then all other tokens by (score - 1), the subtraction rounded in the score's own dtype; equal values
// by lower token id.  Instead of sorting every expert's column, each expert finds its cut-off by a radix
// select over 32-bit order keys:
//
//   keys    : (T,E) scores -> (E,T) keys, transposed through shared memory; per-expert histogram of the top-K
//   select  : one CTA per expert: target count, 4 x 8-bit radix select of the target-th largest key, then an
//             ordered pass that writes the keep bitmask (E, T/32 words)
//   count   : per token, the number of experts that keep it; per-block sums
//   scan    : exclusive prefix over the block sums (one CTA)
//   emit    : (token, expert) pairs, tokens ascending, experts ascending within a token
//
// Integer / byte work on a few MB that stay in L2: coalesced reads, shared-memory histograms, no tensor cores.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <math.h>
#include <stdint.h>

#include "../../include/sonicmoe_b200.h"

namespace smoe {
namespace rounding {

constexpr int kTokTile = 32;       // tokens per transposing CTA
constexpr int kExpTile = 256;      // experts per transposing CTA
constexpr int kSelectThreads = 1024;
constexpr int kCountThreads = 256;

static inline cudaStream_t S(void* s) { return static_cast<cudaStream_t>(s); }
static inline int launch_rc() { return cudaGetLastError() == cudaSuccess ? SMOE_OK : SMOE_ERR_LAUNCH; }

// larger key = ranked earlier; -0.0 == +0.0
__device__ __forceinline__ uint32_t order_key(float v) {
  v = v + 0.0f;
  const uint32_t b = __float_as_uint(v);
  return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}

template <typename T>
struct Val;
template <>
struct Val<float> {
  static __device__ __forceinline__ float load(const float* p) { return *p; }
  static __device__ __forceinline__ float minus_one(float v) { return v - 1.0f; }
};
template <>
struct Val<__nv_bfloat16> {
  static __device__ __forceinline__ float load(const __nv_bfloat16* p) { return __bfloat162float(*p); }
  // the subtraction is done in bf16: exact in fp32, then rounded to nearest even
  static __device__ __forceinline__ float minus_one(float v) {
    return __bfloat162float(__float2bfloat16_rn(v - 1.0f));
  }
};

struct Layout {
  int t_words;            // ceil(T / 32)
  long long t_pad;        // 32 * t_words
  uint32_t* keys;         // (E, t_pad)
  uint32_t* keep;         // (E, t_words)
  int* freq;              // (E)  top-K histogram
  int* cnt_block;         // (blocks + 1) per-block pair counts, then their exclusive prefix
};

static size_t align256(size_t v) { return (v + 255) & ~static_cast<size_t>(255); }

static size_t carve(Layout& L, void* base, int T, int E) {
  L.t_words = (T + 31) / 32;
  L.t_pad = 32ll * L.t_words;
  const int blocks = (T + kCountThreads - 1) / kCountThreads;
  size_t off = 0;
  char* b = static_cast<char*>(base);
  L.keys = reinterpret_cast<uint32_t*>(b + off);
  off += align256(sizeof(uint32_t) * E * L.t_pad);
  L.keep = reinterpret_cast<uint32_t*>(b + off);
  off += align256(sizeof(uint32_t) * E * static_cast<size_t>(L.t_words));
  L.freq = reinterpret_cast<int*>(b + off);
  off += align256(sizeof(int) * E);
  L.cnt_block = reinterpret_cast<int*>(b + off);
  off += align256(sizeof(int) * (blocks + 1));
  return off;
}

// ---- keys ---------------------------------------------------------------------------------------
// grid (ceil(T/32), ceil(E/256)), 256 threads.  Tile [32 tokens][256 experts] in shared memory.
template <typename T>
__global__ void __launch_bounds__(256) keys_kernel(const T* __restrict__ scores, const int* __restrict__ topk,
                                                   int Tn, int E, int K, Layout L) {
  __shared__ uint32_t tile[kTokTile][kExpTile + 1];
  __shared__ int hist[kExpTile];
  const int t0 = blockIdx.x * kTokTile, e0 = blockIdx.y * kExpTile;
  const int tid = threadIdx.x;
  hist[tid] = 0;
  // every entry as "did not choose this expert": key(score - 1)
  for (int r = 0; r < kTokTile; ++r) {
    const int t = t0 + r, e = e0 + tid;
    uint32_t k = 0u;  // padding tokens rank below every real one
    if (t < Tn && e < E) k = order_key(Val<T>::minus_one(Val<T>::load(scores + static_cast<long long>(t) * E + e)));
    tile[r][tid] = k;
  }
  __syncthreads();
  // the top-K entries keep their score
  for (int i = tid; i < kTokTile * K; i += 256) {
    const int r = i / K, t = t0 + r;
    if (t < Tn) {
      const int e = topk[static_cast<long long>(t) * K + (i - r * K)];
      if (e >= e0 && e < e0 + kExpTile && e < E) {
        tile[r][e - e0] = order_key(Val<T>::load(scores + static_cast<long long>(t) * E + e));
        atomicAdd(&hist[e - e0], 1);
      }
    }
  }
  __syncthreads();
  if (e0 + tid < E && hist[tid] != 0) atomicAdd(&L.freq[e0 + tid], hist[tid]);
  // transposed store: 32 consecutive tokens of one expert = one 128-byte line
  const int lane = tid & 31, w = tid >> 5;
  for (int c = w; c < kExpTile; c += 8) {
    const int e = e0 + c;
    if (e < E) L.keys[static_cast<long long>(e) * L.t_pad + t0 + lane] = tile[lane][c];
  }
}

// ---- select -------------------------------------------------------------------------------------
__device__ __forceinline__ int target_count(int freq, int tile, int mode, int Tn) {
  int t;
  if (mode == SMOE_ROUND_DOWN) t = freq / tile * tile;
  else if (mode == SMOE_ROUND_UP) t = static_cast<int>(ceilf(static_cast<float>(freq) / static_cast<float>(tile))) * tile;
  else t = static_cast<int>(rintf(static_cast<float>(freq) / static_cast<float>(tile))) * tile;  // ties to even
  return min(t, Tn);
}

// One CTA per expert.
__global__ void __launch_bounds__(kSelectThreads) select_kernel(int Tn, int tile, int mode, Layout L,
                                                                int* __restrict__ expert_count) {
  __shared__ int hist[256];
  __shared__ int s_warp[kSelectThreads / 32];
  __shared__ uint32_t s_prefix;
  __shared__ int s_remaining;
  const int e = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const uint32_t* keys = L.keys + static_cast<long long>(e) * L.t_pad;
  uint32_t* keep = L.keep + static_cast<long long>(e) * L.t_words;
  const int target = target_count(L.freq[e], tile, mode, Tn);
  if (tid == 0) expert_count[e] = target;
  if (target == 0 || target >= Tn) {
    for (int w = tid; w < L.t_words; w += kSelectThreads) {
      uint32_t bits = 0u;
      if (target != 0) {
        const int left = Tn - 32 * w;
        bits = left >= 32 ? 0xFFFFFFFFu : ((1u << left) - 1u);
      }
      keep[w] = bits;
    }
    return;
  }
  // radix select: the target-th largest key (ties counted), most significant byte first
  uint32_t prefix = 0u;
  int remaining = target;  // rank still to be found among the keys that match the prefix
  for (int shift = 24; shift >= 0; shift -= 8) {
    if (tid < 256) hist[tid] = 0;
    __syncthreads();
    const uint32_t mask = shift == 24 ? 0u : (0xFFFFFFFFu << (shift + 8));
    for (int t = tid; t < Tn; t += kSelectThreads) {
      const uint32_t k = keys[t];
      if ((k & mask) == prefix) atomicAdd(&hist[(k >> shift) & 255u], 1);
    }
    __syncthreads();
    if (warp == 0) {
      // lane l owns digits 255-8l .. 248-8l (descending); find the digit where the running count reaches `remaining`
      int mine[8], sum = 0;
#pragma unroll
      for (int j = 0; j < 8; ++j) { mine[j] = hist[255 - (8 * lane + j)]; sum += mine[j]; }
      int incl = sum;
#pragma unroll
      for (int d = 1; d < 32; d <<= 1) {
        const int o = __shfl_up_sync(0xffffffffu, incl, d);
        if (lane >= d) incl += o;
      }
      int before = incl - sum;
      if (before < remaining && remaining <= incl) {
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          if (before < remaining && remaining <= before + mine[j]) {
            s_prefix = prefix | (static_cast<uint32_t>(255 - (8 * lane + j)) << shift);
            s_remaining = remaining - before;
          }
          before += mine[j];
        }
      }
    }
    __syncthreads();
    prefix = s_prefix;
    remaining = s_remaining;
    __syncthreads();
  }
  // prefix = cut-off key; `remaining` of the tokens with exactly this key are kept, lowest token ids first.
  // Thread i owns words [i*wpt, (i+1)*wpt): count its equal keys, exclusive scan over the block, then mark.
  const uint32_t thr = prefix;
  const int wpt = (L.t_words + kSelectThreads - 1) / kSelectThreads;
  const int w_begin = min(tid * wpt, L.t_words), w_end = min(w_begin + wpt, L.t_words);
  int eq = 0;
  for (int w = w_begin; w < w_end; ++w) {
    const uint4* p = reinterpret_cast<const uint4*>(keys + 32 * w);
#pragma unroll
    for (int q = 0; q < 8; ++q) {
      const uint4 v = p[q];
      eq += (v.x == thr) + (v.y == thr) + (v.z == thr) + (v.w == thr);
    }
  }
  int incl = eq;
#pragma unroll
  for (int d = 1; d < 32; d <<= 1) {
    const int o = __shfl_up_sync(0xffffffffu, incl, d);
    if (lane >= d) incl += o;
  }
  if (lane == 31) s_warp[warp] = incl;
  __syncthreads();
  if (warp == 0) {
    int v = s_warp[lane];
    int inc2 = v;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
      const int o = __shfl_up_sync(0xffffffffu, inc2, d);
      if (lane >= d) inc2 += o;
    }
    s_warp[lane] = inc2 - v;
  }
  __syncthreads();
  int eq_rank = s_warp[warp] + incl - eq;  // equal keys in all lower-numbered tokens
  for (int w = w_begin; w < w_end; ++w) {
    uint32_t bits = 0u;
    for (int b = 0; b < 32; ++b) {
      const uint32_t k = keys[32 * w + b];
      bool on = k > thr;
      if (k == thr) { on = eq_rank < remaining; ++eq_rank; }
      bits |= static_cast<uint32_t>(on) << b;
    }
    keep[w] = bits;
  }
}

// ---- count / scan / emit ------------------------------------------------------------------------
template <bool EMIT>
__global__ void __launch_bounds__(kCountThreads) count_emit_kernel(int Tn, int E, Layout L, int* __restrict__ tokens,
                                                                   int* __restrict__ experts, int capacity) {
  __shared__ int s_warp[kCountThreads / 32];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int t = blockIdx.x * kCountThreads + tid;
  const int w = t >> 5;  // same word for the whole warp
  int cnt = 0;
  if (w < L.t_words) {
    for (int e = 0; e < E; ++e) cnt += (L.keep[static_cast<long long>(e) * L.t_words + w] >> lane) & 1u;
  }
  if (t >= Tn) cnt = 0;
  int incl = cnt;
#pragma unroll
  for (int d = 1; d < 32; d <<= 1) {
    const int o = __shfl_up_sync(0xffffffffu, incl, d);
    if (lane >= d) incl += o;
  }
  if (lane == 31) s_warp[warp] = incl;
  __syncthreads();
  if (!EMIT) {
    if (tid == 0) {
      int s = 0;
      for (int i = 0; i < kCountThreads / 32; ++i) s += s_warp[i];
      L.cnt_block[blockIdx.x] = s;
    }
    return;
  }
  int base = L.cnt_block[blockIdx.x];
  for (int i = 0; i < warp; ++i) base += s_warp[i];
  int pos = base + incl - cnt;
  if (cnt == 0) return;
  for (int e = 0; e < E; ++e) {
    if ((L.keep[static_cast<long long>(e) * L.t_words + w] >> lane) & 1u) {
      if (pos < capacity) { tokens[pos] = t; experts[pos] = e; }
      ++pos;
    }
  }
}

// exclusive scan of cnt_block[0..n) in place; cnt_block[n] and *total = the sum
__global__ void __launch_bounds__(1024) scan_kernel(int* __restrict__ v, int n, int* __restrict__ total) {
  __shared__ int s_warp[32];
  __shared__ int s_carry;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  if (tid == 0) s_carry = 0;
  __syncthreads();
  for (int base = 0; base < n; base += 1024) {
    const int i = base + tid;
    const int x = i < n ? v[i] : 0;
    int incl = x;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
      const int o = __shfl_up_sync(0xffffffffu, incl, d);
      if (lane >= d) incl += o;
    }
    if (lane == 31) s_warp[warp] = incl;
    __syncthreads();
    if (warp == 0) {
      const int y = s_warp[lane];
      int inc2 = y;
#pragma unroll
      for (int d = 1; d < 32; d <<= 1) {
        const int o = __shfl_up_sync(0xffffffffu, inc2, d);
        if (lane >= d) inc2 += o;
      }
      s_warp[lane] = inc2 - y;
    }
    __syncthreads();
    const int carry = s_carry;
    if (i < n) v[i] = carry + s_warp[warp] + incl - x;
    __syncthreads();
    if (tid == 1023) s_carry = carry + s_warp[31] + incl;
    __syncthreads();
  }
  if (tid == 0) { v[n] = s_carry; *total = s_carry; }
}

}  // namespace rounding
}  // namespace smoe

using namespace smoe::rounding;

extern "C" size_t smoe_token_rounding_workspace_bytes(int T, int E) {
  if (T <= 0 || E <= 0) return 256;
  Layout L;
  return carve(L, nullptr, T, E);
}

extern "C" int smoe_token_rounding_select(const void* scores, int scores_dtype, const int* topk_idx, int T, int E, int K,
                                          int tile, int mode, int* expert_count, int* tokens, int* experts,
                                          int* num_pairs, int capacity, void* workspace, void* stream) {
  if (T < 0 || E <= 0 || K <= 0 || K > E || tile <= 0 || capacity < 0) return SMOE_ERR_SHAPE;
  if (mode != SMOE_ROUND_DOWN && mode != SMOE_ROUND_UP && mode != SMOE_ROUND_NEAREST) return SMOE_ERR_SHAPE;
  if (scores_dtype != SMOE_F32 && scores_dtype != SMOE_BF16) return SMOE_ERR_DTYPE;
  if (!expert_count || !num_pairs || !workspace) return SMOE_ERR_SHAPE;
  if (T > 0 && (!scores || !topk_idx || (capacity > 0 && (!tokens || !experts)))) return SMOE_ERR_SHAPE;
  if (reinterpret_cast<uintptr_t>(workspace) % 16 != 0) return SMOE_ERR_ALIGNMENT;
  cudaStream_t st = S(stream);
  if (T == 0) {
    cudaMemsetAsync(expert_count, 0, sizeof(int) * E, st);
    cudaMemsetAsync(num_pairs, 0, sizeof(int), st);
    return launch_rc();
  }
  Layout L;
  carve(L, workspace, T, E);
  cudaMemsetAsync(L.freq, 0, sizeof(int) * E, st);
  const dim3 kgrid((T + kTokTile - 1) / kTokTile, (E + kExpTile - 1) / kExpTile);
  if (scores_dtype == SMOE_F32)
    keys_kernel<float><<<kgrid, 256, 0, st>>>(static_cast<const float*>(scores), topk_idx, T, E, K, L);
  else
    keys_kernel<__nv_bfloat16><<<kgrid, 256, 0, st>>>(static_cast<const __nv_bfloat16*>(scores), topk_idx, T, E, K, L);
  select_kernel<<<E, kSelectThreads, 0, st>>>(T, tile, mode, L, expert_count);
  const int blocks = (T + kCountThreads - 1) / kCountThreads;
  count_emit_kernel<false><<<blocks, kCountThreads, 0, st>>>(T, E, L, nullptr, nullptr, 0);
  scan_kernel<<<1, 1024, 0, st>>>(L.cnt_block, blocks, num_pairs);
  count_emit_kernel<true><<<blocks, kCountThreads, 0, st>>>(T, E, L, tokens, experts, capacity);
  return launch_rc();
}

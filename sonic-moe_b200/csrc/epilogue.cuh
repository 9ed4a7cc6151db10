// Parameter block, status codes and the fused epilogues shared by the grouped GEMM kernels.
#pragma once
#include "ptx.cuh"

namespace smoe {


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

__device__ __forceinline__ float load_score(const void* scores, int is_bf16, int slot) {
  return is_bf16 ? __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(scores)[slot])
                 : reinterpret_cast<const float*>(scores)[slot];
}

__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

__device__ __forceinline__ float sigmoid_f(float x) { return __fdividef(1.0f, 1.0f + __expf(-x)); }

// One 32-column piece of one accumulator row: v[j] = acc[r, n + j] (fp32 bits).  `r` is the grouped row
// (ragged-M) or the output row inside the expert's matrix (ragged-K); only called for rows that exist.
template <int EPI, bool RAGGED_K>
__device__ __forceinline__ void epilogue_chunk(const GemmParams& p, int expert, int r, int n, const uint32_t (&v)[32],
                                       float score, float& ds_acc) {
  if constexpr (EPI == EPI_STORE) {
    __nv_bfloat16* dst = p.out0 + (RAGGED_K ? expert * p.out0_expert_stride : 0ll) + r * p.ld0 + n;
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

}  // namespace smoe

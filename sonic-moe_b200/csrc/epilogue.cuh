// Parameter block, status codes and the fused epilogues shared by the grouped GEMM kernels.
#pragma once
#include "ptx.cuh"

namespace smoe {


enum Epilogue : int {
  EPI_STORE = 0,    // out0[r, n] = bf16(acc)
  EPI_SWIGLU = 1,   // out0[r, n] = bf16(acc) (unless out0 == nullptr); out1[r, n/2] = silu(acc[2j]) * acc[2j+1]
  EPI_DSWIGLU = 2,  // acc = dy1; reads z, score; writes dz (out0), y1*s (out1), per-row partial of ds
  EPI_SCATTER = 3,  // red.add fp32: acc_out[token(r), n] += score(r) * acc
  // general forms: any activation of the layer, optional per-expert bias (GemmParams::act, ::bias)
  EPI_ACT = 4,         // z = acc + b1 -> out0 (unless nullptr); y1 = act(z) (gated: act(z_even) * z_odd) -> out1
  EPI_DACT = 5,        // acc = dy1; reads z, score; writes dz (out0), y1*s (out1), per-row partial of ds
  EPI_STORE_BIAS = 6,  // out0[r, n] = bf16(acc + bias[e, n])
  EPI_STORE_ROWS = 7,  // out0[gather[r], n] = bf16(score(r) * bf16(acc)) (score 1 when scores == nullptr): grouped rows
                       // written straight back to their source rows -- the combine of a layer whose tokens have one
                       // routed row each, with the rounding points of the store + gather_sum pair it replaces
};

// Activation codes (GemmParams::act).  The first three are gated: the pre-activation has 2I columns,
// gate = even column, up = odd column.
enum Activation : int { ACT_SWIGLU = 0, ACT_GEGLU = 1, ACT_REGLU = 2, ACT_RELU_SQ = 3, ACT_RELU = 4, ACT_GELU = 5,
                        ACT_SILU = 6 };
__host__ __device__ constexpr bool act_is_gated(int act) { return act <= ACT_REGLU; }

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
  int accumulate;           // plain-store epilogues: add to what out0 holds (bf16, fp32 sum, one rounding) instead of
                            // overwriting it -- weight gradients summed over several chunks of tokens
  // general epilogues
  const __nv_bfloat16* bias;  // (E, N) added to the accumulator, or nullptr
  int act;                    // Activation code
  // EPI_DSWIGLU of the hardware-scaled FP8 kernel: dz also leaves the epilogue quantised (E4M3, one UE8M0 scale
  // byte per row and 128 columns), nullptr = not wanted
  uint8_t* q_out;             // (total_rows, 2N)
  uint8_t* q_scale;           // (total_rows, q_scale_ld)
  long long q_scale_ld;
};

__device__ __forceinline__ float load_score(const void* scores, int is_bf16, int slot) {
  return is_bf16 ? __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(scores)[slot])
                 : reinterpret_cast<const float*>(scores)[slot];
}

__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

// sigmoid(x) = 0.5 tanh(x / 2) + 0.5 with the hardware tanh: one special-function operation per value instead of
// an exponential and a reciprocal (the epilogues are bound by those), the form the reference's epilogue uses too
// (sonicmoe/functional/grouped_gemm.py:413-421).  Absolute error about 2.5e-4, far below one bf16 step of the outputs.
__device__ __forceinline__ float sigmoid_f(float x) {
  float t;
  asm("tanh.approx.f32 %0, %1;" : "=f"(t) : "f"(0.5f * x));
  return fmaf(0.5f, t, 0.5f);
}

// Ask the L2 for `lines` consecutive 128-byte lines starting at p (no register, no wait).
__device__ __forceinline__ void prefetch_l2_lines(const void* p, int lines) {
  const char* c = static_cast<const char*>(p);
  for (int i = 0; i < lines; ++i) asm volatile("prefetch.global.L2 [%0];" ::"l"(c + 128 * i));
}

// value and derivative of the elementwise function behind every activation of the layer
__device__ __forceinline__ void act_value_grad(int act, float x, float& a, float& da) {
  switch (act) {
    case ACT_SWIGLU:
    case ACT_SILU: {
      const float sig = sigmoid_f(x);
      a = x * sig;
      da = sig * (1.f + x * (1.f - sig));
      break;
    }
    case ACT_GEGLU:
    case ACT_GELU: {  // exact (erf) GELU
      const float cdf = 0.5f * (1.f + erff(x * 0.70710678118654752f));
      a = x * cdf;
      da = cdf + x * 0.3989422804014327f * __expf(-0.5f * x * x);
      break;
    }
    case ACT_RELU_SQ: {
      const float r = fmaxf(x, 0.f);
      a = r * r;
      da = 2.f * r;
      break;
    }
    default: {  // ACT_REGLU, ACT_RELU
      a = fmaxf(x, 0.f);
      da = x > 0.f ? 1.f : 0.f;
      break;
    }
  }
}

__device__ __forceinline__ void store_bf16x32(__nv_bfloat16* dst, const float (&f)[32]) {
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    uint4 w;
    w.x = pack_bf16(f[8 * j + 0], f[8 * j + 1]);
    w.y = pack_bf16(f[8 * j + 2], f[8 * j + 3]);
    w.z = pack_bf16(f[8 * j + 4], f[8 * j + 5]);
    w.w = pack_bf16(f[8 * j + 6], f[8 * j + 7]);
    reinterpret_cast<uint4*>(dst)[j] = w;
  }
}

// Warp-cooperative row I/O through a warp's staging rows (32 rows of PITCH bytes).  Lane l owns row l of a 32-row
// block; global memory is touched with consecutive lanes on consecutive 16-byte pieces of one row, so an instruction
// moves whole 64- or 128-byte row segments.  Rows at or beyond row_end are skipped.  Every lane must call.
template <int PITCH>
__device__ __forceinline__ void warp_store_rows64(uint32_t stage, int lane, const uint32_t (&w)[16], __nv_bfloat16* out,
                                                  long long ld, int row_base, int row_end, int col) {
#pragma unroll
  for (int q = 0; q < 4; ++q) st_shared_v4(stage + lane * PITCH + 16 * q, w[4 * q], w[4 * q + 1], w[4 * q + 2], w[4 * q + 3]);
  __syncwarp();
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int rr = 8 * i + (lane >> 2);
    const uint4 v = ld_shared_v4(stage + rr * PITCH + 16 * (lane & 3));
    if (row_base + rr < row_end) *reinterpret_cast<uint4*>(out + (row_base + rr) * ld + col + 8 * (lane & 3)) = v;
  }
  __syncwarp();
}

template <int PITCH>
__device__ __forceinline__ void warp_store_rows128(uint32_t stage, int lane, const uint32_t (&w)[32], __nv_bfloat16* out,
                                                   long long ld, int row_base, int row_end, int col) {
  static_assert(PITCH >= 128 + 16, "128-byte payload");
#pragma unroll
  for (int q = 0; q < 8; ++q) st_shared_v4(stage + lane * PITCH + 16 * q, w[4 * q], w[4 * q + 1], w[4 * q + 2], w[4 * q + 3]);
  __syncwarp();
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int rr = 4 * i + (lane >> 3);
    const uint4 v = ld_shared_v4(stage + rr * PITCH + 16 * (lane & 7));
    if (row_base + rr < row_end) *reinterpret_cast<uint4*>(out + (row_base + rr) * ld + col + 8 * (lane & 7)) = v;
  }
  __syncwarp();
}

// The inverse: 32 rows x 128 bytes read with whole-row-segment loads; lane l ends with row l (zeros past row_end).
template <int PITCH>
__device__ __forceinline__ void warp_load_rows128(uint32_t stage, int lane, uint32_t (&w)[32], const __nv_bfloat16* src,
                                                  long long ld, int row_base, int row_end, int col) {
  static_assert(PITCH >= 128 + 16, "128-byte payload");
  uint4 v[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int rr = 4 * i + (lane >> 3);
    v[i] = make_uint4(0u, 0u, 0u, 0u);
    if (row_base + rr < row_end)
      v[i] = *reinterpret_cast<const uint4*>(src + (row_base + rr) * ld + col + 8 * (lane & 7));
  }
#pragma unroll
  for (int i = 0; i < 8; ++i)
    st_shared_v4(stage + (4 * i + (lane >> 3)) * PITCH + 16 * (lane & 7), v[i].x, v[i].y, v[i].z, v[i].w);
  __syncwarp();
#pragma unroll
  for (int q = 0; q < 8; ++q) {
    const uint4 t = ld_shared_v4(stage + lane * PITCH + 16 * q);
    w[4 * q] = t.x; w[4 * q + 1] = t.y; w[4 * q + 2] = t.z; w[4 * q + 3] = t.w;
  }
  __syncwarp();
}

// eight packed bf16 values plus the eight at dst (fp32 sums, rounded once)
__device__ __forceinline__ uint4 add_bf16x8(uint4 a, const uint4* dst) {
  const uint4 b = *dst;
  const uint32_t aw[4] = {a.x, a.y, a.z, a.w}, bw[4] = {b.x, b.y, b.z, b.w};
  uint32_t o[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 x = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&aw[i]));
    const float2 y = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&bw[i]));
    o[i] = pack_bf16(x.x + y.x, x.y + y.y);
  }
  return make_uint4(o[0], o[1], o[2], o[3]);
}

// acc (+ bias) as 32 floats
__device__ __forceinline__ void load_biased(const GemmParams& p, int expert, int n, const uint32_t (&v)[32],
                                            float (&f)[32]) {
#pragma unroll
  for (int j = 0; j < 32; ++j) f[j] = __uint_as_float(v[j]);
  if (p.bias != nullptr) {
    const uint4* b = reinterpret_cast<const uint4*>(p.bias + static_cast<long long>(expert) * p.N + n);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const uint4 w = b[j];
      const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&w);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float2 t = __bfloat1622float2(h[i]);
        f[8 * j + 2 * i] += t.x;
        f[8 * j + 2 * i + 1] += t.y;
      }
    }
  }
}

// One 32-column piece of one accumulator row: v[j] = acc[r, n + j] (fp32 bits).  `r` is the grouped row
// (ragged-M) or the output row inside the expert's matrix (ragged-K); only called for rows that exist.
// dSwiGLU on 32 accumulator columns (= 64 columns of dz).  acc[., i] = dy1[r, i]; z[r, 2i] = gate, z[r, 2i+1] = up.
// Writes dz (bf16), y1 * score, accumulates ds.  KEEP: the 32 packed bf16x2 words of dz replace v and amax collects
// max |dz| over the bf16 values (for a caller that also quantises dz).
template <bool KEEP>
__device__ __forceinline__ void dswiglu_chunk(const GemmParams& p, int r, int n, uint32_t (&v)[32], float score,
                                              float& ds_acc, float& amax) {
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
    if constexpr (KEEP) {
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        v[8 * j + i] = dzw[i];
        amax = fmaxf(amax, fmaxf(fabsf(__uint_as_float(dzw[i] << 16)), fabsf(__uint_as_float(dzw[i] & 0xFFFF0000u))));
      }
    }
  }
}

// 64-byte variant of warp_load_rows128 (staging rows of PITCH >= 80 bytes).
template <int PITCH>
__device__ __forceinline__ void warp_load_rows64(uint32_t stage, int lane, uint32_t (&w)[16], const __nv_bfloat16* src,
                                                 long long ld, int row_base, int row_end, int col) {
  uint4 v[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int rr = 8 * i + (lane >> 2);
    v[i] = make_uint4(0u, 0u, 0u, 0u);
    if (row_base + rr < row_end)
      v[i] = *reinterpret_cast<const uint4*>(src + (row_base + rr) * ld + col + 8 * (lane & 3));
  }
#pragma unroll
  for (int i = 0; i < 4; ++i)
    st_shared_v4(stage + (8 * i + (lane >> 2)) * PITCH + 16 * (lane & 3), v[i].x, v[i].y, v[i].z, v[i].w);
  __syncwarp();
#pragma unroll
  for (int q = 0; q < 4; ++q) {
    const uint4 t = ld_shared_v4(stage + lane * PITCH + 16 * q);
    w[4 * q] = t.x; w[4 * q + 1] = t.y; w[4 * q + 2] = t.z; w[4 * q + 3] = t.w;
  }
  __syncwarp();
}

// dswiglu_chunk with the row traffic (z in, dz and y1 * score out) going through the warp's staging rows as 64-byte
// row segments.  Every lane of the warp must call (lane l owns row row_base + l; rows at or past row_end read zeros
// and store nothing).  Same arithmetic, same results.
template <bool KEEP, int PITCH>
__device__ __forceinline__ void dswiglu_chunk_staged(const GemmParams& p, uint32_t stage, int lane, int row_base,
                                                     int row_end, int n, uint32_t (&v)[32], float score, float& ds_acc,
                                                     float& amax) {
  uint32_t za[16], zb[16], ys[16];
  warp_load_rows64<PITCH>(stage, lane, za, p.z, 2ll * p.N, row_base, row_end, 2 * n);
  warp_load_rows64<PITCH>(stage, lane, zb, p.z, 2ll * p.N, row_base, row_end, 2 * n + 32);
#pragma unroll
  for (int i = 0; i < 32; ++i) {
    uint32_t& zw = i < 16 ? za[i] : zb[i - 16];
    const __nv_bfloat162 gu = *reinterpret_cast<const __nv_bfloat162*>(&zw);
    const float g = __low2float(gu), u = __high2float(gu);
    const float dy = __uint_as_float(v[i]);
    const float sig = sigmoid_f(g);
    const float silu = g * sig;
    const float y1 = silu * u;
    ds_acc += dy * y1;
    const float dg = dy * u * (sig * (1.f + g * (1.f - sig))) * score;
    const float du = dy * silu * score;
    zw = pack_bf16(dg, du);
    v[i] = __float_as_uint(y1 * score);
  }
#pragma unroll
  for (int j = 0; j < 16; ++j) ys[j] = pack_bf16(__uint_as_float(v[2 * j]), __uint_as_float(v[2 * j + 1]));
  warp_store_rows64<PITCH>(stage, lane, za, p.out0, p.ld0, row_base, row_end, 2 * n);
  warp_store_rows64<PITCH>(stage, lane, zb, p.out0, p.ld0, row_base, row_end, 2 * n + 32);
  warp_store_rows64<PITCH>(stage, lane, ys, p.out1, p.ld1, row_base, row_end, n);
  if constexpr (KEEP) {
#pragma unroll
    for (int i = 0; i < 32; ++i) {
      const uint32_t w = i < 16 ? za[i] : zb[i - 16];
      v[i] = w;
      amax = fmaxf(amax, fmaxf(fabsf(__uint_as_float(w << 16)), fabsf(__uint_as_float(w & 0xFFFF0000u))));
    }
  }
}

template <int EPI, bool RAGGED_K>
__device__ __forceinline__ void epilogue_chunk(const GemmParams& p, int expert, int r, int n, uint32_t (&v)[32],
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
      uint4* d4 = reinterpret_cast<uint4*>(dst) + j;
      *d4 = p.accumulate ? add_bf16x8(w, d4) : w;
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
    float unused = 0.f;
    dswiglu_chunk<false>(p, r, n, v, score, ds_acc, unused);
  } else if constexpr (EPI == EPI_STORE_BIAS) {
    float f[32];
    load_biased(p, expert, n, v, f);
    store_bf16x32(p.out0 + r * p.ld0 + n, f);
  } else if constexpr (EPI == EPI_ACT) {
    float f[32];
    load_biased(p, expert, n, v, f);
    if (p.out0 != nullptr) store_bf16x32(p.out0 + r * p.ld0 + n, f);
    if (act_is_gated(p.act)) {
      float y[16];
#pragma unroll
      for (int j = 0; j < 16; ++j) {
        float a, da;
        act_value_grad(p.act, f[2 * j], a, da);
        y[j] = a * f[2 * j + 1];
      }
      __nv_bfloat16* dst1 = p.out1 + r * p.ld1 + (n >> 1);
#pragma unroll
      for (int j = 0; j < 2; ++j)
        reinterpret_cast<uint4*>(dst1)[j] = make_uint4(pack_bf16(y[8 * j], y[8 * j + 1]), pack_bf16(y[8 * j + 2], y[8 * j + 3]),
                                                       pack_bf16(y[8 * j + 4], y[8 * j + 5]), pack_bf16(y[8 * j + 6], y[8 * j + 7]));
    } else {
#pragma unroll
      for (int j = 0; j < 32; ++j) {
        float a, da;
        act_value_grad(p.act, f[j], a, da);
        f[j] = a;
      }
      store_bf16x32(p.out1 + r * p.ld1 + n, f);
    }
  } else if constexpr (EPI == EPI_DACT) {
    // acc[., i] = dy1[r, i]
    if (act_is_gated(p.act)) {
      const uint4* zsrc = reinterpret_cast<const uint4*>(p.z + static_cast<long long>(r) * (2ll * p.N) + 2 * n);
      __nv_bfloat16* dz_dst = p.out0 + r * p.ld0 + 2 * n;
      __nv_bfloat16* ys_dst = p.out1 + r * p.ld1 + n;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const uint4 za = zsrc[2 * j], zb = zsrc[2 * j + 1];
        const uint32_t zw[8] = {za.x, za.y, za.z, za.w, zb.x, zb.y, zb.z, zb.w};
        uint32_t dzw[8];
        float ys[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const __nv_bfloat162 gu = *reinterpret_cast<const __nv_bfloat162*>(&zw[i]);
          const float g = __low2float(gu), u = __high2float(gu);
          const float dy = __uint_as_float(v[8 * j + i]);
          float a, da;
          act_value_grad(p.act, g, a, da);
          const float y1 = a * u;
          ds_acc += dy * y1;
          dzw[i] = pack_bf16(dy * u * da * score, dy * a * score);
          ys[i] = y1 * score;
        }
        reinterpret_cast<uint4*>(dz_dst)[2 * j] = make_uint4(dzw[0], dzw[1], dzw[2], dzw[3]);
        reinterpret_cast<uint4*>(dz_dst)[2 * j + 1] = make_uint4(dzw[4], dzw[5], dzw[6], dzw[7]);
        reinterpret_cast<uint4*>(ys_dst)[j] = make_uint4(pack_bf16(ys[0], ys[1]), pack_bf16(ys[2], ys[3]),
                                                         pack_bf16(ys[4], ys[5]), pack_bf16(ys[6], ys[7]));
      }
    } else {
      const uint4* zsrc = reinterpret_cast<const uint4*>(p.z + static_cast<long long>(r) * p.N + n);
      float dzf[32], ysf[32];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const uint4 zq = zsrc[j];
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&zq);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const float zval = (i & 1) ? __high2float(h[i >> 1]) : __low2float(h[i >> 1]);
          const float dy = __uint_as_float(v[8 * j + i]);
          float a, da;
          act_value_grad(p.act, zval, a, da);
          ds_acc += dy * a;
          dzf[8 * j + i] = dy * da * score;
          ysf[8 * j + i] = a * score;
        }
      }
      store_bf16x32(p.out0 + r * p.ld0 + n, dzf);
      store_bf16x32(p.out1 + r * p.ld1 + n, ysf);
    }
  } else if constexpr (EPI == EPI_STORE_ROWS) {
    __nv_bfloat16* dst = p.out0 + static_cast<long long>(p.gather[r]) * p.ld0 + n;
    float f[32];
#pragma unroll
    for (int j = 0; j < 32; ++j) f[j] = __uint_as_float(v[j]);
    if (p.scores != nullptr) {
#pragma unroll
      for (int j = 0; j < 32; ++j) f[j] = score * __bfloat162float(__float2bfloat16_rn(f[j]));
    }
    store_bf16x32(dst, f);
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

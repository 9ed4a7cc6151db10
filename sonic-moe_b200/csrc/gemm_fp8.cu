// FP8 (E4M3) entry points: quantisation kernels and the launchers of the FP8 grouped GEMMs, for fp32 block
// scales (amax / 448, applied in software) and for power-of-two UE8M0 block scales (applied by the tensor cores).
#include "device_cache.cuh"
#include "gemm_fp8.cuh"
#include "gemm_mxfp8.cuh"

#include <cuda_fp8.h>

#include <cstdio>
#include <cstdlib>
#include <mutex>

#include "../../include/sonicmoe_b200.h"

namespace smoe {
namespace fp8 {

using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn get_encode_fn() {
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

// 1-byte row-major 2D tensor (rows, cols); box (box_rows, box_cols <= 128), 128-byte swizzle.
static int encode_u8(CUtensorMap* map, const void* base, uint64_t rows, uint64_t cols, uint32_t box_rows,
                     uint32_t box_cols) {
  EncodeTiledFn fn = get_encode_fn();
  if (fn == nullptr) return SMOE_ERR_DRIVER;
  static thread_local bool context_bound = false;
  if (!context_bound) {
    if (cudaFree(nullptr) != cudaSuccess) return SMOE_ERR_DRIVER;
    context_bound = true;
  }
  if ((reinterpret_cast<uintptr_t>(base) & 15u) != 0 || cols % 16 != 0) return SMOE_ERR_ALIGNMENT;
  const cuuint64_t dims[2] = {cols, rows};
  const cuuint64_t strides[1] = {cols};
  const cuuint32_t box[2] = {box_cols, box_rows};
  const cuuint32_t estr[2] = {1, 1};
  const CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box, estr,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? SMOE_OK : SMOE_ERR_TENSORMAP;
}

template <class Kernel, class ScaleArgs>
static int launch_kernel(Kernel kernel, PerDeviceFlag& configured, int smem_bytes, const CUtensorMap& tmA,
                         const CUtensorMap& tmB, const GemmParams& p, const ScaleArgs& sc, cudaStream_t stream) {
  const int dev = current_device();
  if (dev < 0) return SMOE_ERR_DRIVER;
  if (!configured.test(dev)) {
    if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes) != cudaSuccess)
      return SMOE_ERR_LAUNCH;
    // setmaxnreg 56 / 200 in these kernels balances only around 128 registers per thread at launch
    cudaFuncAttributes fa;
    if (cudaFuncGetAttributes(&fa, kernel) != cudaSuccess || fa.numRegs != 128) return SMOE_ERR_LAUNCH;
    configured.set(dev);
  }
  const int sms = num_sms();
  if (sms < 2) return SMOE_ERR_DRIVER;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(static_cast<unsigned>(sms & ~1), 1, 1);
  cfg.blockDim = dim3(THREADS, 1, 1);
  cfg.dynamicSmemBytes = smem_bytes;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kernel, tmA, tmB, p, sc) == cudaSuccess ? SMOE_OK : SMOE_ERR_LAUNCH;
}

template <bool A_GATHER, bool B_MN, int EPI>
static int launch(const CUtensorMap& tmA, const CUtensorMap& tmB, const GemmParams& p, const Scales& sc,
                  cudaStream_t stream) {
  static PerDeviceFlag configured;
  return launch_kernel(grouped_gemm_fp8_kernel<A_GATHER, B_MN, EPI>, configured, SMEM_BYTES, tmA, tmB, p, sc, stream);
}

template <bool A_GATHER, bool B_MN, int EPI>
static int launch_mx(const CUtensorMap& tmA, const CUtensorMap& tmB, const GemmParams& p, const mx8::ScaleBytes& sc,
                     cudaStream_t stream) {
  static PerDeviceFlag configured;
  return launch_kernel(mx8::grouped_gemm_mxfp8_kernel<A_GATHER, B_MN, EPI>, configured, mx8::SMEM_BYTES, tmA, tmB, p,
                       sc, stream);
}

// An empty batch (T == 0, hence TK == 0) is valid: the entry points return at once (weight-gradient entry points
// after zero-filling their output).  What is refused: negative sizes, or routed rows without any token.
static bool bad_tokens(int T, int TK) { return T < 0 || TK < 0 || (T == 0 && TK > 0); }

static bool bad_shape(int H, int I, int E) {
  return H <= 0 || I <= 0 || E <= 0 || E > MAX_EXPERTS || (H % 128) != 0 || (I % 128) != 0;
}

// ---- quantisation ------------------------------------------------------------------------------------
__device__ __forceinline__ uint8_t to_e4m3(float v) {
  return static_cast<uint8_t>(__nv_cvt_float_to_fp8(v, __NV_SATFINITE, __NV_E4M3));
}

// four values -> four E4M3 bytes (two paired conversions), first value in the low byte
__device__ __forceinline__ uint32_t pack_e4m3x4(float a, float b, float c, float d) {
  const uint32_t lo = __nv_cvt_float2_to_fp8x2(make_float2(a, b), __NV_SATFINITE, __NV_E4M3);
  const uint32_t hi = __nv_cvt_float2_to_fp8x2(make_float2(c, d), __NV_SATFINITE, __NV_E4M3);
  return lo | (hi << 16);
}

// Row quantiser: one warp per row and group of four 128-column blocks (512 columns): a lane holds 4 values of each
// block, the four loads are issued together, each block is reduced with shuffles.  POW2: the four scale bytes of the
// group are one 32-bit word of the padded scale row (ld bytes per row, ld % 4 == 0, padding = 2^0); otherwise fp32
// scales amax / 448, one per block (ld = blocks per row).
template <bool POW2>
__global__ void __launch_bounds__(256) quantize_rows_kernel(const __nv_bfloat16* __restrict__ x,
                                                            uint8_t* __restrict__ q, void* __restrict__ scale,
                                                            long long rows, int cols, int ld) {
  const int nblk = cols >> 7;
  const int groups = (nblk + 3) >> 2;
  const long long w = static_cast<long long>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (w >= rows * groups) return;
  const int lane = threadIdx.x & 31;
  const long long row = w / groups;
  const int g = static_cast<int>(w % groups);
  const __nv_bfloat16* src = x + row * cols + g * 512;
  uint2 raw[4];
#pragma unroll
  for (int b = 0; b < 4; ++b) {
    raw[b] = make_uint2(0u, 0u);
    if (4 * g + b < nblk) raw[b] = reinterpret_cast<const uint2*>(src + b * 128)[lane];
  }
  uint32_t word = 0;
#pragma unroll
  for (int b = 0; b < 4; ++b) {
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw[b]);
    const float2 v0 = __bfloat1622float2(h[0]), v1 = __bfloat1622float2(h[1]);
    float amax = fmaxf(fmaxf(fabsf(v0.x), fabsf(v0.y)), fmaxf(fabsf(v1.x), fabsf(v1.y)));
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, d));
    const bool live = 4 * g + b < nblk;
    uint32_t packed;
    if (POW2) {
      float inv;
      const uint32_t byte = pow2_scale(amax, inv);
      word |= (live ? byte : 0x7Fu) << (8 * b);
      packed = pack_e4m3x4(v0.x * inv, v0.y * inv, v1.x * inv, v1.y * inv);
    } else {
      // true division: a reciprocal of a denormal scale would overflow and turn the block's zeros into NaN
      const float sc = amax > 0.f ? amax / 448.f : 1.f;
      packed = pack_e4m3x4(v0.x / sc, v0.y / sc, v1.x / sc, v1.y / sc);
      if (live && lane == 0) static_cast<float*>(scale)[row * ld + 4 * g + b] = sc;
    }
    if (live) reinterpret_cast<uint32_t*>(q + row * cols + g * 512 + b * 128)[lane] = packed;
  }
  if (POW2 && lane == 0) reinterpret_cast<uint32_t*>(static_cast<uint8_t*>(scale) + row * ld)[g] = word;
}

// One CTA per 128 x 128 block of a (batch, rows, cols) tensor; rows need not be a multiple of 128.
// POW2: the scale is a UE8M0 byte (smallest power of two >= amax / 448), else fp32 amax / 448.
template <bool POW2>
__global__ void __launch_bounds__(256) quantize_blocks_kernel(const __nv_bfloat16* __restrict__ w,
                                                              uint8_t* __restrict__ q, void* __restrict__ scale,
                                                              int rows, int cols) {
  __shared__ float warp_max[8];
  const int cb = blockIdx.x, rb = blockIdx.y, e = blockIdx.z;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const long long base = (static_cast<long long>(e) * rows + static_cast<long long>(rb) * 128) * cols + cb * 128;
  const int nrows = min(128, rows - rb * 128);
  float amax = 0.f;
  // pass 1: warp w scans rows 16w .. 16w+15 of the block (a lane covers 4 columns)
  for (int rr = 0; rr < 16; ++rr) {
    const int r = warp * 16 + rr;
    if (r < nrows) {
      const uint2 v = reinterpret_cast<const uint2*>(w + base + static_cast<long long>(r) * cols)[lane];
      const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
      const float2 a = __bfloat1622float2(h[0]), b = __bfloat1622float2(h[1]);
      amax = fmaxf(amax, fmaxf(fmaxf(fabsf(a.x), fabsf(a.y)), fmaxf(fabsf(b.x), fabsf(b.y))));
    }
  }
#pragma unroll
  for (int d = 16; d > 0; d >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, d));
  if (lane == 0) warp_max[warp] = amax;
  __syncthreads();
  amax = warp_max[0];
#pragma unroll
  for (int i = 1; i < 8; ++i) amax = fmaxf(amax, warp_max[i]);
  const float s = amax > 0.f ? amax / 448.f : 1.f;
  float inv = 1.f;
  const uint8_t byte = POW2 ? pow2_scale(amax, inv) : 0;
  // pass 2: the block is still in L1/L2
  for (int rr = 0; rr < 16; ++rr) {
    const int r = warp * 16 + rr;
    if (r < nrows) {
      const uint2 v = reinterpret_cast<const uint2*>(w + base + static_cast<long long>(r) * cols)[lane];
      const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
      const float2 a = __bfloat1622float2(h[0]), b = __bfloat1622float2(h[1]);
      uint32_t packed;
      if (POW2)
        packed = to_e4m3(a.x * inv) | (to_e4m3(a.y * inv) << 8) | (to_e4m3(b.x * inv) << 16) | (to_e4m3(b.y * inv) << 24);
      else
        packed = to_e4m3(a.x / s) | (to_e4m3(a.y / s) << 8) | (to_e4m3(b.x / s) << 16) | (to_e4m3(b.y / s) << 24);
      reinterpret_cast<uint32_t*>(q + base + static_cast<long long>(r) * cols)[lane] = packed;
    }
  }
  if (threadIdx.x == 0) {
    const long long idx = (static_cast<long long>(e) * gridDim.y + rb) * gridDim.x + cb;
    if (POW2) static_cast<uint8_t*>(scale)[idx] = byte;
    else static_cast<float*>(scale)[idx] = s;
  }
}

}  // namespace fp8
}  // namespace smoe

using namespace smoe;
using namespace smoe::fp8;

#define SMOE_TRY(expr)              \
  do {                              \
    const int _rc = (expr);         \
    if (_rc != SMOE_OK) return _rc; \
  } while (0)

extern "C" {

int smoe_fp8_quantize_rows(const void* x, void* q, float* scale, long long rows, int cols, void* stream) {
  if (rows < 0 || cols <= 0 || (cols % 128) != 0) return SMOE_ERR_SHAPE;
  if (rows == 0) return SMOE_OK;
  const int nblk = cols / 128;
  const long long warps = rows * ((nblk + 3) / 4);
  quantize_rows_kernel<false><<<static_cast<unsigned>((warps + 7) / 8), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(x), static_cast<uint8_t*>(q), scale, rows, cols, nblk);
  return cudaGetLastError() == cudaSuccess ? SMOE_OK : SMOE_ERR_LAUNCH;
}

int smoe_fp8_quantize_blocks(const void* w, void* q, float* scale, int batch, int rows, int cols, void* stream) {
  if (batch <= 0 || rows <= 0 || cols <= 0 || (cols % 128) != 0) return SMOE_ERR_SHAPE;
  const dim3 grid(cols / 128, (rows + 127) / 128, batch);
  quantize_blocks_kernel<false><<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(w), static_cast<uint8_t*>(q), scale, rows, cols);
  return cudaGetLastError() == cudaSuccess ? SMOE_OK : SMOE_ERR_LAUNCH;
}

int smoe_fp8_up_projection_forward(const void* xq, const float* x_scale, const void* w1q, const float* w1_scale,
                                   void* z, void* y1, const int* expert_offset, const int* x_gather_idx, int T, int H,
                                   int I, int E, int TK, int* status, void* stream) {
  if (bad_shape(H, I, E) || bad_tokens(T, TK)) return SMOE_ERR_SHAPE;
  if (TK == 0) return SMOE_OK;
  CUtensorMap tmA, tmB;
  SMOE_TRY(encode_u8(&tmA, xq, T, H, 1, BK));
  SMOE_TRY(encode_u8(&tmB, w1q, (uint64_t)E * 2 * I, H, BN_CTA, BK));
  GemmParams p = {};
  p.E = E; p.N = 2 * I; p.K = H; p.total_rows = TK; p.gather_rows = T; p.b_rows_per_expert = 2 * I;
  p.off = expert_offset; p.gather = x_gather_idx;
  p.out0 = static_cast<__nv_bfloat16*>(z); p.ld0 = 2 * I;
  p.out1 = static_cast<__nv_bfloat16*>(y1); p.ld1 = I;
  p.status = status;
  Scales sc = {x_scale, H / 128, w1_scale, (long long)(2 * I / 128) * (H / 128), H / 128, 1};
  return launch<true, false, EPI_SWIGLU>(tmA, tmB, p, sc, static_cast<cudaStream_t>(stream));
}

int smoe_fp8_down_projection_forward(const void* y1q, const float* y1_scale, const void* w2q, const float* w2_scale,
                                     void* y2, const int* expert_offset, int H, int I, int E, int TK, int* status,
                                     void* stream) {
  if (bad_shape(H, I, E) || TK < 0) return SMOE_ERR_SHAPE;
  if (TK == 0) return SMOE_OK;
  CUtensorMap tmA, tmB;
  SMOE_TRY(encode_u8(&tmA, y1q, TK, I, BM, BK));
  SMOE_TRY(encode_u8(&tmB, w2q, (uint64_t)E * H, I, BN_CTA, BK));
  GemmParams p = {};
  p.E = E; p.N = H; p.K = I; p.total_rows = TK; p.b_rows_per_expert = H;
  p.off = expert_offset;
  p.out0 = static_cast<__nv_bfloat16*>(y2); p.ld0 = H;
  p.status = status;
  Scales sc = {y1_scale, I / 128, w2_scale, (long long)(H / 128) * (I / 128), I / 128, 1};
  return launch<false, false, EPI_STORE>(tmA, tmB, p, sc, static_cast<cudaStream_t>(stream));
}

int smoe_fp8_down_projection_backward_act(const void* doutq, const float* dout_scale, const void* w2q,
                                          const float* w2_scale, const void* z, const void* scores,
                                          int scores_are_bf16, void* dz, void* y1s, float* ds_partial,
                                          const int* expert_offset, const int* x_gather_idx,
                                          const int* s_scatter_idx, int T, int H, int I, int E, int TK, int* status,
                                          void* stream) {
  if (bad_shape(H, I, E) || bad_tokens(T, TK)) return SMOE_ERR_SHAPE;
  if (TK == 0) return SMOE_OK;
  CUtensorMap tmA, tmB;
  SMOE_TRY(encode_u8(&tmA, doutq, T, H, 1, BK));
  SMOE_TRY(encode_u8(&tmB, w2q, (uint64_t)E * H, I, BK, BN_CTA));  // W2[e] (H, I): rows are k
  GemmParams p = {};
  p.E = E; p.N = I; p.K = H; p.total_rows = TK; p.gather_rows = T; p.b_rows_per_expert = H;
  p.off = expert_offset; p.gather = x_gather_idx; p.s_scatter = s_scatter_idx;
  p.out0 = static_cast<__nv_bfloat16*>(dz); p.ld0 = 2 * I;
  p.out1 = static_cast<__nv_bfloat16*>(y1s); p.ld1 = I;
  p.z = static_cast<const __nv_bfloat16*>(z);
  p.scores = scores; p.scores_are_bf16 = scores_are_bf16; p.ds_partial = ds_partial;
  p.status = status;
  // blocks of W2[e] are (h/128, i/128): k-block stride = I/128, n-block stride = 1
  Scales sc = {dout_scale, H / 128, w2_scale, (long long)(H / 128) * (I / 128), 1, I / 128};
  return launch<true, true, EPI_DSWIGLU>(tmA, tmB, p, sc, static_cast<cudaStream_t>(stream));
}

int smoe_fp8_up_projection_backward_dx(const void* dzq, const float* dz_scale, const void* w1q, const float* w1_scale,
                                       void* dx_expanded, const int* expert_offset, int H, int I, int E, int TK,
                                       int* status, void* stream) {
  if (bad_shape(H, I, E) || TK < 0) return SMOE_ERR_SHAPE;
  if (TK == 0) return SMOE_OK;
  CUtensorMap tmA, tmB;
  SMOE_TRY(encode_u8(&tmA, dzq, TK, 2 * I, BM, BK));
  SMOE_TRY(encode_u8(&tmB, w1q, (uint64_t)E * 2 * I, H, BK, BN_CTA));  // W1[e] (2I, H): rows are k
  GemmParams p = {};
  p.E = E; p.N = H; p.K = 2 * I; p.total_rows = TK; p.b_rows_per_expert = 2 * I;
  p.off = expert_offset;
  p.out0 = static_cast<__nv_bfloat16*>(dx_expanded); p.ld0 = H;
  p.status = status;
  // blocks of W1[e] are (j/128, h/128): k-block stride = H/128, n-block stride = 1
  Scales sc = {dz_scale, 2 * I / 128, w1_scale, (long long)(2 * I / 128) * (H / 128), 1, H / 128};
  return launch<false, true, EPI_STORE>(tmA, tmB, p, sc, static_cast<cudaStream_t>(stream));
}

/* ---- power-of-two (UE8M0) block scales, applied by the tensor cores ---------------------------------- */

int smoe_mxfp8_scale_row_bytes(int cols) { return cols <= 0 ? 0 : 4 * ((cols / 128 + 3) / 4); }

int smoe_mxfp8_quantize_rows(const void* x, void* q, void* scale, long long rows, int cols, void* stream) {
  if (rows < 0 || cols <= 0 || (cols % 128) != 0) return SMOE_ERR_SHAPE;
  if (rows == 0) return SMOE_OK;
  if ((reinterpret_cast<uintptr_t>(scale) & 3u) != 0) return SMOE_ERR_ALIGNMENT;
  const int ld = smoe_mxfp8_scale_row_bytes(cols);
  const long long warps = rows * (ld / 4);
  quantize_rows_kernel<true><<<static_cast<unsigned>((warps + 7) / 8), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(x), static_cast<uint8_t*>(q), scale, rows, cols, ld);
  return cudaGetLastError() == cudaSuccess ? SMOE_OK : SMOE_ERR_LAUNCH;
}

int smoe_mxfp8_quantize_blocks(const void* w, void* q, void* scale, int batch, int rows, int cols, void* stream) {
  if (batch <= 0 || rows <= 0 || cols <= 0 || (cols % 128) != 0) return SMOE_ERR_SHAPE;
  const dim3 grid(cols / 128, (rows + 127) / 128, batch);
  quantize_blocks_kernel<true><<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(w), static_cast<uint8_t*>(q), scale, rows, cols);
  return cudaGetLastError() == cudaSuccess ? SMOE_OK : SMOE_ERR_LAUNCH;
}

static mx8::ScaleBytes mx_scales(const void* a, int a_cols, const void* b, long long b_expert, long long b_n,
                                 long long b_k) {
  mx8::ScaleBytes sc;
  sc.a = static_cast<const uint32_t*>(a);
  sc.a_ld = smoe_mxfp8_scale_row_bytes(a_cols) / 4;
  sc.b = static_cast<const uint8_t*>(b);
  sc.b_expert_stride = b_expert;
  sc.b_n_stride = b_n;
  sc.b_k_stride = b_k;
  return sc;
}

int smoe_mxfp8_up_projection_forward(const void* xq, const void* x_scale, const void* w1q, const void* w1_scale,
                                     void* z, void* y1, const int* expert_offset, const int* x_gather_idx, int T,
                                     int H, int I, int E, int TK, int* status, void* stream) {
  if (bad_shape(H, I, E) || bad_tokens(T, TK)) return SMOE_ERR_SHAPE;
  if (TK == 0) return SMOE_OK;
  CUtensorMap tmA, tmB;
  SMOE_TRY(encode_u8(&tmA, xq, T, H, 1, BK));
  SMOE_TRY(encode_u8(&tmB, w1q, (uint64_t)E * 2 * I, H, BN_CTA, BK));
  GemmParams p = {};
  p.E = E; p.N = 2 * I; p.K = H; p.total_rows = TK; p.gather_rows = T; p.b_rows_per_expert = 2 * I;
  p.off = expert_offset; p.gather = x_gather_idx;
  p.out0 = static_cast<__nv_bfloat16*>(z); p.ld0 = 2 * I;
  p.out1 = static_cast<__nv_bfloat16*>(y1); p.ld1 = I;
  p.status = status;
  const mx8::ScaleBytes sc = mx_scales(x_scale, H, w1_scale, (long long)(2 * I / 128) * (H / 128), H / 128, 1);
  return launch_mx<true, false, EPI_SWIGLU>(tmA, tmB, p, sc, static_cast<cudaStream_t>(stream));
}

int smoe_mxfp8_up_projection_forward_q(const void* xq, const void* x_scale, const void* w1q, const void* w1_scale,
                                       void* z, void* y1q, void* y1_scale, const int* expert_offset,
                                       const int* x_gather_idx, int T, int H, int I, int E, int TK, int* status,
                                       void* stream) {
  if (bad_shape(H, I, E) || bad_tokens(T, TK)) return SMOE_ERR_SHAPE;
  if (TK == 0) return SMOE_OK;  // nothing to write: the (empty) output buffers may be null
  if (y1q == nullptr || y1_scale == nullptr) return SMOE_ERR_SHAPE;
  CUtensorMap tmA, tmB;
  SMOE_TRY(encode_u8(&tmA, xq, T, H, 1, BK));
  SMOE_TRY(encode_u8(&tmB, w1q, (uint64_t)E * 2 * I, H, BN_CTA, BK));
  GemmParams p = {};
  p.E = E; p.N = 2 * I; p.K = H; p.total_rows = TK; p.gather_rows = T; p.b_rows_per_expert = 2 * I;
  p.off = expert_offset; p.gather = x_gather_idx;
  p.out0 = static_cast<__nv_bfloat16*>(z); p.ld0 = 2 * I;
  p.q_out = static_cast<uint8_t*>(y1q); p.q_scale = static_cast<uint8_t*>(y1_scale);
  p.q_scale_ld = smoe_mxfp8_scale_row_bytes(I);
  p.status = status;
  const mx8::ScaleBytes sc = mx_scales(x_scale, H, w1_scale, (long long)(2 * I / 128) * (H / 128), H / 128, 1);
  return launch_mx<true, false, EPI_SWIGLU>(tmA, tmB, p, sc, static_cast<cudaStream_t>(stream));
}

int smoe_mxfp8_down_projection_forward(const void* y1q, const void* y1_scale, const void* w2q, const void* w2_scale,
                                       void* y2, const int* expert_offset, int H, int I, int E, int TK, int* status,
                                       void* stream) {
  if (bad_shape(H, I, E) || TK < 0) return SMOE_ERR_SHAPE;
  if (TK == 0) return SMOE_OK;
  CUtensorMap tmA, tmB;
  SMOE_TRY(encode_u8(&tmA, y1q, TK, I, BM, BK));
  SMOE_TRY(encode_u8(&tmB, w2q, (uint64_t)E * H, I, BN_CTA, BK));
  GemmParams p = {};
  p.E = E; p.N = H; p.K = I; p.total_rows = TK; p.b_rows_per_expert = H;
  p.off = expert_offset;
  p.out0 = static_cast<__nv_bfloat16*>(y2); p.ld0 = H;
  p.status = status;
  const mx8::ScaleBytes sc = mx_scales(y1_scale, I, w2_scale, (long long)(H / 128) * (I / 128), I / 128, 1);
  return launch_mx<false, false, EPI_STORE>(tmA, tmB, p, sc, static_cast<cudaStream_t>(stream));
}

int smoe_mxfp8_down_projection_forward_rows(const void* y1q, const void* y1_scale, const void* w2q,
                                            const void* w2_scale, void* o, const void* scores, int scores_are_bf16,
                                            const int* expert_offset, const int* x_gather_idx,
                                            const int* s_scatter_idx, int H, int I, int E, int TK, int* status,
                                            void* stream) {
  if (bad_shape(H, I, E) || TK < 0) return SMOE_ERR_SHAPE;
  if (TK == 0) return SMOE_OK;
  if (x_gather_idx == nullptr || (scores != nullptr && s_scatter_idx == nullptr)) return SMOE_ERR_SHAPE;
  CUtensorMap tmA, tmB;
  SMOE_TRY(encode_u8(&tmA, y1q, TK, I, BM, BK));
  SMOE_TRY(encode_u8(&tmB, w2q, (uint64_t)E * H, I, BN_CTA, BK));
  GemmParams p = {};
  p.E = E; p.N = H; p.K = I; p.total_rows = TK; p.b_rows_per_expert = H;
  p.off = expert_offset; p.gather = x_gather_idx; p.s_scatter = s_scatter_idx;
  p.scores = scores; p.scores_are_bf16 = scores_are_bf16;
  p.out0 = static_cast<__nv_bfloat16*>(o); p.ld0 = H;
  p.status = status;
  const mx8::ScaleBytes sc = mx_scales(y1_scale, I, w2_scale, (long long)(H / 128) * (I / 128), I / 128, 1);
  return launch_mx<false, false, EPI_STORE_ROWS>(tmA, tmB, p, sc, static_cast<cudaStream_t>(stream));
}

int smoe_mxfp8_up_projection_backward_dx_rows(const void* dzq, const void* dz_scale, const void* w1q,
                                              const void* w1_scale, void* dx, const int* expert_offset,
                                              const int* x_gather_idx, int H, int I, int E, int TK, int* status,
                                              void* stream) {
  if (bad_shape(H, I, E) || TK < 0) return SMOE_ERR_SHAPE;
  if (TK == 0) return SMOE_OK;
  if (x_gather_idx == nullptr) return SMOE_ERR_SHAPE;
  CUtensorMap tmA, tmB;
  SMOE_TRY(encode_u8(&tmA, dzq, TK, 2 * I, BM, BK));
  SMOE_TRY(encode_u8(&tmB, w1q, (uint64_t)E * 2 * I, H, BK, BN_CTA));  // W1[e] (2I, H): rows are k
  GemmParams p = {};
  p.E = E; p.N = H; p.K = 2 * I; p.total_rows = TK; p.b_rows_per_expert = 2 * I;
  p.off = expert_offset; p.gather = x_gather_idx;
  p.out0 = static_cast<__nv_bfloat16*>(dx); p.ld0 = H;
  p.status = status;
  const mx8::ScaleBytes sc = mx_scales(dz_scale, 2 * I, w1_scale, (long long)(2 * I / 128) * (H / 128), 1, H / 128);
  return launch_mx<false, true, EPI_STORE_ROWS>(tmA, tmB, p, sc, static_cast<cudaStream_t>(stream));
}

static int mxfp8_dh(void* dzq, void* dz_scale, const void* doutq, const void* dout_scale, const void* w2q,
                                            const void* w2_scale, const void* z, const void* scores,
                                            int scores_are_bf16, void* dz, void* y1s, float* ds_partial,
                                            const int* expert_offset, const int* x_gather_idx,
                                            const int* s_scatter_idx, int T, int H, int I, int E, int TK, int* status,
                                            void* stream) {
  if (bad_shape(H, I, E) || bad_tokens(T, TK)) return SMOE_ERR_SHAPE;
  if (TK == 0) return SMOE_OK;
  CUtensorMap tmA, tmB;
  SMOE_TRY(encode_u8(&tmA, doutq, T, H, 1, BK));
  SMOE_TRY(encode_u8(&tmB, w2q, (uint64_t)E * H, I, BK, BN_CTA));  // W2[e] (H, I): rows are k
  GemmParams p = {};
  p.E = E; p.N = I; p.K = H; p.total_rows = TK; p.gather_rows = T; p.b_rows_per_expert = H;
  p.off = expert_offset; p.gather = x_gather_idx; p.s_scatter = s_scatter_idx;
  p.out0 = static_cast<__nv_bfloat16*>(dz); p.ld0 = 2 * I;
  p.out1 = static_cast<__nv_bfloat16*>(y1s); p.ld1 = I;
  p.z = static_cast<const __nv_bfloat16*>(z);
  p.scores = scores; p.scores_are_bf16 = scores_are_bf16; p.ds_partial = ds_partial;
  p.status = status;
  p.q_out = static_cast<uint8_t*>(dzq); p.q_scale = static_cast<uint8_t*>(dz_scale);
  p.q_scale_ld = smoe_mxfp8_scale_row_bytes(2 * I);
  const mx8::ScaleBytes sc = mx_scales(dout_scale, H, w2_scale, (long long)(H / 128) * (I / 128), 1, I / 128);
  return launch_mx<true, true, EPI_DSWIGLU>(tmA, tmB, p, sc, static_cast<cudaStream_t>(stream));
}

int smoe_mxfp8_down_projection_backward_act(const void* doutq, const void* dout_scale, const void* w2q,
                                            const void* w2_scale, const void* z, const void* scores,
                                            int scores_are_bf16, void* dz, void* y1s, float* ds_partial,
                                            const int* expert_offset, const int* x_gather_idx,
                                            const int* s_scatter_idx, int T, int H, int I, int E, int TK, int* status,
                                            void* stream) {
  return mxfp8_dh(nullptr, nullptr, doutq, dout_scale, w2q, w2_scale, z, scores, scores_are_bf16, dz, y1s, ds_partial,
                  expert_offset, x_gather_idx, s_scatter_idx, T, H, I, E, TK, status, stream);
}

int smoe_mxfp8_down_projection_backward_act_q(const void* doutq, const void* dout_scale, const void* w2q,
                                              const void* w2_scale, const void* z, const void* scores,
                                              int scores_are_bf16, void* dz, void* y1s, float* ds_partial, void* dzq,
                                              void* dz_scale, const int* expert_offset, const int* x_gather_idx,
                                              const int* s_scatter_idx, int T, int H, int I, int E, int TK,
                                              int* status, void* stream) {
  if (TK > 0 && (dzq == nullptr || dz_scale == nullptr)) return SMOE_ERR_SHAPE;
  return mxfp8_dh(dzq, dz_scale, doutq, dout_scale, w2q, w2_scale, z, scores, scores_are_bf16, dz, y1s, ds_partial,
                  expert_offset, x_gather_idx, s_scatter_idx, T, H, I, E, TK, status, stream);
}

int smoe_mxfp8_up_projection_backward_dx(const void* dzq, const void* dz_scale, const void* w1q, const void* w1_scale,
                                         void* dx_expanded, const int* expert_offset, int H, int I, int E, int TK,
                                         int* status, void* stream) {
  if (bad_shape(H, I, E) || TK < 0) return SMOE_ERR_SHAPE;
  if (TK == 0) return SMOE_OK;
  CUtensorMap tmA, tmB;
  SMOE_TRY(encode_u8(&tmA, dzq, TK, 2 * I, BM, BK));
  SMOE_TRY(encode_u8(&tmB, w1q, (uint64_t)E * 2 * I, H, BK, BN_CTA));  // W1[e] (2I, H): rows are k
  GemmParams p = {};
  p.E = E; p.N = H; p.K = 2 * I; p.total_rows = TK; p.b_rows_per_expert = 2 * I;
  p.off = expert_offset;
  p.out0 = static_cast<__nv_bfloat16*>(dx_expanded); p.ld0 = H;
  p.status = status;
  const mx8::ScaleBytes sc = mx_scales(dz_scale, 2 * I, w1_scale, (long long)(2 * I / 128) * (H / 128), 1, H / 128);
  return launch_mx<false, true, EPI_STORE>(tmA, tmB, p, sc, static_cast<cudaStream_t>(stream));
}

}  // extern "C"

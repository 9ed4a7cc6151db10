// Host side of the grouped GEMMs: tensor-map construction and the C-ABI launchers.
#include "device_cache.cuh"
#include "gemm_pair.cuh"

#include <cstdlib>
#include <mutex>

#include "../../include/sonicmoe_b200.h"

namespace smoe {

using pair::BK;
using pair::BM;
using pair::BN;
using pair::MAX_EXPERTS;

// cuTensorMapEncodeTiled is fetched through the runtime so that the library links against cudart
// only and still loads on a machine without a driver.
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
        q == cudaDriverEntryPointSuccess) {
      fn = reinterpret_cast<EncodeTiledFn>(ptr);
    }
  });
  return fn;
}

// bf16 row-major 2D tensor (rows, cols) with a row pitch in elements; box = (box_rows, box_cols),
// 128-byte swizzle, out-of-bounds elements read as zero.
static int encode_2d(CUtensorMap* map, const void* base, uint64_t rows, uint64_t cols, uint64_t pitch_elems,
                     uint32_t box_rows, uint32_t box_cols) {
  EncodeTiledFn fn = get_encode_fn();
  if (fn == nullptr) return SMOE_ERR_DRIVER;
  // The encoder is a driver-API call and needs the device's primary context current on the calling
  // thread; a thread that has made no runtime call yet (an autograd worker) has none.  A no-op runtime
  // call binds it.
  static thread_local bool context_bound = false;
  if (!context_bound) {
    if (cudaFree(nullptr) != cudaSuccess) return SMOE_ERR_DRIVER;
    context_bound = true;
  }
  if ((reinterpret_cast<uintptr_t>(base) & 15u) != 0 || (pitch_elems * 2) % 16 != 0) return SMOE_ERR_ALIGNMENT;
  const cuuint64_t dims[2] = {cols, rows};
  const cuuint64_t strides[1] = {pitch_elems * 2};
  const cuuint32_t box[2] = {box_cols, box_rows};
  const cuuint32_t estr[2] = {1, 1};
  const CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? SMOE_OK : SMOE_ERR_TENSORMAP;
}

// Kernels with a gathered operand work on two tiles per gathered stage (256 x 512 or 512 x 256 units) unless
// SMOE_DUAL=0 (kept for the test that compares the two forms).
static bool use_dual_tiles() {
  static const bool v = [] {
    const char* e = getenv("SMOE_DUAL");
    return !(e != nullptr && e[0] == '0');
  }();
  return v;
}

template <bool RAGGED_K, bool A_GATHER, bool A_MN, bool B_GATHER, bool B_MN, int EPI, int EW, int GW,
          int DUAL = pair::DUAL_NONE>
static int launch_variant(const CUtensorMap& tmA, const CUtensorMap& tmB, const GemmParams& p, cudaStream_t stream) {
  auto kernel = pair::grouped_gemm_pair_kernel<RAGGED_K, A_GATHER, A_MN, B_GATHER, B_MN, EPI, EW, GW, DUAL>;
  static PerDeviceFlag configured;
  const int dev = current_device();
  if (dev < 0) return SMOE_ERR_DRIVER;
  if (!configured.test(dev)) {
    if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, pair::SMEM_BYTES) != cudaSuccess)
      return SMOE_ERR_LAUNCH;
    if (DUAL != pair::DUAL_NONE) {
      // the kernel re-partitions registers between its warpgroups (setmaxnreg 56 / 200 around 128): that only
      // balances if it was compiled to exactly 128 registers per thread -- refuse to launch otherwise
      cudaFuncAttributes fa;
      if (cudaFuncGetAttributes(&fa, kernel) != cudaSuccess || fa.numRegs != 128) return SMOE_ERR_LAUNCH;
    }
    configured.set(dev);
  }
  const int sms = num_sms();
  if (sms < 2) return SMOE_ERR_DRIVER;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(static_cast<unsigned>(sms & ~1), 1, 1);
  cfg.blockDim = dim3(pair::threads(EW, GW, DUAL != pair::DUAL_NONE), 1, 1);
  cfg.dynamicSmemBytes = pair::SMEM_BYTES;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kernel, tmA, tmB, p) == cudaSuccess ? SMOE_OK : SMOE_ERR_LAUNCH;
}

// Kernels without a gathered operand: 4 epilogue warps.  Kernels with one: dual tiles (8 epilogue + 4 gather
// warps) where they pay, else single tiles with 4 epilogue + 8 gather warps.
template <bool RAGGED_K, bool A_GATHER, bool A_MN, bool B_GATHER, bool B_MN, int EPI>
static int launch(const CUtensorMap& tmA, const CUtensorMap& tmB, const GemmParams& p, cudaStream_t stream) {
  constexpr bool kGather = A_GATHER || B_GATHER;
  if constexpr (!kGather) {
    return launch_variant<RAGGED_K, A_GATHER, A_MN, B_GATHER, B_MN, EPI, 4, 0>(tmA, tmB, p, stream);
  } else {
    // not when the doubled dimension is so far from a multiple of 512 that the half-empty last unit wastes more
    // than an eighth of the MMA work (e.g. N = 768)
    const int doubled = A_GATHER ? p.N : p.M;
    const bool fits = ((doubled + 511) / 512 * 512 - doubled) * 8 <= doubled;
    // The activation-gradient epilogues keep single tiles: with both accumulators belonging to one unit the next
    // unit's second MMA group waits for the first accumulator's dSwiGLU pass.  Measured at the benchmark shape with
    // that pass staged through shared memory like the single-tile one: step 17.75-17.97 ms dual against 17.88-18.13 ms
    // single in alternating runs, the kernel alone 2.26-2.69 against 2.09-2.58 ms -- no gain worth a second variant.
    if constexpr (EPI != EPI_DSWIGLU && EPI != EPI_DACT) {
    if (use_dual_tiles() && fits) {
      constexpr int kDual = A_GATHER ? pair::DUAL_N : pair::DUAL_M;
      return launch_variant<RAGGED_K, A_GATHER, A_MN, B_GATHER, B_MN, EPI, 8, 4, kDual>(tmA, tmB, p, stream);
    }
    }
    return launch_variant<RAGGED_K, A_GATHER, A_MN, B_GATHER, B_MN, EPI, 4, 8>(tmA, tmB, p, stream);
  }
}

// An empty batch (T == 0, hence TK == 0) is valid: the entry points return at once (weight-gradient entry points
// after zero-filling their output).  What is refused: negative sizes, or routed rows without any token.
static bool bad_tokens(int T, int TK) { return T < 0 || TK < 0 || (T == 0 && TK > 0); }

static bool bad_shape(int H, int I, int E) {
  return H <= 0 || I <= 0 || E <= 0 || E > MAX_EXPERTS || (H % 64) != 0 || (I % 64) != 0;
}

}  // namespace smoe

using namespace smoe;

#define SMOE_TRY(expr)              \
  do {                              \
    const int _rc = (expr);         \
    if (_rc != SMOE_OK) return _rc; \
  } while (0)

extern "C" {

int smoe_up_projection_forward(const void* x, const void* w1, void* z, void* y1, const int* expert_offset,
                               const int* x_gather_idx, int T, int H, int I, int E, int TK, int* status,
                               void* stream) {
  if (bad_shape(H, I, E) || bad_tokens(T, TK)) return SMOE_ERR_SHAPE;
  if (TK == 0) return SMOE_OK;
  CUtensorMap tmA, tmB;
  SMOE_TRY(encode_2d(&tmA, x, T, H, H, 1, BK));                        // gather4 rows of x
  SMOE_TRY(encode_2d(&tmB, w1, (uint64_t)E * 2 * I, H, H, pair::BN_CTA, BK));    // W1[e] rows = output features, K-major
  GemmParams p = {};
  p.E = E; p.N = 2 * I; p.K = H; p.total_rows = TK; p.gather_rows = T; p.b_rows_per_expert = 2 * I;
  p.off = expert_offset; p.gather = x_gather_idx;
  p.out0 = static_cast<__nv_bfloat16*>(z); p.ld0 = 2 * I;
  p.out1 = static_cast<__nv_bfloat16*>(y1); p.ld1 = I;
  p.status = status;
  return launch<false, true, false, false, false, EPI_SWIGLU>(tmA, tmB, p, static_cast<cudaStream_t>(stream));
}

int smoe_down_projection_forward(const void* y1, const void* w2, void* y2, const int* expert_offset, int H, int I,
                                 int E, int TK, int* status, void* stream) {
  if (bad_shape(H, I, E) || TK < 0) return SMOE_ERR_SHAPE;
  if (TK == 0) return SMOE_OK;
  CUtensorMap tmA, tmB;
  SMOE_TRY(encode_2d(&tmA, y1, TK, I, I, BM, BK));
  SMOE_TRY(encode_2d(&tmB, w2, (uint64_t)E * H, I, I, pair::BN_CTA, BK));        // W2[e] is (H, I): K-major
  GemmParams p = {};
  p.E = E; p.N = H; p.K = I; p.total_rows = TK; p.b_rows_per_expert = H;
  p.off = expert_offset;
  p.out0 = static_cast<__nv_bfloat16*>(y2); p.ld0 = H;
  p.status = status;
  return launch<false, false, false, false, false, EPI_STORE>(tmA, tmB, p, static_cast<cudaStream_t>(stream));
}

int smoe_down_projection_forward_rows(const void* y1, const void* w2, void* o, const void* scores, int scores_are_bf16,
                                      const int* expert_offset, const int* x_gather_idx, const int* s_scatter_idx,
                                      int H, int I, int E, int TK, int* status, void* stream) {
  if (bad_shape(H, I, E) || TK < 0) return SMOE_ERR_SHAPE;
  if (TK == 0) return SMOE_OK;
  if (x_gather_idx == nullptr || (scores != nullptr && s_scatter_idx == nullptr)) return SMOE_ERR_SHAPE;
  CUtensorMap tmA, tmB;
  SMOE_TRY(encode_2d(&tmA, y1, TK, I, I, BM, BK));
  SMOE_TRY(encode_2d(&tmB, w2, (uint64_t)E * H, I, I, pair::BN_CTA, BK));
  GemmParams p = {};
  p.E = E; p.N = H; p.K = I; p.total_rows = TK; p.b_rows_per_expert = H;
  p.off = expert_offset; p.gather = x_gather_idx; p.s_scatter = s_scatter_idx;
  p.scores = scores; p.scores_are_bf16 = scores_are_bf16;
  p.out0 = static_cast<__nv_bfloat16*>(o); p.ld0 = H;
  p.status = status;
  return launch<false, false, false, false, false, EPI_STORE_ROWS>(tmA, tmB, p, static_cast<cudaStream_t>(stream));
}

int smoe_down_projection_forward_scatter(const void* y1, const void* w2, float* o_acc, const void* scores,
                                         int scores_are_bf16, const int* expert_offset, const int* x_gather_idx,
                                         const int* s_scatter_idx, int T, int H, int I, int E, int TK, int* status,
                                         void* stream) {
  if (bad_shape(H, I, E) || bad_tokens(T, TK)) return SMOE_ERR_SHAPE;
  if (TK == 0) return SMOE_OK;
  CUtensorMap tmA, tmB;
  SMOE_TRY(encode_2d(&tmA, y1, TK, I, I, BM, BK));
  SMOE_TRY(encode_2d(&tmB, w2, (uint64_t)E * H, I, I, pair::BN_CTA, BK));
  GemmParams p = {};
  p.E = E; p.N = H; p.K = I; p.total_rows = TK; p.gather_rows = T; p.b_rows_per_expert = H;
  p.off = expert_offset; p.gather = x_gather_idx; p.s_scatter = s_scatter_idx;
  p.scores = scores; p.scores_are_bf16 = scores_are_bf16; p.acc_out = o_acc;
  p.status = status;
  return launch<false, false, false, false, false, EPI_SCATTER>(tmA, tmB, p, static_cast<cudaStream_t>(stream));
}

int smoe_down_projection_backward_act(const void* dout, const void* w2, const void* z, const void* scores,
                                      int scores_are_bf16, void* dz, void* y1s, float* ds_partial,
                                      const int* expert_offset, const int* x_gather_idx, const int* s_scatter_idx,
                                      int T, int H, int I, int E, int TK, int* status, void* stream) {
  if (bad_shape(H, I, E) || bad_tokens(T, TK)) return SMOE_ERR_SHAPE;
  if (TK == 0) return SMOE_OK;
  CUtensorMap tmA, tmB;
  SMOE_TRY(encode_2d(&tmA, dout, T, H, H, 1, BK));                     // gather4 rows of dout
  SMOE_TRY(encode_2d(&tmB, w2, (uint64_t)E * H, I, I, BK, 64));        // W2[e] (H, I): rows are k, MN-major
  GemmParams p = {};
  p.E = E; p.N = I; p.K = H; p.total_rows = TK; p.gather_rows = T; p.b_rows_per_expert = H;
  p.off = expert_offset; p.gather = x_gather_idx; p.s_scatter = s_scatter_idx;
  p.out0 = static_cast<__nv_bfloat16*>(dz); p.ld0 = 2 * I;
  p.out1 = static_cast<__nv_bfloat16*>(y1s); p.ld1 = I;
  p.z = static_cast<const __nv_bfloat16*>(z);
  p.scores = scores; p.scores_are_bf16 = scores_are_bf16; p.ds_partial = ds_partial;
  p.status = status;
  return launch<false, true, false, false, true, EPI_DSWIGLU>(tmA, tmB, p, static_cast<cudaStream_t>(stream));
}

// ---- general activations and biases ---------------------------------------------
static bool bad_activation(int a) { return a < ACT_SWIGLU || a > ACT_SILU; }

int smoe_up_projection_forward_act(const void* x, const void* w1, const void* b1, void* z, void* y1,
                                   const int* expert_offset, const int* x_gather_idx, int T, int H, int N1, int E,
                                   int TK, int activation, int* status, void* stream) {
  if (bad_activation(activation) || H <= 0 || (H % 64) != 0 || N1 <= 0 || (N1 % 128) != 0 || E <= 0 ||
      E > MAX_EXPERTS || bad_tokens(T, TK))
    return SMOE_ERR_SHAPE;
  if (TK == 0) return SMOE_OK;
  CUtensorMap tmA, tmB;
  SMOE_TRY(encode_2d(&tmA, x, T, H, H, 1, BK));
  SMOE_TRY(encode_2d(&tmB, w1, (uint64_t)E * N1, H, H, pair::BN_CTA, BK));
  GemmParams p = {};
  p.E = E; p.N = N1; p.K = H; p.total_rows = TK; p.gather_rows = T; p.b_rows_per_expert = N1;
  p.off = expert_offset; p.gather = x_gather_idx;
  p.out0 = static_cast<__nv_bfloat16*>(z); p.ld0 = N1;
  p.out1 = static_cast<__nv_bfloat16*>(y1); p.ld1 = act_is_gated(activation) ? N1 / 2 : N1;
  p.bias = static_cast<const __nv_bfloat16*>(b1); p.act = activation;
  p.status = status;
  return launch<false, true, false, false, false, EPI_ACT>(tmA, tmB, p, static_cast<cudaStream_t>(stream));
}

int smoe_down_projection_forward_bias(const void* y1, const void* w2, const void* b2, void* y2,
                                      const int* expert_offset, int H, int I, int E, int TK, int* status,
                                      void* stream) {
  if (bad_shape(H, I, E) || TK < 0) return SMOE_ERR_SHAPE;
  if (TK == 0) return SMOE_OK;
  CUtensorMap tmA, tmB;
  SMOE_TRY(encode_2d(&tmA, y1, TK, I, I, BM, BK));
  SMOE_TRY(encode_2d(&tmB, w2, (uint64_t)E * H, I, I, pair::BN_CTA, BK));
  GemmParams p = {};
  p.E = E; p.N = H; p.K = I; p.total_rows = TK; p.b_rows_per_expert = H;
  p.off = expert_offset;
  p.out0 = static_cast<__nv_bfloat16*>(y2); p.ld0 = H;
  p.bias = static_cast<const __nv_bfloat16*>(b2);
  p.status = status;
  return launch<false, false, false, false, false, EPI_STORE_BIAS>(tmA, tmB, p,
                                                                        static_cast<cudaStream_t>(stream));
}

int smoe_down_projection_backward_dact(const void* dout, const void* w2, const void* z, const void* scores,
                                       int scores_are_bf16, void* dz, void* y1s, float* ds_partial,
                                       const int* expert_offset, const int* x_gather_idx, const int* s_scatter_idx,
                                       int T, int H, int I, int E, int TK, int activation, int* status,
                                       void* stream) {
  if (bad_activation(activation) || bad_shape(H, I, E) || bad_tokens(T, TK)) return SMOE_ERR_SHAPE;
  if (TK == 0) return SMOE_OK;
  CUtensorMap tmA, tmB;
  SMOE_TRY(encode_2d(&tmA, dout, T, H, H, 1, BK));
  SMOE_TRY(encode_2d(&tmB, w2, (uint64_t)E * H, I, I, BK, 64));
  const int n1 = act_is_gated(activation) ? 2 * I : I;
  GemmParams p = {};
  p.E = E; p.N = I; p.K = H; p.total_rows = TK; p.gather_rows = T; p.b_rows_per_expert = H;
  p.off = expert_offset; p.gather = x_gather_idx; p.s_scatter = s_scatter_idx;
  p.out0 = static_cast<__nv_bfloat16*>(dz); p.ld0 = n1;
  p.out1 = static_cast<__nv_bfloat16*>(y1s); p.ld1 = I;
  p.z = static_cast<const __nv_bfloat16*>(z);
  p.scores = scores; p.scores_are_bf16 = scores_are_bf16; p.ds_partial = ds_partial;
  p.act = activation;
  p.status = status;
  return launch<false, true, false, false, true, EPI_DACT>(tmA, tmB, p, static_cast<cudaStream_t>(stream));
}

int smoe_ds_partial_columns(int I) { return 2 * ((I + BN - 1) / BN); }

int smoe_up_projection_backward_dx(const void* dz, const void* w1, void* dx_expanded, const int* expert_offset, int H,
                                   int I, int E, int TK, int* status, void* stream) {
  if (bad_shape(H, I, E) || TK < 0) return SMOE_ERR_SHAPE;
  if (TK == 0) return SMOE_OK;
  CUtensorMap tmA, tmB;
  SMOE_TRY(encode_2d(&tmA, dz, TK, 2 * I, 2 * I, BM, BK));
  SMOE_TRY(encode_2d(&tmB, w1, (uint64_t)E * 2 * I, H, H, BK, 64));    // W1[e] (2I, H): rows are k, MN-major
  GemmParams p = {};
  p.E = E; p.N = H; p.K = 2 * I; p.total_rows = TK; p.b_rows_per_expert = 2 * I;
  p.off = expert_offset;
  p.out0 = static_cast<__nv_bfloat16*>(dx_expanded); p.ld0 = H;
  p.status = status;
  return launch<false, false, false, false, true, EPI_STORE>(tmA, tmB, p, static_cast<cudaStream_t>(stream));
}

int smoe_up_projection_backward_dx_rows(const void* dz, const void* w1, void* dx, const int* expert_offset,
                                        const int* x_gather_idx, int H, int I, int E, int TK, int* status,
                                        void* stream) {
  if (bad_shape(H, I, E) || TK < 0) return SMOE_ERR_SHAPE;
  if (TK == 0) return SMOE_OK;
  if (x_gather_idx == nullptr) return SMOE_ERR_SHAPE;
  CUtensorMap tmA, tmB;
  SMOE_TRY(encode_2d(&tmA, dz, TK, 2 * I, 2 * I, BM, BK));
  SMOE_TRY(encode_2d(&tmB, w1, (uint64_t)E * 2 * I, H, H, BK, 64));    // W1[e] (2I, H): rows are k, MN-major
  GemmParams p = {};
  p.E = E; p.N = H; p.K = 2 * I; p.total_rows = TK; p.b_rows_per_expert = 2 * I;
  p.off = expert_offset; p.gather = x_gather_idx;
  p.out0 = static_cast<__nv_bfloat16*>(dx); p.ld0 = H;
  p.status = status;
  return launch<false, false, false, false, true, EPI_STORE_ROWS>(tmA, tmB, p, static_cast<cudaStream_t>(stream));
}

static int down_weight_grad(const void* dout, const void* y1s, void* dw2, const int* expert_offset,
                            const int* x_gather_idx, int T, int H, int I, int E, int TK, int* status, void* stream,
                            int accumulate) {
  if (bad_shape(H, I, E) || bad_tokens(T, TK)) return SMOE_ERR_SHAPE;
  if (TK == 0) {
    if (accumulate) return SMOE_OK;
    return cudaMemsetAsync(dw2, 0, (size_t)E * H * I * 2, static_cast<cudaStream_t>(stream)) == cudaSuccess
               ? SMOE_OK : SMOE_ERR_LAUNCH;
  }
  CUtensorMap tmA, tmB;
  SMOE_TRY(encode_2d(&tmA, dout, T, H, H, 1, 64));                     // A[h, t] = dout[gather[t], h]
  SMOE_TRY(encode_2d(&tmB, y1s, TK, I, I, BK, 64));                    // B[i, t] = y1s[t, i]
  GemmParams p = {};
  p.E = E; p.M = H; p.N = I; p.total_rows = TK; p.gather_rows = T;
  p.off = expert_offset; p.gather = x_gather_idx;
  p.out0 = static_cast<__nv_bfloat16*>(dw2); p.ld0 = I; p.out0_expert_stride = (long long)H * I;
  p.status = status; p.accumulate = accumulate;
  return launch<true, true, true, false, true, EPI_STORE>(tmA, tmB, p, static_cast<cudaStream_t>(stream));
}

static int up_weight_grad(const void* x, const void* dz, void* dw1, const int* expert_offset, const int* x_gather_idx,
                          int T, int H, int I, int E, int TK, int* status, void* stream, int accumulate) {
  if (bad_shape(H, I, E) || bad_tokens(T, TK)) return SMOE_ERR_SHAPE;
  if (TK == 0) {
    if (accumulate) return SMOE_OK;
    return cudaMemsetAsync(dw1, 0, (size_t)E * 2 * I * H * 2, static_cast<cudaStream_t>(stream)) == cudaSuccess
               ? SMOE_OK : SMOE_ERR_LAUNCH;
  }
  CUtensorMap tmA, tmB;
  SMOE_TRY(encode_2d(&tmA, dz, TK, 2 * I, 2 * I, BK, 64));             // A[j, t] = dz[t, j]
  SMOE_TRY(encode_2d(&tmB, x, T, H, H, 1, 64));                        // B[h, t] = x[gather[t], h]
  GemmParams p = {};
  p.E = E; p.M = 2 * I; p.N = H; p.total_rows = TK; p.gather_rows = T;
  p.off = expert_offset; p.gather = x_gather_idx;
  p.out0 = static_cast<__nv_bfloat16*>(dw1); p.ld0 = H; p.out0_expert_stride = (long long)2 * I * H;
  p.status = status; p.accumulate = accumulate;
  return launch<true, false, true, true, true, EPI_STORE>(tmA, tmB, p, static_cast<cudaStream_t>(stream));
}

int smoe_down_projection_weight_grad(const void* dout, const void* y1s, void* dw2, const int* expert_offset,
                                     const int* x_gather_idx, int T, int H, int I, int E, int TK, int* status,
                                     void* stream) {
  return down_weight_grad(dout, y1s, dw2, expert_offset, x_gather_idx, T, H, I, E, TK, status, stream, 0);
}

int smoe_down_projection_weight_grad_accumulate(const void* dout, const void* y1s, void* dw2,
                                                const int* expert_offset, const int* x_gather_idx, int T, int H, int I,
                                                int E, int TK, int* status, void* stream) {
  return down_weight_grad(dout, y1s, dw2, expert_offset, x_gather_idx, T, H, I, E, TK, status, stream, 1);
}

int smoe_up_projection_weight_grad(const void* x, const void* dz, void* dw1, const int* expert_offset,
                                   const int* x_gather_idx, int T, int H, int I, int E, int TK, int* status,
                                   void* stream) {
  return up_weight_grad(x, dz, dw1, expert_offset, x_gather_idx, T, H, I, E, TK, status, stream, 0);
}

int smoe_up_projection_weight_grad_accumulate(const void* x, const void* dz, void* dw1, const int* expert_offset,
                                              const int* x_gather_idx, int T, int H, int I, int E, int TK, int* status,
                                              void* stream) {
  return up_weight_grad(x, dz, dw1, expert_offset, x_gather_idx, T, H, I, E, TK, status, stream, 1);
}

}  // extern "C"

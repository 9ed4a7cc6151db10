// Expert-parallel exchange over peer memory (NVLink / NVSwitch): buffers that the other ranks of one node map
// through CUDA IPC, a gather-and-sum kernel whose OUTPUT rows go straight into those buffers with peer stores
// (the dispatch of routed token rows and the return of per-token partial sums are fused with the row gather /
// the reduction that produces them: no staging copy, every row crosses the link once), and copy-engine copies
// for segments that are already contiguous.  Plain peer loads and stores only: no multicast of any kind.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <string.h>

#include <mutex>

#include "../../include/sonicmoe_b200.h"

namespace smoe {

static inline int rc_of(cudaError_t e) { return e == cudaSuccess ? SMOE_OK : SMOE_ERR_DRIVER; }

// Stream memory operations of the driver (a 32-bit write / a wait for a 32-bit value, executed by the stream itself:
// no kernel, no multiprocessor), resolved at run time so that the library links against the CUDA runtime only.
using StreamWrite32Fn = CUresult (*)(CUstream, CUdeviceptr, cuuint32_t, unsigned int);
using StreamWait32Fn = CUresult (*)(CUstream, CUdeviceptr, cuuint32_t, unsigned int);

struct StreamMemOps {
  StreamWrite32Fn write = nullptr;
  StreamWait32Fn wait = nullptr;
};

static const StreamMemOps& stream_mem_ops() {
  static StreamMemOps ops;
  static std::once_flag once;
  std::call_once(once, [] {
    void* w = nullptr;
    void* q = nullptr;
    cudaDriverEntryPointQueryResult rw, rq;
    if (cudaGetDriverEntryPoint("cuStreamWriteValue32", &w, cudaEnableDefault, &rw) == cudaSuccess &&
        rw == cudaDriverEntryPointSuccess &&
        cudaGetDriverEntryPoint("cuStreamWaitValue32", &q, cudaEnableDefault, &rq) == cudaSuccess &&
        rq == cudaDriverEntryPointSuccess) {
      ops.write = reinterpret_cast<StreamWrite32Fn>(w);
      ops.wait = reinterpret_cast<StreamWait32Fn>(q);
    } else {
      cudaGetLastError();
    }
  });
  return ops;
}

struct PeerSegments {
  __nv_bfloat16* ptr[SMOE_MAX_PEERS];  // where segment s starts (in whichever GPU's memory)
  int start[SMOE_MAX_PEERS + 1];       // first output row of segment s; start[n] = number of output rows
  int n;
};

// out_s[t - start[s], :] = sum_{p in [tok_off[t], tok_off[t+1])} w[p] * src[rev[p], :]  for the segment s that
// holds output row t (tok_off == nullptr: fixed K rows per output row; w == nullptr: plain sum).
// One thread per 8 consecutive columns of one output row, fp32 accumulation, 16-byte stores (peer or local).
template <typename W>
__global__ void __launch_bounds__(256) gather_sum_to_segments_kernel(const __nv_bfloat16* __restrict__ src,
                                                                     const W* __restrict__ w,
                                                                     const int* __restrict__ rev,
                                                                     const int* __restrict__ tok_off, int T, int H,
                                                                     int K, int first_row, const PeerSegments seg) {
  const int vec_per_row = H >> 3;
  const long long g = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (g >= static_cast<long long>(T) * vec_per_row) return;
  // the grid walks the output rows starting at first_row and wrapping around: ranks that all start with the segment
  // of their right-hand neighbour never write to the same destination at the same time
  int t = static_cast<int>(g / vec_per_row) + first_row;
  if (t >= T) t -= T;
  const int c = static_cast<int>(g % vec_per_row);
  int s = 0;
  while (s + 1 < seg.n && t >= seg.start[s + 1]) ++s;
  int p0, p1;
  if (tok_off != nullptr) { p0 = tok_off[t]; p1 = tok_off[t + 1]; } else { p0 = t * K; p1 = p0 + K; }
  uint4 o;
  if (p1 - p0 == 1 && w == nullptr) {  // a pure row move: no arithmetic, bit-exact
    o = reinterpret_cast<const uint4*>(src + static_cast<long long>(rev[p0]) * H)[c];
  } else {
    float acc[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] = 0.f;
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
    __nv_bfloat162* oh = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
    for (int j = 0; j < 4; ++j) oh[j] = __floats2bfloat162_rn(acc[2 * j], acc[2 * j + 1]);
  }
  reinterpret_cast<uint4*>(seg.ptr[s] + static_cast<long long>(t - seg.start[s]) * H)[c] = o;
}

}  // namespace smoe

using namespace smoe;

extern "C" {

int smoe_peer_alloc(size_t bytes, void** ptr) {
  if (ptr == nullptr || bytes == 0) return SMOE_ERR_SHAPE;
  *ptr = nullptr;
  if (cudaMalloc(ptr, bytes) != cudaSuccess) {
    cudaGetLastError();
    return SMOE_ERR_DRIVER;
  }
  return rc_of(cudaMemset(*ptr, 0, bytes));
}

int smoe_peer_free(void* ptr) { return ptr == nullptr ? SMOE_OK : rc_of(cudaFree(ptr)); }

int smoe_peer_export(const void* ptr, unsigned char* handle64) {
  if (ptr == nullptr || handle64 == nullptr) return SMOE_ERR_SHAPE;
  static_assert(sizeof(cudaIpcMemHandle_t) == SMOE_PEER_HANDLE_BYTES, "IPC handle size");
  cudaIpcMemHandle_t h;
  if (cudaIpcGetMemHandle(&h, const_cast<void*>(ptr)) != cudaSuccess) {
    cudaGetLastError();
    return SMOE_ERR_DRIVER;
  }
  memcpy(handle64, &h, sizeof(h));
  return SMOE_OK;
}

int smoe_peer_open(const unsigned char* handle64, void** ptr) {
  if (ptr == nullptr || handle64 == nullptr) return SMOE_ERR_SHAPE;
  cudaIpcMemHandle_t h;
  memcpy(&h, handle64, sizeof(h));
  *ptr = nullptr;
  if (cudaIpcOpenMemHandle(ptr, h, cudaIpcMemLazyEnablePeerAccess) != cudaSuccess) {
    cudaGetLastError();
    return SMOE_ERR_DRIVER;
  }
  return SMOE_OK;
}

int smoe_peer_close(void* ptr) { return ptr == nullptr ? SMOE_OK : rc_of(cudaIpcCloseMemHandle(ptr)); }

int smoe_peer_copy(void* dst, const void* src, size_t bytes, void* stream) {
  if (bytes == 0) return SMOE_OK;
  if (dst == nullptr || src == nullptr) return SMOE_ERR_SHAPE;
  return rc_of(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDefault, static_cast<cudaStream_t>(stream)));
}

int smoe_stream_write_value(void* addr, unsigned int value, void* stream) {
  if (addr == nullptr || (reinterpret_cast<uintptr_t>(addr) & 3u) != 0) return SMOE_ERR_ALIGNMENT;
  const StreamMemOps& ops = stream_mem_ops();
  if (ops.write == nullptr) return SMOE_ERR_DRIVER;
  return ops.write(static_cast<CUstream>(stream), reinterpret_cast<CUdeviceptr>(addr), value,
                   CU_STREAM_WRITE_VALUE_DEFAULT) == CUDA_SUCCESS ? SMOE_OK : SMOE_ERR_DRIVER;
}

int smoe_stream_wait_values(const void* addr, int count, unsigned int value, void* stream) {
  if (count < 0) return SMOE_ERR_SHAPE;
  if (count == 0) return SMOE_OK;
  if (addr == nullptr || (reinterpret_cast<uintptr_t>(addr) & 3u) != 0) return SMOE_ERR_ALIGNMENT;
  const StreamMemOps& ops = stream_mem_ops();
  if (ops.wait == nullptr) return SMOE_ERR_DRIVER;
  for (int i = 0; i < count; ++i) {
    const CUdeviceptr a = reinterpret_cast<CUdeviceptr>(addr) + 4ull * static_cast<unsigned>(i);
    if (ops.wait(static_cast<CUstream>(stream), a, value, CU_STREAM_WAIT_VALUE_GEQ) != CUDA_SUCCESS)
      return SMOE_ERR_DRIVER;
  }
  return SMOE_OK;
}

int smoe_gather_sum_to_peers(const void* src, const void* weights, int weights_dtype, const int* reverse_idx,
                             const int* token_offset, int T, int H, int K, void* const* segment_ptr,
                             const int* segment_start, int num_segments, int first_row, void* stream) {
  if (T < 0 || H <= 0 || (H % 8) != 0 || num_segments <= 0 || num_segments > SMOE_MAX_PEERS) return SMOE_ERR_SHAPE;
  if (first_row < 0 || (T > 0 && first_row >= T)) return SMOE_ERR_SHAPE;
  if (token_offset == nullptr && K <= 0) return SMOE_ERR_SHAPE;
  if (segment_ptr == nullptr || segment_start == nullptr) return SMOE_ERR_SHAPE;
  if (segment_start[0] != 0 || segment_start[num_segments] != T) return SMOE_ERR_SHAPE;
  if (T == 0) return SMOE_OK;
  PeerSegments seg = {};
  seg.n = num_segments;
  for (int s = 0; s < num_segments; ++s) {
    if (segment_start[s + 1] < segment_start[s]) return SMOE_ERR_SHAPE;
    if (segment_start[s + 1] > segment_start[s] &&
        (segment_ptr[s] == nullptr || (reinterpret_cast<uintptr_t>(segment_ptr[s]) & 15u) != 0))
      return SMOE_ERR_ALIGNMENT;
    seg.ptr[s] = static_cast<__nv_bfloat16*>(segment_ptr[s]);
    seg.start[s] = segment_start[s];
  }
  seg.start[num_segments] = T;
  const long long total = static_cast<long long>(T) * (H / 8);
  const unsigned grid = static_cast<unsigned>((total + 255) / 256);
  const __nv_bfloat16* s_ = static_cast<const __nv_bfloat16*>(src);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (weights == nullptr || weights_dtype == SMOE_F32)
    gather_sum_to_segments_kernel<float><<<grid, 256, 0, st>>>(s_, static_cast<const float*>(weights), reverse_idx,
                                                                token_offset, T, H, K, first_row, seg);
  else if (weights_dtype == SMOE_BF16)
    gather_sum_to_segments_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>(
        s_, static_cast<const __nv_bfloat16*>(weights), reverse_idx, token_offset, T, H, K, first_row, seg);
  else
    return SMOE_ERR_DTYPE;
  return cudaGetLastError() == cudaSuccess ? SMOE_OK : SMOE_ERR_LAUNCH;
}

}  // extern "C"

#include "moe_local_noalloc.h"

#include <cuda_runtime.h>

#include <mutex>

#include "../common/ptx.cuh"

namespace {

// Scratch of every call on this GPU: [0, MAX) segment starts, [MAX, 2*MAX) slot
// cursors, then spare words. In host code this name is only a stand-in for the
// device object; kernels receive the address obtained with cudaGetSymbolAddress.
static __device__ __align__(256) unsigned char g_noalloc_scratch[TDB_NOALLOC_SCRATCH_BYTES];

constexpr int kMaxDevices = 64;
std::mutex g_mu;
int32_t* g_scratch_ptr[kMaxDevices] = {};
bool g_scratch_known[kMaxDevices] = {};

// Device address of the scratch array on the current device (looked up once per device).
int scratch_for_current_device(int32_t** out) {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return TDB_NOALLOC_ECUDA;
  std::lock_guard<std::mutex> lk(g_mu);
  if (!g_scratch_known[dev]) {
    void* p = nullptr;
    if (cudaGetSymbolAddress(&p, g_noalloc_scratch) != cudaSuccess || p == nullptr) {
      cudaGetLastError();
      return TDB_NOALLOC_ECUDA;
    }
    g_scratch_ptr[dev] = reinterpret_cast<int32_t*>(p);
    g_scratch_known[dev] = true;
  }
  *out = g_scratch_ptr[dev];
  return TDB_NOALLOC_OK;
}

// One CTA: histogram of expert ids -> exclusive prefix -> segment starts; cursors cleared.
__global__ void __launch_bounds__(1024)
noalloc_plan_kernel(const int32_t* __restrict__ topk_idx, int pairs, int E, int32_t* scratch,
                    int32_t* __restrict__ seg_start, int32_t* __restrict__ recv_total) {
  __shared__ int32_t hist[TDB_NOALLOC_MAX_EXPERTS];
  const int tid = threadIdx.x;
  for (int e = tid; e < E; e += blockDim.x) hist[e] = 0;
  __syncthreads();
  for (int i = tid; i < pairs; i += blockDim.x) {
    const int e = topk_idx[i];
    if (e >= 0 && e < E) atomicAdd(&hist[e], 1);
  }
  __syncthreads();
  if (tid == 0) {
    int run = 0;
    for (int e = 0; e < E; ++e) {
      const int c = hist[e];
      hist[e] = run;
      run += c;
    }
    *recv_total = run;
  }
  __syncthreads();
  int32_t* seg = scratch;
  int32_t* cursor = scratch + TDB_NOALLOC_MAX_EXPERTS;
  for (int e = tid; e < E; e += blockDim.x) {
    seg[e] = hist[e];
    seg_start[e] = hist[e];
    cursor[e] = 0;            // the array keeps the previous call's cursors: start from zero
  }
}

// One warp per (token, k): claim a slot in the expert's segment, copy the row.
__global__ void __launch_bounds__(256)
noalloc_dispatch_kernel(const uint8_t* __restrict__ tokens, const int32_t* __restrict__ topk_idx,
                        uint8_t* __restrict__ recv, int32_t* __restrict__ scatter_idx,
                        int32_t* scratch, int pairs, int topk, int E, int64_t row_bytes,
                        int64_t max_recv_rows) {
  const int32_t* seg = scratch;
  int32_t* cursor = scratch + TDB_NOALLOC_MAX_EXPERTS;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n16 = static_cast<int>(row_bytes >> 4);
  for (int pair = blockIdx.x * 8 + warp; pair < pairs; pair += gridDim.x * 8) {
    const int t = pair / topk;
    const int e = topk_idx[pair];
    int row = -1;
    if (lane == 0) {
      if (e >= 0 && e < E) {
        row = seg[e] + atomicAdd(&cursor[e], 1);
        if (row >= max_recv_rows) row = -1;
      }
      scatter_idx[pair] = row;
    }
    row = __shfl_sync(0xFFFFFFFFu, row, 0);
    if (row < 0) continue;
    const uint8_t* src = tokens + t * row_bytes;
    uint8_t* dst = recv + row * row_bytes;
    for (int i = lane; i < n16; i += 32)
      tdb::st_global_v4(dst + (static_cast<int64_t>(i) << 4), tdb::ld_global_nc_v4(src + (static_cast<int64_t>(i) << 4)));
  }
}

}  // namespace

extern "C" int tdb_moe_local_dispatch_noalloc(const void* tokens, const int32_t* topk_idx, void* recv,
                                              int32_t* scatter_idx, int32_t* seg_start,
                                              int32_t* recv_total, int T, int H, int topk, int E,
                                              int64_t max_recv_rows, void* stream_) {
  if (!topk_idx || !scatter_idx || !seg_start || !recv_total) return TDB_NOALLOC_ENULL;
  if (E < 1 || E > TDB_NOALLOC_MAX_EXPERTS) return TDB_NOALLOC_EEXPERTS;
  if (topk < 1 || topk > 32) return TDB_NOALLOC_ETOPK;
  if (H < 8 || H % 8 != 0) return TDB_NOALLOC_EHIDDEN;
  if (T < 0) return TDB_NOALLOC_EROWS;
  const int64_t pairs64 = static_cast<int64_t>(T) * topk;
  if (pairs64 >= (1ll << 31) || max_recv_rows < pairs64) return TDB_NOALLOC_EROWS;
  if (T > 0 && (!tokens || !recv)) return TDB_NOALLOC_ENULL;
  if ((reinterpret_cast<uintptr_t>(tokens) | reinterpret_cast<uintptr_t>(recv)) & 15u) return TDB_NOALLOC_EALIGN;
  int32_t* scratch = nullptr;
  const int rc = scratch_for_current_device(&scratch);
  if (rc != TDB_NOALLOC_OK) return rc;
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  const int pairs = static_cast<int>(pairs64);
  noalloc_plan_kernel<<<1, 1024, 0, stream>>>(topk_idx, pairs, E, scratch, seg_start, recv_total);
  if (cudaGetLastError() != cudaSuccess) return TDB_NOALLOC_ECUDA;
  if (pairs > 0) {
    int grid = (pairs + 7) / 8;
    if (grid > 148 * 8) grid = 148 * 8;
    noalloc_dispatch_kernel<<<grid, 256, 0, stream>>>(
        reinterpret_cast<const uint8_t*>(tokens), topk_idx, reinterpret_cast<uint8_t*>(recv), scatter_idx,
        scratch, pairs, topk, E, static_cast<int64_t>(H) * 2, max_recv_rows);
    if (cudaGetLastError() != cudaSuccess) return TDB_NOALLOC_ECUDA;
  }
  return TDB_NOALLOC_OK;
}

extern "C" const char* tdb_noalloc_strerror(int code) {
  switch (code) {
    case TDB_NOALLOC_OK: return "ok";
    case TDB_NOALLOC_ENULL: return "a required pointer is null";
    case TDB_NOALLOC_EEXPERTS: return "number of experts must be in [1, 1024] (fixed scratch size)";
    case TDB_NOALLOC_ETOPK: return "topk must be in [1, 32]";
    case TDB_NOALLOC_EHIDDEN: return "hidden size must be a positive multiple of 8";
    case TDB_NOALLOC_EROWS: return "T * topk must be < 2^31 and recv must hold at least T * topk rows";
    case TDB_NOALLOC_ECUDA: return "a CUDA call failed (scratch symbol lookup or kernel launch)";
    case TDB_NOALLOC_EALIGN: return "tokens and recv must start on 16-byte boundaries";
    default: return "unknown code";
  }
}

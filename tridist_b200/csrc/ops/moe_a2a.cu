#include "moe_a2a.h"

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <stdexcept>
#include <string>

#include "../common/ptx.cuh"
#include "../common/sync.cuh"
#include "fused_gemm.h"

namespace tdb {

static void check(cudaError_t e, const char* what) {
  if (e != cudaSuccess)
    throw std::runtime_error(std::string("tridist_b200: ") + what + ": " + cudaGetErrorString(e));
}

// With nv > 1 one launch carries several emulated ranks: consecutive CTAs
// belong to consecutive ranks so that the first CTA of every rank is in the
// first wave (those CTAs raise the flags all others wait on).
#define TDB_MOE_PROLOGUE                                              \
  const int vr = (nv > 1) ? static_cast<int>(blockIdx.x % nv) : 0;    \
  const int cta = (nv > 1) ? static_cast<int>(blockIdx.x / nv) : static_cast<int>(blockIdx.x); \
  const int ncta = (nv > 1) ? static_cast<int>(gridDim.x / nv) : static_cast<int>(gridDim.x);  \
  const MoeDesc& d = (nv > 1) ? dv[vr] : d0;                          \
  (void)cta; (void)ncta;

// ----------------------------------------------------------------------------
// Metadata: histogram of topk_idx -> splits; exchange with every rank by direct
// peer stores + ticket; prefix sums -> segment tables. One CTA, no host sync
// (the reference needs two: moe_a2a.py:463-492).
// ----------------------------------------------------------------------------
__global__ void __launch_bounds__(1024)
moe_meta_kernel(const __grid_constant__ MoeDesc d0, const MoeDesc* __restrict__ dv, int nv) {
  TDB_MOE_PROLOGUE
  extern __shared__ int32_t sm[];
  int32_t* hist = sm;                 // [E]
  int32_t* meta = sm + d.E;           // [R * E]
  __shared__ int s_ok;
  const int tid = threadIdx.x;
  const int E = d.E, R = d.R;

  for (int e = tid; e < E; e += blockDim.x) hist[e] = 0;
  if (tid == 0) s_ok = 1;
  __syncthreads();
  const int pairs = d.T * d.topk;
  for (int i = tid; i < pairs; i += blockDim.x) {
    const int e = d.topk_idx[i];
    if (e >= 0 && e < E) atomicAdd(&hist[e], 1);
  }
  __syncthreads();
  for (int i = tid; i < R * E; i += blockDim.x) {
    const int dst = i / E, e = i - dst * E;
    d.peer_meta[dst][d.rank * E + e] = hist[e];
  }
  for (int e = tid; e < E; e += blockDim.x) {
    d.splits[e] = hist[e];
    d.counters[e] = 0;
  }
  // the barrier orders every thread's stores before the releases below (cumulative)
  __syncthreads();
  if (tid < R) {
    st_release_sys(d.peer_meta_flags[tid] + d.rank, d.round);
    if (!wait_flag_ge(d.peer_meta_flags[d.rank] + tid, d.round, d.env, SITE_MOE_META, tid)) s_ok = 0;
  }
  __syncthreads();
  if (s_ok == 0) return;
  for (int i = tid; i < R * E; i += blockDim.x)
    meta[i] = *reinterpret_cast<const volatile int32_t*>(d.peer_meta[d.rank] + i);
  __syncthreads();

  // me as a source: where my rows for expert e start inside the owner's buffer
  for (int e = tid; e < E; e += blockDim.x) {
    const int own = e / d.epr, le = e - own * d.epr;
    int base = 0;
    for (int s = 0; s < d.rank; ++s)
      for (int k = 0; k < d.epr; ++k) base += meta[s * E + own * d.epr + k];
    for (int k = 0; k < le; ++k) base += meta[d.rank * E + own * d.epr + k];
    d.dst_row_base[e] = base;
  }
  // me as a destination: (source, local expert) segments in order
  if (tid == 0) {
    int run = 0;
    for (int s = 0; s < R; ++s)
      for (int k = 0; k < d.epr; ++k) {
        const int cnt = meta[s * E + d.rank * d.epr + k];
        d.recv_seg[s * d.epr + k] = run;
        d.recv_counts[s * d.epr + k] = cnt;
        run += cnt;
      }
    *d.recv_total = run;
    if (run > d.max_recv_rows)
      report_failure(d.env, ST_OVERFLOW, SITE_MOE_META, d.max_recv_rows, run, 0);
  }
}

// ----------------------------------------------------------------------------
// Dispatch: one warp per (token, k). Slot allocation by a local atomic cursor per
// expert; the row is stored directly into the owner rank's receive buffer.
// The last CTA to finish tells every rank "my rows are in place" and waits until
// every rank said the same, so the kernel's completion means recv is complete.
// ----------------------------------------------------------------------------
__global__ void __launch_bounds__(256)
moe_dispatch_kernel(const __grid_constant__ MoeDesc d0, const MoeDesc* __restrict__ dv, int nv) {
  TDB_MOE_PROLOGUE
  __shared__ int s_last;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int pairs = d.T * d.topk;
  const int64_t row_bytes = static_cast<int64_t>(d.H) * 2;
  const int n16 = static_cast<int>(row_bytes >> 4);
  for (int pair = cta * 8 + warp; pair < pairs; pair += ncta * 8) {
    const int t = pair / d.topk;
    const int e = d.topk_idx[pair];
    int row = -1;
    if (lane == 0) {
      if (e >= 0 && e < d.E) {
        const int slot = atomicAdd(&d.counters[e], 1);
        row = d.dst_row_base[e] + slot;
        if (row < 0) {
          // the base comes from counts other ranks wrote: a negative row is recorded, never used
          report_failure(d.env, ST_BAD_INDEX, SITE_INDEX_CHECK, 0u, static_cast<uint32_t>(row), e);
          row = -1;
        } else if (row >= d.max_recv_rows) {
          report_failure(d.env, ST_OVERFLOW, SITE_MOE_DISPATCH_DONE, d.max_recv_rows, row, e);
          row = -1;
        }
      }
      d.scatter_idx[pair] = row;
    }
    row = __shfl_sync(0xFFFFFFFFu, row, 0);
    if (row < 0) continue;
    const int dest = e / d.epr;
    const uint8_t* src = reinterpret_cast<const uint8_t*>(d.tokens) + t * row_bytes;
    uint8_t* dst = reinterpret_cast<uint8_t*>(d.peer_recv[dest]) + row * row_bytes;
    // eight 16-byte pieces per lane in flight (4 KB per warp): a row of 8 KB is two such batches
    int i = lane;
    for (; i + 224 < n16; i += 256) {
      uint4 v[8];
#pragma unroll
      for (int u = 0; u < 8; ++u) v[u] = ld_global_nc_v4(src + ((i + 32 * u) << 4));
#pragma unroll
      for (int u = 0; u < 8; ++u) st_global_v4(dst + ((i + 32 * u) << 4), v[u]);
    }
    for (; i + 96 < n16; i += 128) {
      uint4 v[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) v[u] = ld_global_nc_v4(src + ((i + 32 * u) << 4));
#pragma unroll
      for (int u = 0; u < 4; ++u) st_global_v4(dst + ((i + 32 * u) << 4), v[u]);
    }
    for (; i < n16; i += 32) st_global_v4(dst + (i << 4), ld_global_nc_v4(src + (i << 4)));
  }
  // one system fence per CTA, by the thread that counts the CTA in, after the barrier that
  // orders all of the CTA's row stores before it (a fence in every thread costs microseconds)
  __syncthreads();
  if (tid == 0) {
    __threadfence_system();
    const uint32_t old = atomicAdd(d.done_counter, 1u);
    s_last = (old + 1u == static_cast<uint32_t>(ncta)) ? 1 : 0;
  }
  __syncthreads();
  if (s_last) {
    if (tid == 0) {
      atomicExch(d.done_counter, 0u);
      __threadfence_system();
    }
    __syncthreads();
    if (tid < d.R) {
      st_release_sys(d.peer_done_flags[tid] + d.rank, d.round);
      wait_flag_ge(d.peer_done_flags[d.rank] + tid, d.round, d.env, SITE_MOE_DISPATCH_DONE, tid);
    }
  }
}

// ----------------------------------------------------------------------------
// Combine: pull model. One CTA per token; 16-byte loads from the owner ranks'
// expert-output buffers, fp32 weighted accumulation.
// ----------------------------------------------------------------------------
template <bool kBf16>
__device__ __forceinline__ void fma8(float (&acc)[8], const uint4& v, float w) {
  const uint32_t u[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    float2 f;
    if constexpr (kBf16) f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&u[j]));
    else f = __half22float2(*reinterpret_cast<const __half2*>(&u[j]));
    acc[2 * j] = fmaf(w, f.x, acc[2 * j]);
    acc[2 * j + 1] = fmaf(w, f.y, acc[2 * j + 1]);
  }
}

template <bool kBf16>
__device__ __forceinline__ uint4 pack8(const float (&a)[8]) {
  uint4 o;
  uint32_t* w = reinterpret_cast<uint32_t*>(&o);
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    if constexpr (kBf16) {
      __nv_bfloat162 v = __floats2bfloat162_rn(a[2 * j], a[2 * j + 1]);
      w[j] = *reinterpret_cast<uint32_t*>(&v);
    } else {
      __half2 v = __floats2half2_rn(a[2 * j], a[2 * j + 1]);
      w[j] = *reinterpret_cast<uint32_t*>(&v);
    }
  }
  return o;
}

constexpr int kMaxTopk = 32;

template <bool kBf16>
__global__ void __launch_bounds__(128)
moe_combine_kernel(const __grid_constant__ MoeDesc d0, const MoeDesc* __restrict__ dv, int nv) {
  TDB_MOE_PROLOGUE
  __shared__ const uint8_t* s_src[kMaxTopk];
  __shared__ float s_w[kMaxTopk];
  const int tid = threadIdx.x;
  if (cta == 0 && tid < d.R) {
    __threadfence_system();
    st_release_sys(d.peer_ready_flags[tid] + d.rank, d.round);
  }
  int ok = 1;
  if (tid < d.R)
    ok = wait_flag_ge(d.peer_ready_flags[d.rank] + tid, d.round, d.env, SITE_MOE_COMBINE_READY, tid) ? 1 : 0;
  if (!__syncthreads_and(ok)) return;

  const int64_t row_bytes = static_cast<int64_t>(d.H) * 2;
  const int n16 = static_cast<int>(row_bytes >> 4);
  for (int t = cta; t < d.T; t += ncta) {
    if (tid < d.topk) {
      const int pair = t * d.topk + tid;
      const int e = d.topk_idx[pair];
      const int row = d.scatter_idx[pair];
      const bool valid = (e >= 0 && e < d.E && row >= 0 && row < d.max_recv_rows);
      if (e >= 0 && e < d.E && (row < -1 || row >= d.max_recv_rows))      // -1 = dropped at dispatch
        report_failure(d.env, ST_BAD_INDEX, SITE_INDEX_CHECK, static_cast<uint32_t>(d.max_recv_rows),
                       static_cast<uint32_t>(row), e);
      s_src[tid] = valid ? reinterpret_cast<const uint8_t*>(d.peer_out[e / d.epr]) + row * row_bytes
                         : nullptr;
      s_w[tid] = d.has_weights ? d.topk_weights[pair] : 1.0f;
    }
    __syncthreads();
    for (int v = tid; v < n16; v += blockDim.x) {
      float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
      for (int j0 = 0; j0 < d.topk; j0 += 8) {
        uint4 val[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) {
          const int j = j0 + u;
          val[u] = (j < d.topk && s_src[j] != nullptr) ? ld_global_cg_v4(s_src[j] + (v << 4))
                                                       : make_uint4(0u, 0u, 0u, 0u);
        }
#pragma unroll
        for (int u = 0; u < 8; ++u)
          if (j0 + u < d.topk) fma8<kBf16>(acc, val[u], s_w[j0 + u]);
      }
      st_global_v4(reinterpret_cast<uint8_t*>(d.output) + t * row_bytes + (v << 4), pack8<kBf16>(acc));
    }
    __syncthreads();
  }
}

// ----------------------------------------------------------------------------
// Launchers
// ----------------------------------------------------------------------------
static void validate(const MoeDesc& d) {
  if (d.R < 1 || d.R > 8) throw std::runtime_error("tridist_b200: MoE needs 1..8 ranks");
  if (d.E < 1 || d.E > 1024 || d.E % d.R != 0)
    throw std::runtime_error("tridist_b200: MoE needs num_experts <= 1024 and divisible by ranks");
  if (d.topk < 1 || d.topk > kMaxTopk) throw std::runtime_error("tridist_b200: MoE needs topk <= 32");
  if ((static_cast<int64_t>(d.H) * 2) % 16 != 0)
    throw std::runtime_error("tridist_b200: MoE needs hidden % 8 == 0");
}

static int dispatch_ctas(const MoeDesc& d) {
  const int pairs = d.T * d.topk;
  int g = (pairs + 7) / 8;
  if (g > 148 * 8) g = 148 * 8;
  if (g < 1) g = 1;
  return g;
}

static int combine_ctas(const MoeDesc& d) {
  int g = d.T;
  if (g > 148 * 16) g = 148 * 16;
  if (g < 1) g = 1;
  return g;
}

void moe_meta_launch(const MoeDesc& d, void* stream_) {
  validate(d);
  const size_t smem = sizeof(int32_t) * (d.E + d.R * d.E);
  moe_meta_kernel<<<1, 1024, smem, reinterpret_cast<cudaStream_t>(stream_)>>>(d, nullptr, 1);
  check(cudaGetLastError(), "moe_meta launch");
  launch_count_add(1);
}

void moe_dispatch_launch(const MoeDesc& d, void* stream_) {
  validate(d);
  moe_dispatch_kernel<<<dispatch_ctas(d), 256, 0, reinterpret_cast<cudaStream_t>(stream_)>>>(d, nullptr, 1);
  check(cudaGetLastError(), "moe_dispatch launch");
  launch_count_add(1);
}

void moe_combine_launch(const MoeDesc& d, void* stream_) {
  validate(d);
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream_);
  if (d.bf16) moe_combine_kernel<true><<<combine_ctas(d), 128, 0, s>>>(d, nullptr, 1);
  else moe_combine_kernel<false><<<combine_ctas(d), 128, 0, s>>>(d, nullptr, 1);
  check(cudaGetLastError(), "moe_combine launch");
  launch_count_add(1);
}

void moe_emulated_launch(const std::vector<MoeDesc>& ds, int phase, void* stream_) {
  const int nv = static_cast<int>(ds.size());
  if (nv < 1 || nv > 8) throw std::runtime_error("tridist_b200: bad emulated rank count");
  for (auto& d : ds) validate(d);
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream_);
  static MoeDesc* dev = nullptr;
  if (!dev) check(cudaMalloc(&dev, sizeof(MoeDesc) * 8), "cudaMalloc(moe descs)");
  check(cudaMemcpyAsync(dev, ds.data(), sizeof(MoeDesc) * nv, cudaMemcpyHostToDevice, s), "copy descs");
  check(cudaStreamSynchronize(s), "sync descs");
  const MoeDesc& d = ds[0];
  if (phase == 0) {
    const size_t smem = sizeof(int32_t) * (d.E + d.R * d.E);
    MoeDesc dummy = d;
    const MoeDesc* dp = dev;
    int nvv = nv;
    void* args[3] = {&dummy, &dp, &nvv};
    check(cudaLaunchCooperativeKernel(reinterpret_cast<void*>(moe_meta_kernel), dim3(nv), dim3(1024), args,
                                      smem, s),
          "moe_meta cooperative launch");
  } else if (phase == 1) {
    moe_dispatch_kernel<<<dispatch_ctas(d) * nv, 256, 0, s>>>(d, dev, nv);
  } else {
    if (d.bf16) moe_combine_kernel<true><<<combine_ctas(d) * nv, 128, 0, s>>>(d, dev, nv);
    else moe_combine_kernel<false><<<combine_ctas(d) * nv, 128, 0, s>>>(d, dev, nv);
  }
  check(cudaGetLastError(), "moe emulated launch");
  launch_count_add(1);
}

}  // namespace tdb

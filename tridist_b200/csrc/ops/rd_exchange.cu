#include "rd_exchange.h"

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <stdexcept>
#include <string>

#include "fused_gemm.h"
#include "../common/sync.cuh"

namespace tdb {
namespace {

inline void check(cudaError_t e, const char* what) {
  if (e != cudaSuccess)
    throw std::runtime_error(std::string("tridist_b200: ") + what + ": " + cudaGetErrorString(e));
}

constexpr int kRdThreads = 512;
constexpr int kRdUnroll = 8;          // 16-byte pieces in flight per thread

struct RdArgs {
  RdRankArgs r[8];
  int ranks_in_launch;                // 1 (one rank per process) or R (virtual ranks, grid.y)
};

__device__ __forceinline__ uint4 ld16(const void* p) { return *reinterpret_cast<const uint4*>(p); }
__device__ __forceinline__ void st16(void* p, const uint4& v) { *reinterpret_cast<uint4*>(p) = v; }

// Peer data written with plain stores and published by a release ticket is read with loads that
// bypass L1 (the line could be resident from the slot's previous occupant).
__device__ __forceinline__ uint4 ld16_nc(const void* p) {
  uint4 v;
  asm volatile("ld.global.cg.v4.u32 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p)
               : "memory");
  return v;
}

template <bool kBf16>
__device__ __forceinline__ uint32_t add2(uint32_t a, uint32_t b) {
  if constexpr (kBf16) {
    const float2 x = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&a));
    const float2 y = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&b));
    const __nv_bfloat162 s = __floats2bfloat162_rn(x.x + y.x, x.y + y.y);
    return *reinterpret_cast<const uint32_t*>(&s);
  } else {
    const float2 x = __half22float2(*reinterpret_cast<const __half2*>(&a));
    const float2 y = __half22float2(*reinterpret_cast<const __half2*>(&b));
    const __half2 s = __floats2half2_rn(x.x + y.x, x.y + y.y);
    return *reinterpret_cast<const uint32_t*>(&s);
  }
}

// One CTA owns one slice of the panel (a contiguous range of 16-byte pieces in panel order) through
// ALL exchange phases: what it pushes in phase p + 1 is what it accumulated itself in phase p, so
// the phases of a slice need no grid-wide synchronisation, only the two tickets per (phase, slice)
// that pair it with the same slice of the partner rank.
template <bool kBf16>
__global__ void __launch_bounds__(kRdThreads) rd_exchange_kernel(const __grid_constant__ RdArgs args) {
  const RdRankArgs& a = args.r[args.ranks_in_launch > 1 ? blockIdx.y : 0];
  __shared__ int s_ok;
  const int slice = blockIdx.x;
  const int n_slices = gridDim.x;
  const int tid = threadIdx.x;
  const int64_t row_pieces = a.n_cols / 8;                      // 16-byte pieces per panel row
  const int64_t pieces = static_cast<int64_t>(a.rows) * row_pieces;
  const int64_t per = (pieces + n_slices - 1) / n_slices;
  const int64_t p0 = min(pieces, per * slice);
  const int64_t p1 = min(pieces, p0 + per);
  if (slice >= a.flag_slices || a.slot < 0 || a.slot >= a.slots) {     // never index a ticket plane blindly
    if (tid == 0)
      report_failure(a.env, ST_BAD_INDEX, SITE_INDEX_CHECK, static_cast<uint32_t>(a.flag_slices),
                     static_cast<uint32_t>(slice), static_cast<uint32_t>(a.slot));
    return;
  }
  char* const c = reinterpret_cast<char*>(a.c);
  const int64_t ldc_bytes = a.ldc * 2;
  auto c_addr = [&](int64_t piece) -> char* {
    const int64_t row = piece / row_pieces;
    return c + row * ldc_bytes + (piece - row * row_pieces) * 16;
  };
  for (int ph = 0; ph < a.phases; ++ph) {
    const int64_t flag_idx = (static_cast<int64_t>(a.slot) * a.phases + ph) * a.flag_slices + slice;
    const int64_t region = (static_cast<int64_t>(a.slot) * a.phases + ph) * a.slot_bytes;
    // 1. the partner must have consumed what the previous occupant of this slot pushed to it
    if (tid == 0) s_ok = wait_flag_ge(a.ack + flag_idx, a.prev_ticket, a.env, SITE_RD_ACK, (ph << 16) | slice) ? 1 : 0;
    __syncthreads();
    if (!s_ok) return;
    // 2. push this slice of the current accumulator into the partner's slot
    char* const dst = reinterpret_cast<char*>(a.peer_scatter[ph]) + region;
    for (int64_t base = p0 + tid; base < p1; base += static_cast<int64_t>(kRdThreads) * kRdUnroll) {
      uint4 v[kRdUnroll];
#pragma unroll
      for (int u = 0; u < kRdUnroll; ++u) {
        const int64_t i = base + static_cast<int64_t>(u) * kRdThreads;
        if (i < p1) v[u] = ld16(c_addr(i));
      }
#pragma unroll
      for (int u = 0; u < kRdUnroll; ++u) {
        const int64_t i = base + static_cast<int64_t>(u) * kRdThreads;
        if (i < p1) st16(dst + i * 16, v[u]);
      }
    }
    // 3. publish: the CTA barrier orders all threads' stores before the one release store
    __syncthreads();
    if (tid == 0) st_release_sys(a.peer_arrival[ph] + flag_idx, a.ticket);
    // 4. the partner's slice
    if (tid == 0) s_ok = wait_flag_ge(a.arrival + flag_idx, a.ticket, a.env, SITE_RD_ARRIVAL, (ph << 16) | slice) ? 1 : 0;
    __syncthreads();
    if (!s_ok) return;
    // 5. accumulate in place (fp32 add of two 16-bit values, rounded once: both partners compute
    // the same sum from the same two operands, so their accumulators stay bit-identical)
    const char* const src = reinterpret_cast<const char*>(a.scatter) + region;
    for (int64_t base = p0 + tid; base < p1; base += static_cast<int64_t>(kRdThreads) * kRdUnroll) {
      uint4 x[kRdUnroll], y[kRdUnroll];
#pragma unroll
      for (int u = 0; u < kRdUnroll; ++u) {
        const int64_t i = base + static_cast<int64_t>(u) * kRdThreads;
        if (i < p1) {
          y[u] = ld16_nc(src + i * 16);
          x[u] = ld16(c_addr(i));
        }
      }
#pragma unroll
      for (int u = 0; u < kRdUnroll; ++u) {
        const int64_t i = base + static_cast<int64_t>(u) * kRdThreads;
        if (i < p1) {
          uint4 s;
          s.x = add2<kBf16>(x[u].x, y[u].x);
          s.y = add2<kBf16>(x[u].y, y[u].y);
          s.z = add2<kBf16>(x[u].z, y[u].z);
          s.w = add2<kBf16>(x[u].w, y[u].w);
          st16(c_addr(i), s);
        }
      }
    }
    // 6. hand the slot region back to the partner
    __syncthreads();
    if (tid == 0) st_release_sys(a.peer_ack[ph] + flag_idx, a.ticket);
  }
}

void validate(const RdRankArgs& a) {
  if (a.phases < 1 || a.phases > 3) throw std::runtime_error("tridist_b200: rd exchange needs 2, 4 or 8 ranks");
  if (a.n_cols % 8 != 0 || a.ldc % 8 != 0 || (reinterpret_cast<uintptr_t>(a.c) & 15u))
    throw std::runtime_error("tridist_b200: rd exchange moves 16-byte pieces: N, the row stride and the panel address must be multiples of 8 elements");
  if (static_cast<int64_t>(a.rows) * a.n_cols * 2 > a.slot_bytes)
    throw std::runtime_error("tridist_b200: rd exchange panel larger than a staging slot");
}

}  // namespace

void rd_exchange_launch(const std::vector<RdRankArgs>& ranks, int ctas, bool bf16, void* stream_) {
  if (ranks.empty() || ranks.size() > 8) throw std::runtime_error("tridist_b200: rd exchange takes 1..8 rank blocks");
  RdArgs args{};
  for (size_t i = 0; i < ranks.size(); ++i) {
    validate(ranks[i]);
    args.r[i] = ranks[i];
  }
  args.ranks_in_launch = static_cast<int>(ranks.size());
  if (ctas < 1 || ctas > ranks[0].flag_slices) throw std::runtime_error("tridist_b200: rd exchange CTA count outside the ticket plane");
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  dim3 grid(ctas, static_cast<unsigned>(ranks.size()));
  auto* fn = bf16 ? rd_exchange_kernel<true> : rd_exchange_kernel<false>;
  if (ranks.size() == 1) {
    fn<<<grid, kRdThreads, 0, stream>>>(args);
    check(cudaGetLastError(), "rd exchange launch");
  } else {
    // virtual ranks of one launch wait on one another: all CTAs must be resident together
    void* kargs[] = {&args};
    check(cudaLaunchCooperativeKernel(reinterpret_cast<void*>(fn), grid, dim3(kRdThreads), kargs, 0, stream),
          "rd exchange cooperative launch");
  }
  launch_count_add(1);
}

}  // namespace tdb

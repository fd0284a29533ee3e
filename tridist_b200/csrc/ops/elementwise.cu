#include "elementwise.h"

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

// ----------------------------------------------------------------------------
// SwiGLU. The reference composes it from torch ops between the two fused GEMMs
// (bench/s21_bench_tp_mlp_dcu.py:206-207); gate and up are the two halves of
// each row of the AG+GEMM output. Memory-bound: 16-byte loads and stores.
// ----------------------------------------------------------------------------
template <bool kBf16>
__device__ __forceinline__ uint32_t swiglu2(uint32_t g, uint32_t u) {
  if constexpr (kBf16) {
    const float2 gf = __bfloat1622float2(*reinterpret_cast<__nv_bfloat162*>(&g));
    const float2 uf = __bfloat1622float2(*reinterpret_cast<__nv_bfloat162*>(&u));
    __nv_bfloat162 r = __floats2bfloat162_rn(__fdividef(gf.x, 1.f + __expf(-gf.x)) * uf.x,
                                             __fdividef(gf.y, 1.f + __expf(-gf.y)) * uf.y);
    return *reinterpret_cast<uint32_t*>(&r);
  } else {
    const float2 gf = __half22float2(*reinterpret_cast<__half2*>(&g));
    const float2 uf = __half22float2(*reinterpret_cast<__half2*>(&u));
    __half2 r = __floats2half2_rn(__fdividef(gf.x, 1.f + __expf(-gf.x)) * uf.x,
                                  __fdividef(gf.y, 1.f + __expf(-gf.y)) * uf.y);
    return *reinterpret_cast<uint32_t*>(&r);
  }
}

template <bool kBf16>
__global__ void __launch_bounds__(256) swiglu_kernel(const uint8_t* __restrict__ h,
                                                     uint8_t* __restrict__ out, int64_t rows,
                                                     int64_t inter, int64_t ldh) {
  const int64_t vec_per_row = inter >> 3;
  const int64_t total = rows * vec_per_row;
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  // two independent 16-byte gate/up pairs per iteration keep four loads in flight per thread
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < total; i += 2 * stride) {
    const int64_t i2 = i + stride;
    const bool two = i2 < total;
    const int64_t r0 = i / vec_per_row, v0 = i - r0 * vec_per_row;
    const int64_t r1 = two ? i2 / vec_per_row : r0, v1 = two ? i2 - r1 * vec_per_row : v0;
    const uint8_t* row0 = h + r0 * ldh * 2;
    const uint8_t* row1 = h + r1 * ldh * 2;
    const uint4 g0 = ld_global_nc_v4(row0 + v0 * 16);
    const uint4 u0 = ld_global_nc_v4(row0 + inter * 2 + v0 * 16);
    const uint4 g1 = ld_global_nc_v4(row1 + v1 * 16);
    const uint4 u1 = ld_global_nc_v4(row1 + inter * 2 + v1 * 16);
    uint4 o;
    o.x = swiglu2<kBf16>(g0.x, u0.x);
    o.y = swiglu2<kBf16>(g0.y, u0.y);
    o.z = swiglu2<kBf16>(g0.z, u0.z);
    o.w = swiglu2<kBf16>(g0.w, u0.w);
    st_global_v4(out + (r0 * inter + v0 * 8) * 2, o);
    if (two) {
      o.x = swiglu2<kBf16>(g1.x, u1.x);
      o.y = swiglu2<kBf16>(g1.y, u1.y);
      o.z = swiglu2<kBf16>(g1.z, u1.z);
      o.w = swiglu2<kBf16>(g1.w, u1.w);
      st_global_v4(out + (r1 * inter + v1 * 8) * 2, o);
    }
  }
}

void swiglu_launch(const void* h, void* out, int64_t rows, int64_t inter, int64_t ldh, bool bf16,
                   void* stream_) {
  if (inter % 8 != 0 || ldh % 8 != 0)
    throw std::runtime_error("tridist_b200: swiglu needs inter and row stride % 8 == 0");
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  const int64_t total = rows * (inter >> 3);
  if (total == 0) return;
  int64_t blocks = (total + 255) / 256;
  if (blocks > 148 * 16) blocks = 148 * 16;
  if (bf16)
    swiglu_kernel<true><<<static_cast<int>(blocks), 256, 0, stream>>>(
        reinterpret_cast<const uint8_t*>(h), reinterpret_cast<uint8_t*>(out), rows, inter, ldh);
  else
    swiglu_kernel<false><<<static_cast<int>(blocks), 256, 0, stream>>>(
        reinterpret_cast<const uint8_t*>(h), reinterpret_cast<uint8_t*>(out), rows, inter, ldh);
  check(cudaGetLastError(), "swiglu launch");
  launch_count_add(1);
}

// ----------------------------------------------------------------------------
// Cross-rank ticket barrier (the reference's SymmBarrier, common_ops.py:212-256:
// engine writes of the round number + a spin kernel; here both legs are one
// kernel and the wait is bounded).
// ----------------------------------------------------------------------------
struct BarrierArgs {
  uint32_t* peer_slots[8];
  int rank, R;
  uint32_t ticket;
  WaitEnv env;
};

__global__ void barrier_kernel(const __grid_constant__ BarrierArgs a) {
  const int i = threadIdx.x;
  if (i < a.R) {
    __threadfence_system();
    st_release_sys(a.peer_slots[i] + a.rank, a.ticket);
    wait_flag_ge(a.peer_slots[a.rank] + i, a.ticket, a.env, SITE_BARRIER, i);
  }
}

void barrier_launch(const std::vector<int64_t>& peer_slots, int rank, int R, uint32_t ticket,
                    int64_t status_dev, int64_t abort_word, uint64_t timeout_ns, void* stream_,
                    const std::vector<int64_t>& peer_abort) {
  if (R < 1 || R > 8 || static_cast<int>(peer_slots.size()) < R)
    throw std::runtime_error("tridist_b200: barrier needs 1..8 ranks");
  BarrierArgs a{};
  for (int i = 0; i < R; ++i) a.peer_slots[i] = reinterpret_cast<uint32_t*>(peer_slots[i]);
  a.rank = rank;
  a.R = R;
  a.ticket = ticket;
  a.env.status = reinterpret_cast<StatusBlock*>(status_dev);
  a.env.abort_word = reinterpret_cast<uint32_t*>(abort_word);
  a.env.timeout_ns = timeout_ns;
  a.env.rank = static_cast<uint32_t>(rank);
  for (size_t i = 0; i < peer_abort.size() && i < 8; ++i) {
    a.env.peer_abort[i] = reinterpret_cast<uint32_t*>(peer_abort[i]);
    a.env.n_peers = static_cast<uint32_t>(i + 1);
  }
  barrier_kernel<<<1, 32, 0, reinterpret_cast<cudaStream_t>(stream_)>>>(a);
  check(cudaGetLastError(), "barrier launch");
  launch_count_add(1);
}

// ----------------------------------------------------------------------------
// Bounded-wait self test
// ----------------------------------------------------------------------------
__global__ void wait_flag_test_kernel(const uint32_t* flag, uint32_t ticket, WaitEnv env) {
  wait_flag_ge(flag, ticket, env, SITE_TEST, 0);
}

void wait_flag_test_launch(int64_t flag, uint32_t ticket, int64_t status_dev, int64_t abort_word,
                           uint64_t timeout_ns, void* stream_, const std::vector<int64_t>& peer_abort) {
  WaitEnv env{};
  env.status = reinterpret_cast<StatusBlock*>(status_dev);
  env.abort_word = reinterpret_cast<uint32_t*>(abort_word);
  env.timeout_ns = timeout_ns;
  env.rank = 0;
  for (size_t i = 0; i < peer_abort.size() && i < 8; ++i) {
    env.peer_abort[i] = reinterpret_cast<uint32_t*>(peer_abort[i]);
    env.n_peers = static_cast<uint32_t>(i + 1);
  }
  wait_flag_test_kernel<<<1, 1, 0, reinterpret_cast<cudaStream_t>(stream_)>>>(
      reinterpret_cast<const uint32_t*>(flag), ticket, env);
  check(cudaGetLastError(), "wait_flag_test launch");
  launch_count_add(1);
}

// One thread writes the global timer: a time stamp in stream order, on the clock the kernels'
// own accounting uses (so that "when did the previous kernel end" can be placed on a CTA time line).
__global__ void stamp_kernel(uint64_t* out) { *out = globaltimer_ns(); }

void stamp_globaltimer_launch(int64_t out, void* stream_) {
  stamp_kernel<<<1, 1, 0, reinterpret_cast<cudaStream_t>(stream_)>>>(reinterpret_cast<uint64_t*>(out));
  check(cudaGetLastError(), "stamp launch");
}

__global__ void fill_u32_kernel(uint32_t* p, int64_t n, uint32_t v) {
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < n;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x)
    p[i] = v;
}

void fill_u32_launch(uint32_t* p, int64_t n, uint32_t v, void* stream_) {
  if (n <= 0) return;
  int64_t blocks = (n + 255) / 256;
  if (blocks > 1024) blocks = 1024;
  fill_u32_kernel<<<static_cast<int>(blocks), 256, 0, reinterpret_cast<cudaStream_t>(stream_)>>>(p, n, v);
  check(cudaGetLastError(), "fill_u32 launch");
  launch_count_add(1);
}

// ----------------------------------------------------------------------------
// Spot verification (the reference's in-op self check, ag_tr_pred.py:533-566):
// one warp per (tile, spot) recomputes a dot product in fp32.
// ----------------------------------------------------------------------------
template <bool kBf16>
__device__ __forceinline__ float to_f32(const void* p, int64_t i) {
  if constexpr (kBf16) return __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p)[i]);
  else return __half2float(reinterpret_cast<const __half*>(p)[i]);
}

template <bool kBf16>
__global__ void spot_verify_kernel(const void* a, const void* b, const void* c, int M, int N, int K,
                                   int64_t lda, int64_t ldb, int64_t ldc, int spots, float tol,
                                   int32_t* bad_tiles, int bn) {
  const int n_tiles = (N + bn - 1) / bn;
  const int tile = blockIdx.x;
  const int mt = tile / n_tiles, nt = tile - mt * n_tiles;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int s = warp; s < spots; s += blockDim.x >> 5) {
    uint32_t hsh = (static_cast<uint32_t>(tile) * 2654435761u) ^ (static_cast<uint32_t>(s) * 40503u + 977u);
    hsh ^= hsh >> 13; hsh *= 1274126177u; hsh ^= hsh >> 16;
    const int r = min(mt * 128 + static_cast<int>(hsh % 128u), M - 1);
    const int col = min(nt * bn + static_cast<int>((hsh >> 8) % static_cast<uint32_t>(bn)), N - 1);
    float acc = 0.f;
    for (int k = lane; k < K; k += 32)
      acc += to_f32<kBf16>(a, static_cast<int64_t>(r) * lda + k) *
             to_f32<kBf16>(b, static_cast<int64_t>(col) * ldb + k);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xFFFFFFFFu, acc, o);
    if (lane == 0) {
      const float got = to_f32<kBf16>(c, static_cast<int64_t>(r) * ldc + col);
      if (!(fabsf(got - acc) <= tol * (1.f + fabsf(acc)))) bad_tiles[tile] = 1;
    }
  }
}

void spot_verify_launch(int64_t a, int64_t b, int64_t c, int M, int N, int K, int64_t lda,
                        int64_t ldb, int64_t ldc, bool bf16, int spots, float tol,
                        int64_t bad_tiles, int bn, void* stream_) {
  const int tiles = ((M + 127) / 128) * ((N + bn - 1) / bn);
  if (tiles == 0) return;
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  if (bf16)
    spot_verify_kernel<true><<<tiles, 128, 0, stream>>>(
        reinterpret_cast<const void*>(a), reinterpret_cast<const void*>(b),
        reinterpret_cast<const void*>(c), M, N, K, lda, ldb, ldc, spots, tol,
        reinterpret_cast<int32_t*>(bad_tiles), bn);
  else
    spot_verify_kernel<false><<<tiles, 128, 0, stream>>>(
        reinterpret_cast<const void*>(a), reinterpret_cast<const void*>(b),
        reinterpret_cast<const void*>(c), M, N, K, lda, ldb, ldc, spots, tol,
        reinterpret_cast<int32_t*>(bad_tiles), bn);
  check(cudaGetLastError(), "spot_verify launch");
  launch_count_add(1);
}

// ----------------------------------------------------------------------------
// multimem transport probe: reduce-load 16-byte pieces of [begin, end) through the switch and
// write them back (replicated through the switch, or to local memory). No waits, no flags:
// ranks run it side by side on disjoint ranges. Reads how throughput depends on the number of
// threads, the pieces each thread keeps in flight and the ordering qualifier.
// ----------------------------------------------------------------------------
template <int kU, bool kWeak, bool kLocalStore>
__global__ void multimem_probe_kernel(const uint8_t* __restrict__ mc_in, uint8_t* __restrict__ mc_out,
                                      uint8_t* __restrict__ local_out, int64_t begin, int64_t end) {
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  for (int64_t i0 = begin + static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i0 < end;
       i0 += stride * kU) {
    uint4 v[kU];
#pragma unroll
    for (int u = 0; u < kU; ++u) {
      const int64_t i = i0 + u * stride;
      if (i < end) {
        if constexpr (kWeak)
          asm volatile("multimem.ld_reduce.weak.global.add.acc::f32.v4.bf16x2 {%0,%1,%2,%3}, [%4];"
                       : "=r"(v[u].x), "=r"(v[u].y), "=r"(v[u].z), "=r"(v[u].w)
                       : "l"(mc_in + i * 16)
                       : "memory");
        else
          v[u] = multimem_ld_reduce_add_v4<true>(mc_in + i * 16);
      }
    }
#pragma unroll
    for (int u = 0; u < kU; ++u) {
      const int64_t i = i0 + u * stride;
      if (i < end) {
        if constexpr (kLocalStore) {
          st_global_v4(local_out + i * 16, v[u]);
        } else if constexpr (kWeak) {
          asm volatile("multimem.st.weak.global.v4.f32 [%0], {%1,%2,%3,%4};" ::"l"(mc_out + i * 16),
                       "r"(v[u].x), "r"(v[u].y), "r"(v[u].z), "r"(v[u].w)
                       : "memory");
        } else {
          multimem_st_v4(mc_out + i * 16, v[u]);
        }
      }
    }
  }
}

void multimem_probe_launch(int64_t mc_in, int64_t mc_out, int64_t local_out, int64_t begin, int64_t end,
                           int blocks, int threads, int unroll, bool weak, bool local_store,
                           void* stream_) {
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  if (blocks < 1 || threads < 32 || threads > 1024) throw std::runtime_error("tridist_b200: bad probe launch shape");
  auto* in = reinterpret_cast<const uint8_t*>(mc_in);
  auto* out = reinterpret_cast<uint8_t*>(mc_out);
  auto* lo = reinterpret_cast<uint8_t*>(local_out);
#define TDB_PROBE(U_)                                                                              \
  do {                                                                                             \
    if (weak && local_store) multimem_probe_kernel<U_, true, true><<<blocks, threads, 0, stream>>>(in, out, lo, begin, end);   \
    else if (weak) multimem_probe_kernel<U_, true, false><<<blocks, threads, 0, stream>>>(in, out, lo, begin, end);           \
    else if (local_store) multimem_probe_kernel<U_, false, true><<<blocks, threads, 0, stream>>>(in, out, lo, begin, end);    \
    else multimem_probe_kernel<U_, false, false><<<blocks, threads, 0, stream>>>(in, out, lo, begin, end);                    \
  } while (0)
  if (unroll == 1) TDB_PROBE(1);
  else if (unroll == 4) TDB_PROBE(4);
  else if (unroll == 8) TDB_PROBE(8);
  else throw std::runtime_error("tridist_b200: probe unroll must be 1, 4 or 8");
#undef TDB_PROBE
  check(cudaGetLastError(), "multimem_probe launch");
  launch_count_add(1);
}

}  // namespace tdb

// Small sm_100a kernels around the fused operators: SwiGLU, the cross-rank
// ticket barrier, the bounded-wait self test, and spot verification of a GEMM result.
//
// Reference counterparts: the monotonic-round barrier (engine writes of the round number into every
// rank's slot + a one-CTA spin kernel, triton_dist/kernels/dcu/common_ops.py:212-256), the
// flag wait kernel (gemm_ar_rd.py:112-125), SwiGLU of the TP-MLP bench
// (bench/s21_bench_tp_mlp_dcu.py:21-22) and the spot verification of the skew layer
// (ag_tr_pred.py:533-566).
#pragma once
#include <cstdint>
#include <vector>

namespace tdb {

// out[r, j] = silu(h[r, j]) * h[r, inter + j]   (gate and up halves stored side by side)
void swiglu_launch(const void* h, void* out, int64_t rows, int64_t inter, int64_t ldh, bool bf16,
                   void* stream);

// Cross-rank barrier: writes `ticket` into slot [rank] of every rank's slot array, then
// waits (bounded) until all R local slots reached the ticket.
// `peer_abort`: every rank's abort word (raised together when this wait gives up); may be empty.
void barrier_launch(const std::vector<int64_t>& peer_slots, int rank, int R, uint32_t ticket,
                    int64_t status_dev, int64_t abort_word, uint64_t timeout_ns, void* stream,
                    const std::vector<int64_t>& peer_abort = {});

// One thread waits for *flag >= ticket with the given limit; exercises timeout -> status.
void wait_flag_test_launch(int64_t flag, uint32_t ticket, int64_t status_dev, int64_t abort_word,
                           uint64_t timeout_ns, void* stream, const std::vector<int64_t>& peer_abort = {});

void fill_u32_launch(uint32_t* p, int64_t n, uint32_t v, void* stream);

// Writes the device's global timer (ns) to `out` (8 bytes of device memory) in stream order.
void stamp_globaltimer_launch(int64_t out, void* stream);

// Recomputes `spots` pseudo-randomly chosen elements of every 128 x bn tile of
// C = A @ B^T in fp32 and sets bad_tiles[tile] = 1 where |c - ref| > tol * (1 + |ref|).
void spot_verify_launch(int64_t a, int64_t b, int64_t c, int M, int N, int K, int64_t lda,
                        int64_t ldb, int64_t ldc, bool bf16, int spots, float tol,
                        int64_t bad_tiles, int bn, void* stream);

// Transport probe for the NVSwitch multicast path (see the kernel): pieces are 16 bytes,
// [begin, end) counts pieces; `mc_in` / `mc_out` are multicast addresses.
void multimem_probe_launch(int64_t mc_in, int64_t mc_out, int64_t local_out, int64_t begin, int64_t end,
                           int blocks, int threads, int unroll, bool weak, bool local_store, void* stream);

}  // namespace tdb

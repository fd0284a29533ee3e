// MoE all-to-all: routing metadata, dispatch (push rows straight into the
// destination ranks' receive buffers) and combine (pull + weighted sum).
//
// Contract kept from the reference (triton_dist/kernels/dcu/moe_a2a.py):
//   * topk_idx holds global expert ids; expert e lives on rank e / epr (:207-210)
//   * a destination's receive rows are ordered by (source rank, local expert)
//     segments (:398-403); scatter_idx[t, j] is the row inside that buffer
//   * the expert phase writes out[row] 1:1 for row < recv_total
//   * combine: output[t] = sum_j w[t, j] * out_{rank(e_j)}[scatter_idx[t, j]] in fp32 (:245-263)
// What differs: no staging buffer, no host round trip and no host-issued copies;
// the segment table is built on the device and rows travel by in-kernel stores.
#pragma once
#include <cstdint>
#include <vector>

#include "../common/status.h"

namespace tdb {

struct alignas(16) MoeDesc {
  int32_t rank, R, E, epr, H, T, topk, max_recv_rows;
  int32_t bf16, has_weights;
  uint32_t round;
  int32_t pad0;
  const void* tokens;          // [T, H]
  const int32_t* topk_idx;     // [T, topk]
  const float* topk_weights;   // [T, topk] or nullptr
  void* output;                // [T, H] combine result
  void* peer_recv[8];          // [max_recv_rows, H] on every rank
  void* peer_out[8];           // [max_recv_rows, H] on every rank
  int32_t* peer_meta[8];       // [R, E] split counts on every rank, row = source
  uint32_t* peer_meta_flags[8];   // [R] tickets, indexed by source
  uint32_t* peer_done_flags[8];   // [R] "all my rows for you are stored"
  uint32_t* peer_ready_flags[8];  // [R] "my expert outputs are complete"
  int32_t* splits;             // [E] this rank's tokens per global expert
  int32_t* dst_row_base;       // [E] first row of (me, expert) inside the owner's recv buffer
  int32_t* counters;           // [E] slot allocation cursors
  int32_t* recv_seg;           // [R, epr] first row of segment (source, local expert) here
  int32_t* recv_counts;        // [R, epr]
  int32_t* recv_total;         // [1]
  int32_t* scatter_idx;        // [T, topk]
  uint32_t* done_counter;      // [1] CTAs of the dispatch kernel that finished
  WaitEnv env;
};

void moe_meta_launch(const MoeDesc& d, void* stream);
void moe_dispatch_launch(const MoeDesc& d, void* stream);
void moe_combine_launch(const MoeDesc& d, void* stream);
// phase 0 = meta, 1 = dispatch, 2 = combine; all ranks in ONE launch on one GPU.
void moe_emulated_launch(const std::vector<MoeDesc>& ds, int phase, void* stream);

}  // namespace tdb

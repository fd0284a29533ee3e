// Recursive-doubling panel exchange for the all-reduce: log2(R) rounds with XOR partners instead of
// a full-mesh fan-out.
//
// Reference behaviour covered: triton_dist/kernels/dcu/gemm_ar_rd.py:399-495 (per row panel: the panel
// GEMM writes the accumulator, then per phase p the current accumulator is pushed to partner
// rank ^ (1 << p), the partner's arrival ticket is awaited, the partner's snapshot is added in place;
// staging slots are recycled under monotonic arrival / ack tickets, never under a barrier) and its
// two kernels, the panel GEMM (:189-246) and the in-place accumulate (:128-160). The reference runs
// the exchange as copy-engine transfers and stream waits issued by the host; here one kernel per
// panel does push, ticket, wait, accumulate and ack for all phases, every CTA owning one slice of
// the panel from the first phase to the last, and every wait carries a limit.
//
// On an NVSwitch fabric the full-mesh two-shot and the switch-reduced all-reduce move fewer bytes
// per rank than log2(R) whole-panel exchanges, so the fused kernel stays the default transport of
// the all-reduce; this transport exists for fabrics (and experiments) where pairwise exchange is
// the better pattern, and is what the "rd" entry points run.
#pragma once
#include <cstdint>
#include <vector>

#include "../common/status.h"

namespace tdb {

constexpr int kRdMaxSlices = 64;   // slices (CTAs) a panel can be cut into; size of a ticket row

struct RdRankArgs {
  void* c;                    // this rank's panel of the accumulator: rows x n_cols, 16-bit
  int64_t ldc;                // row stride of c in elements
  int rows, n_cols;
  int phases;                 // log2(R)
  int slot, slots;            // staging slot of this panel
  int flag_slices;            // ticket row length (>= CTAs of the launch)
  int64_t slot_bytes;         // bytes of one (slot, phase) staging region
  void* scatter;              // own staging: [slots][phases][slot_bytes]
  void* peer_scatter[3];      // the phase partner's staging base
  uint32_t* arrival;          // own tickets [slots][phases][flag_slices], written by the partner
  uint32_t* ack;              // own tickets, same shape: "the partner consumed my push"
  uint32_t* peer_arrival[3];
  uint32_t* peer_ack[3];
  uint32_t ticket;            // this panel's ticket
  uint32_t prev_ticket;       // ticket of the slot's previous occupant (0: none)
  WaitEnv env;
};

// One launch per panel. `ranks` holds one block (one rank per process) or R blocks (virtual ranks
// of a single-GPU test: one cooperative launch, grid.y = rank).
void rd_exchange_launch(const std::vector<RdRankArgs>& ranks, int ctas, bool bf16, void* stream);

}  // namespace tdb

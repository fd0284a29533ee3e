// Plain-C++ interface of the fused GEMM family (no torch / pybind types here).
//
// One plan type covers what the reference implements as separate producer / consumer kernels
// plus host-driven copies per operator: all_gather_gemm.py:98-230 (consumer GEMM gated on arrival
// flags), gemm_reduce_scatter.py:39-135 (producer GEMM, scatter, consumer reduce),
// gemm_allreduce.py:73-181 (producer GEMM, push, consumer reduce), all under
// triton_dist/kernels/dcu/.
#pragma once
#include <array>
#include <cstdint>
#include <cstring>
#include <string>
#include <vector>

namespace tdb {

// All pointers are device addresses passed as integers. Arrays indexed [parity][rank]
// hold the two generations of a double-buffered symmetric buffer: a call with an
// odd round uses parity 1. Because a rank can only enter round n+1 after every
// peer finished round n-1, writes of round n+1 never touch memory a peer still reads.
struct GemmPlanDesc {
  int op = 0, epi = 0, sched = 0;
  int bn = 256;
  bool bf16 = false;
  int rank = 0, R = 1;
  int M = 0, N = 0, K = 0;
  int64_t a = 0, a_rows = 0, lda = 0;
  int64_t b = 0, b_rows = 0, ldb = 0;
  int64_t c = 0, ldc = 0;
  int m_per_rank = 0;
  int seg_order[8] = {0, 1, 2, 3, 4, 5, 6, 7};
  int64_t order_table = 0;
  int order_table_header = 0;   // order_table is part of a full skew table (see gemm_plan_launch, flag bit 3)
  int check_residency = 0;      // refuse a plan whose grid cannot be resident in one wave (needs a device)
  int strided_interleave = 0;
  int seg_bands = 0;        // SCHED_SEGMENT: row bands per segment walked band-major (0 / 1 = source-major)
  int seg_own_first = 0; // band-major walk: the order's first segment whole, then the bands of the others
  int seg_interleave = 0;   // SCHED_SEGMENT: all ranks walk the segments in lockstep (tile k of every segment, then k + 1)
  int64_t tile_list = 0;
  int list_len = 0;
  int swiglu_up_row0 = 0;
  int max_ctas = 0;
  int allow_pair = 1;   // let 256-wide tiles run on CTA pairs (cluster of 2, cta_group::2 MMA)
  int allow_wide = 1;   // let CTA pairs take 512 x 256 tiles (256 rows per CTA) where the rows allow
  int allow_splitk = 1; // let the tiles of the last, partial scheduling round be cut along K
  int raster_g = 0;     // row units walked together (0 = sized so that their A rows stay in L2)
  int l2_ahead = 0;      // k-blocks of L2 look-ahead of the operand loads (0 = none)
  // all-gather
  int64_t peer_ws[2][8] = {};
  int64_t peer_ag_flags[8] = {};
  int64_t peer_ag_arrive[8] = {};   // pull transport: "source staged its chunk" tickets on every rank
  int ag_pull = 0;
  int64_t ag_counters = 0;
  int64_t arrival_ns = 0;
  int chunk_rows = 0, n_chunks = 0, push_parts = 0, skip_comm = 0, push_ctas = 0, push_skip_rounds = 0;
  // reduce-scatter / all-reduce
  int64_t peer_slots[2][8] = {};
  int64_t peer_tile_flags[8] = {};
  int64_t slot_stride = 0;
  // Words between two sources' rows of the ticket planes (0 = this call's own tile / chunk
  // count). A context passes the counts of its LARGEST shape, so that a ticket word keeps one
  // (source, index) meaning for every M the context is called with.
  int ticket_stride = 0;
  int ag_flag_stride = 0;
  int64_t peer_res[2][8] = {};
  int64_t peer_res_flags[8] = {};
  int res_is_c = 0;
  // two-shot all-reduce through the switch (multimem): multicast addresses, by parity, of the
  // partial and result buffers; peer_slots then holds this rank's own partial buffer in every
  // entry and slot_stride is 0
  int nvls = 0;
  int reduce_ctas = 0, reduce_tail = 0;   // reduce-scatter through the switch: steady CTA budget, tail window
  int64_t mc_part[2] = {};
  int64_t mc_res[2] = {};
  // failure reporting
  int64_t prof = 0;       // optional uint64 [grid][16] stall accounting (see ProfSlot)
  int64_t status_dev = 0;
  int64_t abort_word = 0;
  int64_t peer_abort[8] = {};   // the abort word of every rank (raised together when one rank gives up)
  uint64_t timeout_ns = 2000000000ull;
  int probe = 0;          // pipeline probes of the plain GEMM (see GemmParams::probe)
  uint32_t poll_ns = 0;   // pause between two polls of a cross-rank flag
};

int64_t gemm_plan_create(const GemmPlanDesc& d);
void gemm_plan_destroy(int64_t id);
// `order_table`: optional device int32[R] overriding the segment order for this call.
// `flags`: bit 0 = no communication (GEMM only), bit 1 = communication only, bit 2 = publish
// partial tiles but reduce nothing (all-reduce decomposition), bit 3 = order_table is the order[]
// part of a full skew table (4 header words in front, R spin budgets behind).
void gemm_plan_launch(int64_t id, uint32_t round, int parity, int64_t order_table, int flags,
                      void* stream);
// Runs several ranks' plans as ONE cooperative kernel on one GPU (grid.y = rank).
void gemm_plans_launch_emulated(const std::vector<int64_t>& ids, uint32_t round, int parity,
                                int skip_comm, void* stream);

// Host-side replay of the kernel's tile schedule (same functions as the device code, no GPU
// needed): for every CTA of the grid the tiles it would process, in order, as
// {m_tile, n_tile, ticket index, owner key, scheduling position}. `sms` = SMs of the target GPU.
std::vector<std::vector<std::array<int, 5>>> schedule_dump(const GemmPlanDesc& d, int sms);

// The tiles cut along K: {position, first CTA of the worker, slice, slices, first k-block, end k-block}.
std::vector<std::array<int, 6>> splitk_dump(const GemmPlanDesc& d, int sms);

// Sizes of the buffers a plan will touch (0 = not given, that check is skipped).
struct PlanExtents {
  int64_t c_bytes = 0;           // caller's output, from its first element
  int64_t ws_bytes = 0;          // all-gather workspace, one parity
  int64_t slot_bytes = 0;        // partial slots (or the local partial plane), one parity
  int64_t res_bytes = 0;         // all-reduce result plane, one parity
  int64_t ag_flag_words = 0;     // all-gather chunk tickets
  int64_t tile_flag_words = 0;   // tile tickets
  int64_t res_flag_words = 0;    // result tickets
};

// Trap-free bounds check on the host, before any launch: replays the plan's tile schedule with the
// functions the kernel uses and checks every ticket index and every buffer offset the kernel will
// compute against the given extents. Returns one sentence per violation (empty = consistent).
std::vector<std::string> plan_check(const GemmPlanDesc& d, const PlanExtents& e, int sms);

int64_t launch_count();
void launch_count_add(int64_t n);

}  // namespace tdb

// Allocation-free single-GPU MoE dispatch, exported with C linkage.
//
// This entry point has no counterpart in the reference library.
//
// Who it is for: code that must not allocate device memory while it runs --
// a serving loop that has handed all free memory to a KV cache or memory pool,
// a plugin called from inside another framework's allocator callback, a
// real-time path where the latency of cudaMalloc (an implicit device
// synchronisation) is not acceptable, or a host that simply forbids driver
// allocations after start-up. The regular dispatch path keeps its slot cursors
// and segment table in tensors the context allocated; here that scratch lives in
// a fixed array inside the library image instead, so the call needs nothing but
// the caller's own input and output buffers.
//
// What it does: the same job as the metadata + dispatch kernels for one rank
// (num_ranks == 1): rows of `tokens` are copied into `recv`, grouped by expert
// id; within an expert the order is unspecified.
//
//   tokens       [T, H]      16-bit elements (fp16 or bf16; rows are moved as bytes)
//   topk_idx     [T, topk]   int32 expert ids in [0, E); other values are dropped
//   recv         [>= T*topk, H]   output rows, expert e occupies rows
//                            [seg_start[e], seg_start[e] + count(e))
//   scatter_idx  [T, topk]   output: row of each (t, j) in recv, or -1 if dropped
//   seg_start    [E]         output: first row of every expert's segment
//   recv_total   [1]         output: number of rows written
//
// Limits and rules
//   * E <= TDB_NOALLOC_MAX_EXPERTS (1024), topk <= 32, H % 8 == 0, T * topk < 2^31,
//     max_recv_rows >= T * topk; `tokens` and `recv` start on 16-byte boundaries (rows are
//     moved with 16-byte loads and stores; a view at an odd offset is refused instead of
//     faulting on the GPU). Anything else is refused with a negative return code before
//     any kernel is launched; tdb_noalloc_strerror() names the reason.
//   * `stream` must belong to the device that is current in the calling thread: the scratch
//     address is looked up for the current device. The cached address does not outlive a
//     cudaDeviceReset of that device.
//   * The scratch is one file-scope device array of TDB_NOALLOC_SCRATCH_BYTES
//     (8448 bytes) per GPU that loads this library; it stays resident until the
//     process exits.
//   * The first call on each device looks up the array's device address (once per
//     device, with that device current). Make that first call outside any CUDA
//     stream capture.
//   * Every call on a device shares that one array, and it keeps the previous
//     call's contents; each call re-initialises the part it needs. Two calls
//     that overlap on the same GPU (different streams, or different host
//     threads) race on it -- serialise them.
//   * The function calls no cudaMalloc / cudaFree and no library routine that
//     allocates (nothing from torch either); it launches two kernels on `stream`
//     and returns without synchronising.
#pragma once
#include <stdint.h>

#define TDB_NOALLOC_MAX_EXPERTS 1024
#define TDB_NOALLOC_SCRATCH_BYTES (2 * TDB_NOALLOC_MAX_EXPERTS * 4 + 256)

#ifdef __cplusplus
extern "C" {
#endif

// Returns 0 on success, a negative TDB_NOALLOC_E* code otherwise.
int tdb_moe_local_dispatch_noalloc(const void* tokens, const int32_t* topk_idx, void* recv,
                                   int32_t* scatter_idx, int32_t* seg_start, int32_t* recv_total,
                                   int T, int H, int topk, int E, int64_t max_recv_rows,
                                   void* stream);

// Human-readable text for a return code of the function above.
const char* tdb_noalloc_strerror(int code);

#ifdef __cplusplus
}
#endif

#define TDB_NOALLOC_OK 0
#define TDB_NOALLOC_ENULL (-1)       // a required pointer is null
#define TDB_NOALLOC_EEXPERTS (-2)    // E outside [1, TDB_NOALLOC_MAX_EXPERTS]
#define TDB_NOALLOC_ETOPK (-3)       // topk outside [1, 32]
#define TDB_NOALLOC_EHIDDEN (-4)     // H not a positive multiple of 8
#define TDB_NOALLOC_EROWS (-5)       // T < 0, T * topk too large, or recv too small
#define TDB_NOALLOC_ECUDA (-6)       // a CUDA call failed (symbol lookup or launch)
#define TDB_NOALLOC_EALIGN (-7)      // tokens or recv does not start on a 16-byte boundary

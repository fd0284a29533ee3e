// Error-status records shared by host and device code (no device intrinsics here).
#pragma once
#include <cstdint>

namespace tdb {

enum StatusCode : uint32_t {
  ST_OK = 0,
  ST_TIMEOUT_FLAG = 1,     // a cross-rank flag did not reach its ticket in time
  ST_TIMEOUT_MBAR = 2,     // an intra-CTA pipeline barrier did not flip in time
  ST_BAD_INDEX = 3,        // a computed row / tile / ticket index failed its range check; the access was skipped
  ST_OVERFLOW = 4,         // a receive buffer would be oversubscribed
  ST_PEER_ABORT = 5,       // a wait was abandoned because another role or another rank gave up first
};

// Wait sites (the `site` word of the record).
enum WaitSite : uint32_t {
  SITE_AG_CHUNK = 1,
  SITE_RS_TILE = 2,
  SITE_AR_TILE = 3,
  SITE_AR_RESULT = 4,
  SITE_BARRIER = 5,
  SITE_MOE_META = 6,
  SITE_MOE_DISPATCH_DONE = 7,
  SITE_MOE_COMBINE_READY = 8,
  SITE_SPLITK = 9,         // split-K finisher waiting for another slice's partial
  SITE_AG_ARRIVE = 10,     // pull all-gather: waiting for a source to stage its chunk
  SITE_INDEX_CHECK = 11,   // a computed ticket / row / chunk index failed its range check (nothing was accessed)
  SITE_RD_ARRIVAL = 12,    // recursive-doubling exchange: waiting for the partner's panel slice
  SITE_RD_ACK = 13,        // recursive-doubling exchange: waiting for the partner to free a staging slot
  SITE_PIPE_FULL = 16,
  SITE_PIPE_EMPTY = 17,
  SITE_TMEM_FULL = 18,
  SITE_TMEM_EMPTY = 19,
  SITE_TEST = 32,
};

// Lives in pinned, device-mapped host memory: the host can poll it without a
// stream synchronisation. Written only on failure.
struct StatusBlock {
  uint32_t code;
  uint32_t rank;
  uint32_t site;
  uint32_t expected;
  uint32_t seen;
  uint32_t aux;
  uint32_t pad[2];
};

struct WaitEnv {
  StatusBlock* status;      // mapped host memory (may be nullptr)
  uint32_t* abort_word;     // device memory, one word per context; non-zero = give up
  uint64_t timeout_ns;      // limit for a single wait
  uint32_t rank;
  uint32_t poll_ns;         // pause between two polls of a flag (0 = poll back to back)
  // The same word on every rank (the abort buffer is symmetric): a rank that gives up raises all
  // of them, so that its peers leave their waits at once instead of each burning its own limit.
  uint32_t* peer_abort[8];
  uint32_t n_peers;         // entries of peer_abort in use (0 = this rank's word only)
  uint32_t pad_;
};

}  // namespace tdb

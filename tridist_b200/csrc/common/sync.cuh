// Bounded waits and the error-status plane shared by every kernel.
//
// The reference waits inside its kernels with an unbounded hybrid spin on monotonic flags (128
// volatile loads, then one atomic probe: triton_dist/kernels/dcu/all_gather_gemm.py:169-186) or
// with a one-CTA spin kernel / stream wait value (gemm_ar_rd.py:96-125,:167-180), and diagnoses a
// wedge from the host (tests/dbg_rs_big.py). Here the wait itself carries the limit and the
// diagnosis.
//
// No kernel in this library spins without a limit. A wait that runs out writes
// one record {code, rank, site, expected, seen, aux} to the context's status
// block (first writer wins), raises the context-wide abort word that every
// other wait polls, and returns false; callers unwind to their teardown (free
// TMEM, fall through the final CTA barrier) and the kernel ends normally, so
// the CUDA context stays usable and the host can raise a Python exception.
#pragma once
#include "ptx.cuh"
#include "status.h"

namespace tdb {

__device__ __forceinline__ void report_failure(const WaitEnv& env, uint32_t code, uint32_t site,
                                               uint32_t expected, uint32_t seen, uint32_t aux) {
  // the record first, the abort words second: whoever leaves a wait because of the abort word
  // then finds the cause already written
  if (env.status) {
    if (atomicCAS_system(&env.status->code, 0u, code) == 0u) {
      env.status->rank = env.rank;
      env.status->site = site;
      env.status->expected = expected;
      env.status->seen = seen;
      env.status->aux = aux;
      __threadfence_system();
    }
  }
  if (env.abort_word) atomicExch(env.abort_word, code);
  for (uint32_t i = 0; i < env.n_peers && i < 8u; ++i)
    if (env.peer_abort[i] != nullptr && env.peer_abort[i] != env.abort_word)
      st_relaxed_sys(env.peer_abort[i], code);
}

// True when this context's abort word is raised. A wait that leaves for this reason records
// ST_PEER_ABORT unless a cause is already on record (on the rank that gave up first it is), so
// that no rank returns garbage without its host noticing.
__device__ __forceinline__ bool aborted(const WaitEnv& env, uint32_t site = 0u) {
  if (env.abort_word == nullptr) return false;
  const uint32_t v = *reinterpret_cast<volatile uint32_t*>(env.abort_word);
  if (v == 0u) return false;
  if (env.status && atomicCAS_system(&env.status->code, 0u, static_cast<uint32_t>(ST_PEER_ABORT)) == 0u) {
    env.status->rank = env.rank;
    env.status->site = site;
    env.status->expected = 0u;
    env.status->seen = v;
    env.status->aux = 0u;
    __threadfence_system();
  }
  return true;
}

// Spin until *flag >= ticket (monotonic tickets; wrap-safe signed difference). The polls are
// relaxed loads (an acquire per poll would run its cache maintenance hundreds of times while
// the tensor pipeline of the same SM is streaming); one acquire load follows the poll that
// saw the ticket, which is what orders the caller's reads of the published data.
// `batch`: polls between two looks at the abort word and the clock (the spin budget of the
// reference's order table, ag_tr_pred.py:366-375).
__device__ __forceinline__ bool wait_flag_ge(const uint32_t* flag, uint32_t ticket,
                                             const WaitEnv& env, uint32_t site, uint32_t aux,
                                             uint32_t batch = 64u) {
  uint32_t v = ld_relaxed_sys(flag);
  if (static_cast<int32_t>(v - ticket) < 0) {
    const uint64_t t0 = globaltimer_ns();
    uint32_t it = 0;
    if (batch < 1u) batch = 1u;
    while (true) {
      if (env.poll_ns) __nanosleep(env.poll_ns);
      v = ld_relaxed_sys(flag);
      if (static_cast<int32_t>(v - ticket) >= 0) break;
      if (++it >= batch) {
        it = 0;
        if (aborted(env, site)) return false;
        if (globaltimer_ns() - t0 > env.timeout_ns) {
          report_failure(env, ST_TIMEOUT_FLAG, site, ticket, v, aux);
          return false;
        }
        __nanosleep(64);
      }
    }
  }
  v = ld_acquire_sys(flag);          // tickets only grow: still >= ticket
  return static_cast<int32_t>(v - ticket) >= 0;
}

// Wait for an mbarrier phase. The limit is twice that of a flag wait: the pipeline barriers of a
// kernel depend on its flag waits (no operands without the ticket), so when a ticket never
// comes the flag wait is the one that runs out first and names the cause; the pipeline waits
// then leave through the abort word.
__device__ __forceinline__ bool wait_mbar(uint64_t* bar, uint32_t parity, const WaitEnv& env,
                                          uint32_t site, uint32_t aux) {
#pragma unroll 1
  for (int i = 0; i < 32; ++i)
    if (mbar_try_wait(bar, parity)) return true;
  const uint64_t t0 = globaltimer_ns();
  uint32_t it = 0;
  while (true) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((++it & 31u) == 0u) {
      if (aborted(env, site)) return false;
      if (globaltimer_ns() - t0 > 2 * env.timeout_ns + 10000000ull) {
        report_failure(env, ST_TIMEOUT_MBAR, site, parity, 0u, aux);
        return false;
      }
    }
  }
}

}  // namespace tdb

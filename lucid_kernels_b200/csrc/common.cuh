// Shared definitions for the LUCID kernels: problem description, workspace layout, status reporting
// and bounded waits.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include "ptx.cuh"
#include "schedule.h"

namespace lucid {

constexpr int kBlock = 128;          // rows per block == head_dim
constexpr int kTileBytes = 32768;    // one 128 x 128 16-bit tile
constexpr int kHalfBytes = 16384;    // one 64-column panel (or 64-row half) of a tile
constexpr float kLog2e = 1.4426950408889634f;

// status codes written to the status buffer (word 0 = code, words 1.. = location)
enum : int {
  kOk = 0,
  kErrBarrierTimeout = 1,   // an in-CTA mbarrier wait ran out of time
  kErrFlagTimeout = 2,      // a row-block's predecessor was never published
  kErrAborted = 3,          // left early because another CTA reported an error
};

// Control words at the start of the workspace (int32 each).
struct Control {
  int ticket;        // next work item
  int status[7];     // [0] code, [1] chain, [2] row-block, [3] detail, [4] barrier id, [5..6] spare
};

// Element strides (in elements, not bytes) of a (B, N, H, 128) tensor whose last dim is contiguous.
struct Strides {
  long long b, n, h;
};

struct Problem {
  int B, N, H, T;    // T = N / 128
  int C;             // chains = B * H
  int group;         // chains advanced together by the scheduler
  int head;          // leading steps that are scheduled for all chains together before the groups start
  int overlap;       // steps of a group's start that are dealt out alternately with the previous group's end
  int use_diag;      // apply the diagonal-block solve
  int window;        // forward only: number of previous blocks used (< 0: all, 0: none)
  int no_sync;       // skip flag waits (profiling only; results are then meaningless)
  int instrument;    // write per-row-block timestamps
  int reuse_diag;    // the workspace already holds X and lam_inv for this K (host decides)
  float exp_scale;   // log2(e) * k_scale^2: the operator acts on k_scale * K, the kernels read K itself
  float out_scale;   // k_scale^2: factor of dK with respect to the unscaled K
  unsigned long long wait_ns;  // time limit of every device-side wait
};

// ---------------------------------------------------------------------------------------------
// error reporting and bounded waits
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ void report_error(Control* ctl, int code, int chain, int row, int detail, int bar_id) {
  if (atomicCAS(&ctl->status[0], 0, code) == 0) {
    ctl->status[1] = chain;
    ctl->status[2] = row;
    ctl->status[3] = detail;
    ctl->status[4] = bar_id;
    __threadfence();
  }
}

// Wait for an mbarrier phase with a time limit.  Returns false (after flagging the CTA-wide abort
// word) when the limit runs out or another role of this CTA has already given up.  The clock is looked at
// only every few hundred polls, so a limit shorter than that takes effect late; a limit of 0 is exact: a
// wait that is not satisfied at its first poll fails at once (used by the test of this path).
__device__ __forceinline__ bool wait_barrier(uint64_t* bar, uint32_t parity, volatile int* cta_abort, Control* ctl,
                                             unsigned long long limit_ns, int chain, int row, int bar_id) {
  if (mbar_try_wait(bar, parity)) return true;
  if (limit_ns == 0) {      // "do not wait at all": whatever is not ready at once counts as timed out
    *cta_abort = 1;
    report_error(ctl, kErrBarrierTimeout, chain, row, 0, bar_id);
    return false;
  }
  const uint64_t t0 = globaltimer_ns();
  uint32_t spins = 0;
  while (!mbar_try_wait(bar, parity)) {
    if ((++spins & 255u) == 0) {
      if (*cta_abort) return false;
      if (globaltimer_ns() - t0 > limit_ns) {
        *cta_abort = 1;
        report_error(ctl, kErrBarrierTimeout, chain, row, 0, bar_id);
        return false;
      }
    }
  }
  return true;
}

// A row-block is complete when its flag reaches kFlagComplete: set at once by the thread that stored the
// block with TMA, or reached by the storing warps (8 or 16 of them) each adding their share with release
// semantics after their own plain stores.
constexpr int kFlagComplete = 16;

// Wait until the flag reaches kFlagComplete (acquire).  Polls the global status word so that one CTA's
// failure releases every waiter.  Returns the nanoseconds spent waiting through *waited when non-null.
__device__ __forceinline__ bool wait_flag(const int* flag, volatile int* cta_abort, Control* ctl,
                                          unsigned long long limit_ns, int chain, int row, int dep_row,
                                          unsigned long long* waited) {
  if (ld_acquire_gpu(flag) >= kFlagComplete) return true;
  if (limit_ns == 0) {
    *cta_abort = 1;
    report_error(ctl, kErrFlagTimeout, chain, row, dep_row, -1);
    return false;
  }
  const uint64_t t0 = globaltimer_ns();
  uint32_t spins = 0;
  bool ok = true;
  while (ld_acquire_gpu(flag) < kFlagComplete) {
    if ((++spins & 63u) == 0) {
      if (*cta_abort) { ok = false; break; }
      if (ld_relaxed_gpu(&ctl->status[0]) != 0) {
        *cta_abort = 1;
        ok = false;
        break;
      }
      if (globaltimer_ns() - t0 > limit_ns) {
        *cta_abort = 1;
        report_error(ctl, kErrFlagTimeout, chain, row, dep_row, -1);
        ok = false;
        break;
      }
    }
  }
  if (waited) *waited += globaltimer_ns() - t0;
  return ok;
}

// Tiles of an item are visited oldest predecessor first, the newest (tile n - 1) last.  A row-block raises its
// flag only after it has acquired the flags of all its predecessors, so a flag that is up vouches (with its
// acquire) for every block published before it.  Looks once at the flag of tile n - kFlagProbe (row-block
// `probe_row` of the chain whose flags start at `chain_flags`) and returns the number of leading tiles that need
// no flag check of their own: n - kFlagProbe + 1 if that flag is up, else 0.  The proxy fence that must stand
// between an acquire in the generic proxy and TMA loads of the data is issued here when the answer is not 0.
#ifndef LUCID_FLAG_PROBE
#define LUCID_FLAG_PROBE 48
#endif
constexpr int kFlagProbe = LUCID_FLAG_PROBE;
__device__ __forceinline__ int flags_known_up(const int* chain_flags, int n, int probe_row) {
  if (n <= kFlagProbe) return 0;
  if (ld_acquire_gpu(chain_flags + probe_row) < kFlagComplete) return 0;
  fence_proxy_async_all();
  return n - kFlagProbe + 1;
}

// Event trace of one CTA (debugging builds only): role r appends {tag, q, clock} triples.
#ifdef LUCID_TRACE
constexpr int kTraceMax = 8192;
#ifndef LUCID_TRACE_ROLES
#define LUCID_TRACE_ROLES 0xffffffffu       // bit r: role r is traced
#endif
#ifndef LUCID_TRACE_BLOCK
#define LUCID_TRACE_BLOCK 0                 // the first CTA that is traced
#endif
#ifndef LUCID_TRACE_NBLOCKS
#define LUCID_TRACE_NBLOCKS 1               // how many consecutive CTAs are traced (8 role slots each)
#endif
#define LUCID_TR(buf, role, cnt, tag, q)                                              \
  do {                                                                                \
    const unsigned tb_ = blockIdx.x - (LUCID_TRACE_BLOCK);                            \
    if ((((LUCID_TRACE_ROLES) >> (role)) & 1u) && (buf) != nullptr && tb_ < (LUCID_TRACE_NBLOCKS) && (cnt) < kTraceMax) { \
      long long* e_ = (buf) + ((long long)((role) + 8 * tb_) * kTraceMax + (cnt)) * 3; \
      e_[0] = (tag);                                                                  \
      e_[1] = (q);                                                                    \
      e_[2] = clock64();                                                              \
      ++(cnt);                                                                        \
    }                                                                                 \
  } while (0)
#else
#define LUCID_TR(buf, role, cnt, tag, q) do { } while (0)
#endif

__device__ __forceinline__ void named_bar_sync(int id, int nthreads) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(nthreads) : "memory");
}

__device__ __forceinline__ uint64_t desc_advance(uint64_t desc, uint32_t bytes) { return desc + (bytes >> 4); }

}  // namespace lucid

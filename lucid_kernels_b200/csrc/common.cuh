// Shared definitions for the LUCID kernels: problem description, workspace layout, status reporting
// and bounded waits.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include "ptx.cuh"

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
  int overlap;       // steps of the next group interleaved with the end of the current one (2*overlap <= T)
  int use_diag;      // apply the diagonal-block solve
  int window;        // forward only: number of previous blocks used (<= 0: all)
  int no_sync;       // skip flag waits (profiling only; results are then meaningless)
  int instrument;    // write per-row-block timestamps
  int reuse_diag;    // the workspace already holds X and lam_inv for this K (host decides)
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
// word) when the limit runs out or another role of this CTA has already given up.
__device__ __forceinline__ bool wait_barrier(uint64_t* bar, uint32_t parity, volatile int* cta_abort, Control* ctl,
                                             unsigned long long limit_ns, int chain, int row, int bar_id) {
  if (mbar_try_wait(bar, parity)) return true;
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

// A row-block is published by eight warps, each adding 1 to its flag with release semantics after its
// own stores; the block is complete when the flag reaches kFlagComplete.
constexpr int kFlagComplete = 8;

// Wait until the flag reaches kFlagComplete (acquire).  Polls the global status word so that one CTA's
// failure releases every waiter.  Returns the nanoseconds spent waiting through *waited when non-null.
__device__ __forceinline__ bool wait_flag(const int* flag, volatile int* cta_abort, Control* ctl,
                                          unsigned long long limit_ns, int chain, int row, int dep_row,
                                          unsigned long long* waited) {
  if (ld_acquire_gpu(flag) >= kFlagComplete) return true;
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

// Work item t -> (chain, step).  Chains are advanced in groups of `group` (sized so that a group's K and
// Y stay in the L2); inside a group the order is step-major, so an item's predecessors (same chain,
// smaller step) always have smaller tickets.  The first `overlap` steps of group g+1, which are short and
// bound by the chain latency rather than by throughput, are interleaved with the last `overlap` steps of
// group g, so that the machine stays busy while the next group ramps up.  Sequence of segments:
//   solo(0) | mixed(0,1) | solo(1) | mixed(1,2) | ... | solo(last)
// with solo(g) = steps [g ? overlap : 0, last ? T : T - overlap) of group g, and mixed(g-1, g) = for
// x in [0, overlap): step T - overlap + x of group g-1, then step x of group g.
__device__ __forceinline__ bool decode_ticket(int t, int C, int T, int group, int overlap, int& chain, int& step) {
  if (t >= C * T) return false;
  const int ng = (C + group - 1) / group;
  if (ng == 1 || overlap <= 0) {
    const int per = group * T;
    const int g = t / per;
    const int base = g * group;
    const int gsz = min(group, C - base);
    const int tl = t - g * per;
    step = tl / gsz;
    chain = base + tl % gsz;
    return true;
  }
  for (int g = 0; g < ng; ++g) {
    const int base = g * group;
    const int gsz = min(group, C - base);
    if (g > 0) {
      // mixed segment between group g-1 (full size `group`) and group g
      const int per_x = group + gsz;
      const int n_mixed = overlap * per_x;
      if (t < n_mixed) {
        const int x = t / per_x, r = t - x * per_x;
        if (r < group) {
          step = T - overlap + x;
          chain = base - group + r;
        } else {
          step = x;
          chain = base + (r - group);
        }
        return true;
      }
      t -= n_mixed;
    }
    const int lo = g ? overlap : 0;
    const int hi = (g == ng - 1) ? T : T - overlap;
    const int n_solo = (hi - lo) * gsz;
    if (t < n_solo) {
      step = lo + t / gsz;
      chain = base + t % gsz;
      return true;
    }
    t -= n_solo;
  }
  return false;
}

// Event trace of one CTA (debugging builds only): role r appends {tag, q, clock} triples.
#ifdef LUCID_TRACE
constexpr int kTraceMax = 8192;
#define LUCID_TR(buf, role, cnt, tag, q)                                              \
  do {                                                                                \
    if ((buf) != nullptr && blockIdx.x == 0 && (cnt) < kTraceMax) {                   \
      long long* e_ = (buf) + ((long long)(role) * kTraceMax + (cnt)) * 3;            \
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

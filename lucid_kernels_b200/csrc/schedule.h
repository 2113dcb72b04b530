// Order in which the persistent solve kernels take their work items.  Plain integer arithmetic, usable from
// host code as well (the order is what makes the flag waits deadlock-free, so it is checked on the CPU).
#pragma once
#if defined(__CUDACC__)
#define LUCID_HD __host__ __device__ __forceinline__
#else
#define LUCID_HD inline
#endif

namespace lucid {

LUCID_HD int imin(int a, int b) { return a < b ? a : b; }

// Work item t -> (chain, step).  The first `head` steps of ALL chains come first, step-major: those
// row-blocks are short, their chains advance at the pace of the hand-over latency rather than of the
// arithmetic, so as many chains as possible should be in flight, and their K and Y rows are few enough to
// share the L2.  The remaining steps follow in groups of `group` chains (sized so that a group's K and Y
// stay in the L2), step-major inside a group.  An item's predecessors (same chain, smaller step) always
// have smaller tickets.
// With `overlap` > 0 (needs equal groups and at least 2 * overlap steps after the head) the first `overlap`
// of those steps of every group but the first alternate, item by item, with the last `overlap` steps of the
// group before:
// a group's short first row-blocks, which advance at the pace of the hand-over latency, then run beside
// long row-blocks of the previous group that keep the other SMs busy.
LUCID_HD bool decode_ticket(int t, int C, int T, int group, int head, int overlap, int& chain, int& step) {
  if (t >= C * T) return false;
  if (head > T) head = T;
  if (head < 0) head = 0;
  const int n_head = C * head;
  if (t < n_head) {
    step = t / C;
    chain = t - step * C;
    return true;
  }
  t -= n_head;
  const int rest = T - head;          // > 0 here: steps head .. T-1 of every group
  if (overlap > 0 && group < C && C % group == 0 && rest >= 2 * overlap) {
    const int a0 = group * (rest - overlap);
    if (t < a0) {
      step = head + t / group;
      chain = t % group;
      return true;
    }
    t -= a0;
    const int per = group * rest;         // a middle group's merged start + its steps up to rest - overlap
    const int g = imin(1 + t / per, C / group - 1);
    int r = t - (g - 1) * per;
    const int merged = 2 * group * overlap;
    if (r < merged) {
      const int idx = r >> 1, st = idx / group, c = idx - st * group;
      if (r & 1) {
        step = head + st;
        chain = g * group + c;
      } else {
        step = T - overlap + st;
        chain = (g - 1) * group + c;
      }
      return true;
    }
    r -= merged;
    step = head + overlap + r / group;
    chain = g * group + r % group;
    return true;
  }
  const int per = group * rest;
  const int g = t / per;
  const int base = g * group;
  const int gsz = imin(group, C - base);
  const int tl = t - g * per;
  step = head + tl / gsz;
  chain = base + tl % gsz;
  return true;
}

}  // namespace lucid

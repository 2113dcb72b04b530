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

// ---------------------------------------------------------------------------------------------
// dK work items.  Row-block i of a chain streams n = T - 1 (+ 2 with diagonal tiles) tiles: the lower part
// j = 0 .. i-1 (A operand dV_i), with diagonal tiles D1 at j = i, then D2 at j = i (A operand V'_i from here
// on) and the upper part j = i+1 .. T-1.  n_low = number of tiles that use dV_i.  An item covers tiles
// [q0, q1): all of them, or with `split` one half each for two consecutive tickets.  In `follow` order the
// row-blocks come last one first, step-major over the chains (the order in which the reverse solve of the
// same launch publishes them); otherwise chain-major.  With `lower_only` the item ends after the first upper tile.
// ---------------------------------------------------------------------------------------------
LUCID_HD bool dk_item(int ticket, int C, int T, bool follow, bool split, bool diag_tiles, int& chain, int& i,
                      int& n_low, int& q0, int& q1, bool lower_only = false) {
  const int half = split ? (ticket & 1) : 0;
  if (split) ticket >>= 1;
  if (ticket < 0 || ticket >= C * T) return false;
  if (follow) {
    chain = ticket % C;
    i = T - 1 - ticket / C;
  } else if (lower_only) {
    // items shrink with i here: the longest row-blocks of a chain go first, so that the launch ends on short ones
    chain = ticket / T;
    i = T - 1 - ticket % T;
  } else {
    chain = ticket / T;
    i = ticket % T;
  }
  n_low = i + (diag_tiles ? 1 : 0);
  const int n = T - 1 + (diag_tiles ? 2 : 0);
  q0 = 0;
  q1 = n;
  // `lower_only` (needs diag_tiles, no split): the lower part, the two diagonal tiles and the first upper tile
  // (j = i + 1); the rest of the upper part is accumulated by the reverse solve that ran before.
  if (lower_only) q1 = imin(n, n_low + 2);
  if (split) {
    if (half) q0 = n >> 1;
    else q1 = n >> 1;
  }
  return true;
}
// column block of tile q
LUCID_HD int dk_tile_j(int n_low, int q, bool diag_tiles) {
  if (q < n_low) return q;                       // 0 .. i-1, then i (D1)
  return diag_tiles ? q - 1 : q + 1;             // i (D2), i+1 .. | i+1 ..
}
// The single A buffer: loaded before the item's first tile (dV_i if that tile is a lower one, else V'_i) and
// again where the tiles change from lower to upper inside the item; the product issuer waits for a load at
// the same tiles and frees the buffer after the last tile that uses each load.
LUCID_HD bool dk_first_a_is_dv(int q0, int n_low) { return q0 < n_low; }
LUCID_HD bool dk_reloads_a_at(int q, int q0, int n_low) { return q == n_low && q0 < n_low; }
LUCID_HD bool dk_waits_a_at(int q, int q0, int n_low) { return q == q0 || dk_reloads_a_at(q, q0, n_low); }
LUCID_HD bool dk_frees_a_after(int q, int q0, int q1, int n_low) {
  return (q == n_low - 1 && q0 < n_low) || q == q1 - 1;
}

}  // namespace lucid

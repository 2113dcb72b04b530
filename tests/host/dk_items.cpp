// Host check of the dK work items (lucid_kernels_b200/csrc/schedule.h): whole and split items, both ticket
// orders, with and without diagonal tiles.  For every row-block the items together cover each tile exactly
// once with the right column block; inside an item the single A buffer is loaded, waited for and freed the
// same number of times, holds the operand each tile needs (dV_i for lower tiles, V'_i after), and is never
// reloaded before it was freed nor used after it was freed.
#include <cstdio>
#include <vector>
#include "schedule.h"

static int check(int C, int T, bool follow, bool split, bool diag) {
  const int n = T - 1 + (diag ? 2 : 0);
  std::vector<int> seen(C * T * (n > 0 ? n : 1), 0);
  std::vector<int> items(C * T, 0);
  const int tickets = C * T * (split ? 2 : 1);
  int last_rank = -1;
  for (int t = 0; t < tickets; ++t) {
    int chain, i, n_low, q0, q1;
    if (!lucid::dk_item(t, C, T, follow, split, diag, chain, i, n_low, q0, q1)) return 1;
    if (chain < 0 || chain >= C || i < 0 || i >= T || q0 < 0 || q1 > n || q0 > q1) return 2;
    ++items[chain * T + i];
    if (follow) {  // row-blocks never come earlier than the reverse solve publishes them: last one first
      const int rank = T - 1 - i;
      if (rank < last_rank) return 3;
      last_rank = rank;
    }
    int loads = q0 < q1 ? 1 : 0, waits = 0, frees = 0;
    bool holds_dv = lucid::dk_first_a_is_dv(q0, n_low), valid = q0 < q1;
    for (int q = q0; q < q1; ++q) {
      if (lucid::dk_reloads_a_at(q, q0, n_low)) {
        if (valid) return 4;        // reloaded while in use: the producer would wait for a free that never comes
        ++loads;
        holds_dv = false;
        valid = true;
      }
      if (lucid::dk_waits_a_at(q, q0, n_low)) ++waits;
      if (!valid) return 5;
      if (holds_dv != (q < n_low)) return 6;
      const int j = lucid::dk_tile_j(n_low, q, diag);
      const int want = q < n_low ? q : (diag ? q - 1 : q + 1);
      if (j != want || j < 0 || j >= T) return 7;
      if (q < n_low ? (j > i || (j == i && !diag)) : (j < i || (j == i && !diag))) return 8;
      ++seen[(chain * T + i) * (n > 0 ? n : 1) + q];
      if (lucid::dk_frees_a_after(q, q0, q1, n_low)) {
        ++frees;
        valid = false;
      }
    }
    if (loads != waits || loads != frees || valid) return 9;
  }
  int chain, i, n_low, q0, q1;
  if (lucid::dk_item(tickets, C, T, follow, split, diag, chain, i, n_low, q0, q1)) return 10;
  for (int r = 0; r < C * T; ++r) {
    if (items[r] != (split ? 2 : 1)) return 11;
    for (int q = 0; q < n; ++q)
      if (seen[r * n + q] != 1) return 12;
  }
  return 0;
}

// lower_only items (diagonal tiles on, no split, chain-major): every row-block once, the longest first inside a
// chain, tiles 0 .. min(n, n_low + 2) - 1 (lower part, D1, D2, the first upper tile), A buffer balanced.
static int check_lower_only(int C, int T) {
  const int n = T + 1;
  std::vector<int> items(C * T, 0);
  int last_chain = -1, last_i = T;
  for (int t = 0; t < C * T; ++t) {
    int chain, i, n_low, q0, q1;
    if (!lucid::dk_item(t, C, T, false, false, true, chain, i, n_low, q0, q1, true)) return 21;
    if (chain < 0 || chain >= C || i < 0 || i >= T) return 22;
    if (chain != last_chain) { last_chain = chain; last_i = T; }
    if (i != last_i - 1) return 23;             // T-1, T-2, ... 0 inside a chain
    last_i = i;
    ++items[chain * T + i];
    if (n_low != i + 1 || q0 != 0 || q1 != (i + 3 < n ? i + 3 : n)) return 24;
    int loads = 1, waits = 0, frees = 0;
    bool holds_dv = lucid::dk_first_a_is_dv(q0, n_low), valid = true;
    for (int q = q0; q < q1; ++q) {
      if (lucid::dk_reloads_a_at(q, q0, n_low)) {
        if (valid) return 25;
        ++loads; holds_dv = false; valid = true;
      }
      if (lucid::dk_waits_a_at(q, q0, n_low)) ++waits;
      if (!valid || holds_dv != (q < n_low)) return 26;
      const int j = lucid::dk_tile_j(n_low, q, true);
      if (j != (q < n_low ? q : q - 1) || j > i + 1 || j >= T) return 27;
      if (lucid::dk_frees_a_after(q, q0, q1, n_low)) { ++frees; valid = false; }
    }
    if (loads != waits || loads != frees || valid) return 28;
  }
  for (int r = 0; r < C * T; ++r) if (items[r] != 1) return 29;
  return 0;
}

int main() {
  int cases = 0;
  for (int C = 1; C <= 3; ++C)
    for (int T = 1; T <= 40; ++T) {
      const int rc = check_lower_only(C, T);
      if (rc) {
        std::printf("FAIL lower_only C=%d T=%d code %d\n", C, T, rc);
        return 1;
      }
      ++cases;
    }
  for (int C = 1; C <= 3; ++C)
    for (int T = 1; T <= 40; ++T)
      for (int m = 0; m < 8; ++m) {
        const int rc = check(C, T, m & 1, (m >> 1) & 1, (m >> 2) & 1);
        if (rc) {
          std::printf("FAIL C=%d T=%d follow=%d split=%d diag=%d code %d\n", C, T, m & 1, (m >> 1) & 1, (m >> 2) & 1, rc);
          return 1;
        }
        ++cases;
      }
  std::printf("ok %d\n", cases);
  return 0;
}

// Host check of the solve kernels' work-item order (lucid_kernels_b200/csrc/schedule.h): for every
// configuration given on the command line as C,T,group,head,overlap the tickets 0 .. C*T-1 must name every
// (chain, step) exactly once and every chain's steps in increasing order - a CTA that waits for a
// predecessor's flag then only ever waits for a ticket that an earlier, resident CTA holds.
#include <cstdio>
#include <cstdlib>
#include <vector>
#include "schedule.h"

int main(int argc, char** argv) {
  for (int a = 1; a < argc; ++a) {
    int C, T, group, head, overlap;
    if (std::sscanf(argv[a], "%d,%d,%d,%d,%d", &C, &T, &group, &head, &overlap) != 5) return 2;
    std::vector<int> next(C, 0);
    for (int t = 0; t < C * T; ++t) {
      int chain = -1, step = -1;
      if (!lucid::decode_ticket(t, C, T, group, head, overlap, chain, step) || chain < 0 || chain >= C ||
          step != next[chain]) {
        std::printf("FAIL %s ticket %d -> chain %d step %d\n", argv[a], t, chain, step);
        return 1;
      }
      ++next[chain];
    }
    int chain, step;
    if (lucid::decode_ticket(C * T, C, T, group, head, overlap, chain, step)) return 1;
    for (int c = 0; c < C; ++c)
      if (next[c] != T) return 1;
  }
  std::printf("ok %d\n", argc - 1);
  return 0;
}

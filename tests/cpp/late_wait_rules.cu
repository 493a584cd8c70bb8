// Host-only check of the late-wait launch bookkeeping in csrc/kernels/common.cuh: which
// kernels may skip the wait for their predecessor, given what was launched in front of them.
// Launches are simulated by the two effects launch_pdl() has on the bookkeeping.
#include <cstdio>
#include "common.cuh"

namespace lt {
std::atomic<uint64_t> g_ops_launches{0};
int g_pdl_override = -1;
int g_late_chain = 0;
int g_late_side = 0;
unsigned long long g_pdl_seq = 0, g_side_mark = 0;
}  // namespace lt

using namespace lt;

static int failures = 0;
#define EXPECT(cond)                                                    \
  do {                                                                  \
    if (!(cond)) { std::printf("FAILED line %d: %s\n", __LINE__, #cond); ++failures; } \
  } while (0)

// what launch_pdl() does to the bookkeeping
static void launched() { g_late_chain = 0; g_late_side = 0; ++g_pdl_seq; }
// a kernel that asks for late wait, vouching for `n` launches in front of it; returns the verdict
static int ask(int n) {
  const LateWait l = late_wait_begin(n);
  launched();
  late_wait_commit(l);
  return l.on;
}
static void normal() { launched(); }
static void side() { launched(); mark_side_kernel(); }

int main() {
  g_pdl_override = 1;
  normal();
  EXPECT(ask(0) == 0);            // nothing vouched for
  normal();
  EXPECT(ask(1) == 1);            // N C1: independent of N
  EXPECT(ask(1) == 0);            // N C1 C2: C2 vouches for C1 only, N may still run
  normal();
  EXPECT(ask(1) == 1);
  EXPECT(ask(2) == 1);            // N C1 C2 with two launches vouched for
  EXPECT(ask(2) == 0);            // a third one would need three
  normal();
  side();
  EXPECT(ask(0) == 1);            // N S C1: everything is independent of a side kernel
  EXPECT(ask(1) == 1);            // N S C1 C2: C2 vouches for C1, S does not count
  EXPECT(ask(1) == 0);            // C3 would have to vouch for C1 and C2
  side();
  normal();                       // another launch in between: the mark is stale
  EXPECT(ask(0) == 0);
  side();
  EXPECT(ask(1) == 1);
  normal();
  EXPECT(ask(0) == 0);            // the chain's side flag does not outlive a normal launch
  g_pdl_override = 0;             // plain stream order: never late
  side();
  EXPECT(ask(0) == 0);
  EXPECT(ask(3) == 0);
  if (failures == 0) std::printf("RULES_OK\n");
  return failures ? 1 : 0;
}

// Host arithmetic of the scratch arena (csrc/host_layout.h) at the benchmark configurations: region
// order and alignment, queue capacity against the tasks a launch can publish, the addressing limits
// of the dispatch word, and the totals.  No GPU, no CUDA call.
//   layout_test.bin            prints one line per configuration and exits 0 when every check holds
#include <cstdio>
#include <cstdlib>

#include "host_layout.h"

using namespace fdmoe;

static int failures = 0;
#define CHECK(cond)                                                  \
  do {                                                               \
    if (!(cond)) {                                                   \
      ++failures;                                                    \
      std::printf("  FAILED %s (line %d)\n", #cond, __LINE__);       \
    }                                                                \
  } while (0)

struct Case {
  const char* name;
  int H, I, E, K, world, tokens_per_rank;
  bool fits;
};

static void run(const Case& c) {
  Geometry g;
  g.H = c.H; g.I = c.I; g.E = c.E; g.K = c.K; g.world = c.world; g.El = c.E / c.world;
  g.max_tokens_local = g.max_tokens_max = c.tokens_per_rank;
  g.max_tokens_sum = (int64_t)c.tokens_per_rank * c.world;
  g.combine_group = 8;
  const bool ok = FinishGeometry(g, 148);
  std::printf("%s: fits=%d", c.name, (int)ok);
  CHECK(ok == c.fits);
  if (!ok) { std::printf("\n"); return; }
  const ArenaLayout L = MakeLayout(g);
  const double act_gb = (double)g.El * g.cap_rows * g.I * 2 / 1e9;
  std::printf(" cap_rows=%d MT=%d queue_cap=%u arena=%.2f GB activations=%.2f GB\n", g.cap_rows, g.MT, g.queue_cap,
              (double)L.total / 1e9, act_gb);
  // an expert receives at most one row per token of any rank
  CHECK((int64_t)g.cap_rows >= g.max_tokens_sum && g.cap_rows % FDMOE_TILE_M == 0 && g.MT * FDMOE_TILE_M == g.cap_rows);
  CHECK((uint64_t)g.El * g.cap_rows < (1ull << 28));
  // queues: a power of two, at least every task of a launch, with room for the worker count on top
  CHECK((g.queue_cap & (g.queue_cap - 1)) == 0);
  CHECK((uint64_t)g.queue_cap >= WorstCaseQueueTasks(g) + 148);
  // regions in order, none overlapping, aligned for their accesses
  const size_t order[] = {L.ctl, L.expert_cnt, L.landed, L.grp_cnt, L.ffn1_done, L.ffn2_done, L.slots[0], L.slots[1],
                          L.slots[2], L.meta, L.ystage, L.packed, L.total};
  for (size_t i = 0; i + 1 < sizeof(order) / sizeof(order[0]); ++i) CHECK(order[i] <= order[i + 1]);
  CHECK(L.expert_cnt >= sizeof(FdmoeCtl));
  CHECK(L.landed - L.expert_cnt >= (size_t)g.El * 4);
  CHECK(L.grp_cnt - L.landed >= (size_t)g.El * g.MT * 4);
  CHECK(L.ffn1_done - L.grp_cnt >= ((size_t)g.max_tokens_max / g.combine_group + 1) * 4);
  CHECK(L.slots[1] - L.slots[0] >= (size_t)g.queue_cap * sizeof(FdmoeSlot));
  CHECK(L.ystage - L.meta >= (size_t)g.El * g.cap_rows * sizeof(FdmoeRowMeta));
  CHECK(L.packed - L.ystage >= (size_t)g.max_tokens_max * g.K * g.H * 2);
  CHECK(L.total - L.packed >= (size_t)g.El * g.cap_rows * g.H * 2);
  CHECK(L.packed % 1024 == 0 && L.ystage % 1024 == 0 && L.meta % 16 == 0 && L.slots[0] % 16 == 0);
  // the per-launch reset covers the counters and nothing of the queues' slots or the row regions
  CHECK(L.zero_begin >= L.ctl && L.zero_begin < L.expert_cnt && L.zero_end > L.ffn2_done && L.zero_end <= L.slots[0]);
  // a B200 holds the arena, the activations and the rank's expert weights
  const double weights_gb = (double)g.El * 3 * g.H * g.I * 2 / 1e9;
  CHECK((double)L.total / 1e9 + act_gb + weights_gb < 170.0);
}

int main() {
  const Case cases[] = {
      {"cfg1 30B 1x128", 2048, 768, 128, 8, 1, 128, true},
      {"cfg2 30B 1x4096", 2048, 768, 128, 8, 1, 4096, true},
      {"cfg3 30B 8x8192", 2048, 768, 128, 8, 8, 8192, true},
      {"cfg3 30B 2x8192", 2048, 768, 128, 8, 2, 8192, true},
      {"cfg5 235B 8x16384", 4096, 1536, 128, 8, 8, 16384, true},
      {"cfg5 235B 8x64", 4096, 1536, 128, 8, 8, 64, true},
      {"235B 1x2048", 4096, 1536, 128, 8, 1, 2048, true},
      {"tiny 1x0", 256, 128, 8, 2, 1, 0, true},
      {"30B 1x2^21 (more rows than a dispatch word addresses)", 2048, 768, 128, 8, 1, 1 << 21, false},
  };
  for (const Case& c : cases) run(c);
  std::printf(failures ? "FAILED: %d checks\n" : "all checks hold\n", failures);
  return failures ? 1 : 0;
}

// CPU test of the multi-rank rendezvous (csrc/bootstrap.cpp): ranks are forked children, as in the
// reference's fixture (test/multiGPU/cpp/moe/moeDistBaseTest.h:30-104).  No GPU involved.
//   bootstrap_test ok <world>           all ranks join, all-gather and barrier work     -> exit 0
//   bootstrap_test missing <world>      the last rank never joins: everyone times out   -> exit 0 if all fail
//   bootstrap_test mismatch             one rank announces another world size           -> exit 0 if refused
//   bootstrap_test empty                an all-zero id with world 2 is rejected         -> exit 0 if refused
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include <sys/wait.h>
#include <unistd.h>

#include <vector>

#include "../../flash_distributed_moe_b200/csrc/bootstrap.h"

static int RunRank(const uint8_t* uid, int rank, int world, int announced_world, int timeout_ms, bool expect_ok) {
  fdmoe::Bootstrap b;
  const int rc = b.Init(uid, rank, announced_world, timeout_ms);
  if (!expect_ok) {
    // a rank that was admitted before the failure learns of it at the first exchange
    if (rc != 0) return 0;
    int v = rank;
    std::vector<int> all((size_t)announced_world);
    return b.AllGather(&v, all.data(), sizeof(v)) != 0 ? 0 : 1;
  }
  if (rc != 0) return 1;
  struct Blob { int rank; int payload[5]; } mine;
  mine.rank = rank;
  for (int i = 0; i < 5; ++i) mine.payload[i] = rank * 100 + i;
  std::vector<Blob> all((size_t)world);
  for (int rep = 0; rep < 3; ++rep) {
    if (b.AllGather(&mine, all.data(), sizeof(mine)) != 0) return 2;
    for (int r = 0; r < world; ++r)
      if (all[r].rank != r || all[r].payload[4] != r * 100 + 4) return 3;
    if (b.Barrier() != 0) return 4;
  }
  return 0;
}

int main(int argc, char** argv) {
  const char* mode = argc > 1 ? argv[1] : "ok";
  int world = argc > 2 ? atoi(argv[2]) : 4;
  uint8_t uid[128];
  if (fdmoe::MakeUniqueId(uid) != 0) return 10;  // by the parent, before fork, like the reference
  if (!strcmp(mode, "empty")) {
    memset(uid, 0, sizeof(uid));
    fdmoe::Bootstrap b;
    return b.Init(uid, 0, 2, 500) != 0 ? 0 : 1;
  }
  if (!strcmp(mode, "mismatch")) world = 2;
  const bool missing = !strcmp(mode, "missing");
  const int spawned = missing ? world - 1 : world;
  std::vector<pid_t> pids;
  for (int r = 0; r < spawned; ++r) {
    const pid_t pid = fork();
    if (pid == 0) {
      int rc;
      if (missing) rc = RunRank(uid, r, world, world, 1500, /*expect_ok=*/false);
      else if (!strcmp(mode, "mismatch")) rc = RunRank(uid, r, world, r == 1 ? 3 : 2, 3000, /*expect_ok=*/false);
      else rc = RunRank(uid, r, world, world, 20000, true);
      _exit(rc);
    }
    pids.push_back(pid);
  }
  int bad = 0;
  for (pid_t pid : pids) {
    int st = 0;
    waitpid(pid, &st, 0);
    if (!WIFEXITED(st) || WEXITSTATUS(st) != 0) ++bad;
  }
  printf("%s: %d of %d ranks behaved as expected\n", mode, spawned - bad, spawned);
  return bad ? 1 : 0;
}

// Host-side rendezvous for multi-rank launchers: a star of TCP connections
// around rank 0, addressed by the 128-byte unique id.  Replaces the rocSHMEM
// bring-up of the reference (src/hip/kernel/remote/remoteComManager.h:55-87,
// uid produced at src/moeKernelLauncher.cpp:15-30).  No CUDA calls here.
#pragma once
#include <stddef.h>
#include <stdint.h>

#include <vector>

namespace fdmoe {

// Fills a fresh id: magic, IPv4 address, TCP port, random nonce.  Opens no
// persistent resources (safe before fork()).  Returns 0 on success.
int MakeUniqueId(uint8_t out[128]);

class Bootstrap {
 public:
  Bootstrap() = default;
  ~Bootstrap();
  Bootstrap(const Bootstrap&) = delete;
  Bootstrap& operator=(const Bootstrap&) = delete;

  // Rank 0 listens on the id's address, the others connect (with retries) and
  // introduce themselves.  Fails on timeout, on a foreign nonce, or when the
  // ranks disagree about the world size.  Returns 0 on success.
  int Init(const uint8_t uid[128], int rank, int world, int timeout_ms);

  // recv must hold world * bytes; every rank receives all contributions in
  // rank order.  Returns 0 on success.
  int AllGather(const void* send, void* recv, size_t bytes);

  int Barrier();
  void Close();

  int rank() const { return rank_; }
  int world() const { return world_; }

 private:
  int rank_ = 0;
  int world_ = 1;
  int timeout_ms_ = 30000;
  int listen_fd_ = -1;
  int root_fd_ = -1;               // non-root ranks: connection to rank 0
  std::vector<int> peer_fds_;      // rank 0: connection to each rank (index = rank)
};

}  // namespace fdmoe

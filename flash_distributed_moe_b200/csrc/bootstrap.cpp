#include "bootstrap.h"

#include <arpa/inet.h>
#include <errno.h>
#include <fcntl.h>
#include <netinet/in.h>
#include <netinet/tcp.h>
#include <poll.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include <sys/socket.h>
#include <sys/time.h>
#include <time.h>
#include <unistd.h>

namespace fdmoe {
namespace {

constexpr char kMagic[8] = {'F', 'D', 'M', 'O', 'E', 'u', '1', 0};

struct UidFields {
  char magic[8];
  uint32_t ipv4_be;
  uint16_t port_be;
  uint16_t pad;
  uint64_t nonce;
};

struct Hello {
  uint64_t nonce;
  int32_t rank;
  int32_t world;
};

int64_t NowMs() {
  struct timespec ts;
  clock_gettime(CLOCK_MONOTONIC, &ts);
  return (int64_t)ts.tv_sec * 1000 + ts.tv_nsec / 1000000;
}

// Blocking-with-deadline send / receive of exactly n bytes.
int SendAll(int fd, const void* buf, size_t n, int64_t deadline_ms) {
  const char* p = static_cast<const char*>(buf);
  while (n > 0) {
    struct pollfd pfd = {fd, POLLOUT, 0};
    const int64_t left = deadline_ms - NowMs();
    if (left <= 0) return -1;
    const int pr = poll(&pfd, 1, (int)(left > 1000 ? 1000 : left));
    if (pr < 0 && errno != EINTR) return -1;
    if (pr <= 0) continue;
    const ssize_t w = send(fd, p, n, MSG_NOSIGNAL);
    if (w < 0) {
      if (errno == EINTR || errno == EAGAIN) continue;
      return -1;
    }
    p += w;
    n -= (size_t)w;
  }
  return 0;
}

int RecvAll(int fd, void* buf, size_t n, int64_t deadline_ms) {
  char* p = static_cast<char*>(buf);
  while (n > 0) {
    struct pollfd pfd = {fd, POLLIN, 0};
    const int64_t left = deadline_ms - NowMs();
    if (left <= 0) return -1;
    const int pr = poll(&pfd, 1, (int)(left > 1000 ? 1000 : left));
    if (pr < 0 && errno != EINTR) return -1;
    if (pr <= 0) continue;
    const ssize_t r = recv(fd, p, n, 0);
    if (r == 0) return -1;  // peer closed
    if (r < 0) {
      if (errno == EINTR || errno == EAGAIN) continue;
      return -1;
    }
    p += r;
    n -= (size_t)r;
  }
  return 0;
}

void SetNoDelay(int fd) {
  int one = 1;
  setsockopt(fd, IPPROTO_TCP, TCP_NODELAY, &one, sizeof(one));
}

}  // namespace

int MakeUniqueId(uint8_t out[128]) {
  memset(out, 0, 128);
  UidFields f;
  memset(&f, 0, sizeof(f));
  memcpy(f.magic, kMagic, sizeof(kMagic));
  const char* addr = getenv("FLASHMOE_BOOTSTRAP_ADDR");
  struct in_addr ia;
  if (!addr || inet_pton(AF_INET, addr, &ia) != 1) inet_pton(AF_INET, "127.0.0.1", &ia);
  f.ipv4_be = ia.s_addr;

  // Ask the kernel for a free port, then release it: rank 0 binds it again in
  // Bootstrap::Init (SO_REUSEADDR), possibly in another process after fork().
  int fd = socket(AF_INET, SOCK_STREAM, 0);
  if (fd < 0) return -1;
  struct sockaddr_in sa;
  memset(&sa, 0, sizeof(sa));
  sa.sin_family = AF_INET;
  sa.sin_addr.s_addr = f.ipv4_be;
  sa.sin_port = 0;
  socklen_t len = sizeof(sa);
  if (bind(fd, (struct sockaddr*)&sa, sizeof(sa)) != 0 ||
      getsockname(fd, (struct sockaddr*)&sa, &len) != 0) {
    close(fd);
    return -1;
  }
  f.port_be = sa.sin_port;
  close(fd);

  uint64_t nonce = 0;
  int rfd = open("/dev/urandom", O_RDONLY);
  if (rfd >= 0) {
    if (read(rfd, &nonce, sizeof(nonce)) != (ssize_t)sizeof(nonce)) nonce = 0;
    close(rfd);
  }
  if (nonce == 0) nonce = ((uint64_t)getpid() << 32) ^ (uint64_t)NowMs() ^ 0x9E3779B97F4A7C15ull;
  f.nonce = nonce;
  memcpy(out, &f, sizeof(f));
  return 0;
}

Bootstrap::~Bootstrap() { Close(); }

void Bootstrap::Close() {
  for (int fd : peer_fds_)
    if (fd >= 0) close(fd);
  peer_fds_.clear();
  if (root_fd_ >= 0) close(root_fd_);
  if (listen_fd_ >= 0) close(listen_fd_);
  root_fd_ = listen_fd_ = -1;
}

int Bootstrap::Init(const uint8_t uid[128], int rank, int world, int timeout_ms) {
  rank_ = rank;
  world_ = world;
  timeout_ms_ = timeout_ms;
  if (world <= 1) return 0;
  UidFields f;
  memcpy(&f, uid, sizeof(f));
  if (memcmp(f.magic, kMagic, sizeof(kMagic)) != 0 || f.port_be == 0) {
    fprintf(stderr, "[MOE ERROR] bootstrap: unique id is empty or malformed (world size %d)\n", world);
    return -1;
  }
  struct sockaddr_in sa;
  memset(&sa, 0, sizeof(sa));
  sa.sin_family = AF_INET;
  sa.sin_addr.s_addr = f.ipv4_be;
  sa.sin_port = f.port_be;
  const int64_t deadline = NowMs() + timeout_ms;

  if (rank == 0) {
    listen_fd_ = socket(AF_INET, SOCK_STREAM, 0);
    if (listen_fd_ < 0) return -1;
    int one = 1;
    setsockopt(listen_fd_, SOL_SOCKET, SO_REUSEADDR, &one, sizeof(one));
    if (bind(listen_fd_, (struct sockaddr*)&sa, sizeof(sa)) != 0 || listen(listen_fd_, world) != 0) {
      fprintf(stderr, "[MOE ERROR] bootstrap: rank 0 cannot listen: %s\n", strerror(errno));
      return -1;
    }
    peer_fds_.assign(world, -1);
    int connected = 1;
    while (connected < world) {
      struct pollfd pfd = {listen_fd_, POLLIN, 0};
      const int64_t left = deadline - NowMs();
      if (left <= 0) {
        fprintf(stderr, "[MOE ERROR] bootstrap: rank 0 timed out with %d of %d ranks\n", connected, world);
        return -1;
      }
      const int pr = poll(&pfd, 1, (int)(left > 1000 ? 1000 : left));
      if (pr <= 0) continue;
      const int fd = accept(listen_fd_, nullptr, nullptr);
      if (fd < 0) continue;
      SetNoDelay(fd);
      Hello h;
      if (RecvAll(fd, &h, sizeof(h), deadline) != 0 || h.nonce != f.nonce) {
        close(fd);  // stranger: ignore
        continue;
      }
      int32_t verdict = (h.world == world && h.rank > 0 && h.rank < world && peer_fds_[h.rank] < 0) ? 0 : 1;
      SendAll(fd, &verdict, sizeof(verdict), deadline);
      if (verdict != 0) {
        fprintf(stderr, "[MOE ERROR] bootstrap: rank %d announced world size %d, expected %d\n", h.rank,
                h.world, world);
        close(fd);
        return -1;
      }
      peer_fds_[h.rank] = fd;
      ++connected;
    }
    return 0;
  }

  // non-root: connect with retries until rank 0 is listening
  for (;;) {
    if (NowMs() >= deadline) {
      fprintf(stderr, "[MOE ERROR] bootstrap: rank %d could not reach rank 0\n", rank);
      return -1;
    }
    const int fd = socket(AF_INET, SOCK_STREAM, 0);
    if (fd < 0) return -1;
    if (connect(fd, (struct sockaddr*)&sa, sizeof(sa)) == 0) {
      SetNoDelay(fd);
      Hello h = {f.nonce, rank, world};
      int32_t verdict = 1;
      if (SendAll(fd, &h, sizeof(h), deadline) == 0 &&
          RecvAll(fd, &verdict, sizeof(verdict), deadline) == 0 && verdict == 0) {
        root_fd_ = fd;
        return 0;
      }
      close(fd);
      if (verdict != 0) {
        fprintf(stderr, "[MOE ERROR] bootstrap: rank %d was refused by rank 0\n", rank);
        return -1;
      }
    } else {
      close(fd);
    }
    usleep(20000);
  }
}

int Bootstrap::AllGather(const void* send, void* recv, size_t bytes) {
  char* out = static_cast<char*>(recv);
  if (world_ <= 1) {
    memcpy(out, send, bytes);
    return 0;
  }
  const int64_t deadline = NowMs() + timeout_ms_;
  if (rank_ == 0) {
    memcpy(out, send, bytes);
    for (int r = 1; r < world_; ++r)
      if (RecvAll(peer_fds_[r], out + (size_t)r * bytes, bytes, deadline) != 0) return -1;
    for (int r = 1; r < world_; ++r)
      if (SendAll(peer_fds_[r], out, bytes * (size_t)world_, deadline) != 0) return -1;
    return 0;
  }
  if (SendAll(root_fd_, send, bytes, deadline) != 0) return -1;
  return RecvAll(root_fd_, out, bytes * (size_t)world_, deadline);
}

int Bootstrap::Barrier() {
  char token = 1;
  std::vector<char> all((size_t)world_);
  return AllGather(&token, all.data(), 1);
}

}  // namespace fdmoe

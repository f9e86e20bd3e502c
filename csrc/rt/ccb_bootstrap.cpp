#include "ccb_bootstrap.h"

#include <errno.h>
#include <poll.h>
#include <sys/mman.h>
#include <stdio.h>
#include <string.h>
#include <sys/socket.h>
#include <sys/un.h>
#include <time.h>
#include <unistd.h>

namespace ccb {

namespace {

struct WireHeader {
  int32_t type, rank, seq, has_fd;
  uint32_t len;
};

double now_s() {
  timespec ts;
  clock_gettime(CLOCK_MONOTONIC, &ts);
  return ts.tv_sec + ts.tv_nsec * 1e-9;
}

// Abstract-namespace address: sun_path[0] == 0, name follows; no file is created
// and the name disappears with the socket.
socklen_t make_addr(sockaddr_un* a, const std::string& tag, int rank) {
  memset(a, 0, sizeof(*a));
  a->sun_family = AF_UNIX;
  std::string name = "ccb." + tag + "." + std::to_string(rank);
  if (name.size() > sizeof(a->sun_path) - 2) name.resize(sizeof(a->sun_path) - 2);
  memcpy(a->sun_path + 1, name.data(), name.size());
  return (socklen_t)(offsetof(sockaddr_un, sun_path) + 1 + name.size());
}

bool write_all(int fd, const void* p, size_t n) {
  const char* c = static_cast<const char*>(p);
  while (n) {
    ssize_t w = ::send(fd, c, n, MSG_NOSIGNAL);
    if (w < 0) {
      if (errno == EINTR) continue;
      return false;
    }
    c += w;
    n -= (size_t)w;
  }
  return true;
}

bool read_all(int fd, void* p, size_t n) {
  char* c = static_cast<char*>(p);
  while (n) {
    ssize_t r = ::recv(fd, c, n, 0);
    if (r == 0) return false;
    if (r < 0) {
      if (errno == EINTR) continue;
      return false;
    }
    c += r;
    n -= (size_t)r;
  }
  return true;
}

}  // namespace

Bootstrap::Bootstrap(int rank, int nranks, const std::string& tag, int timeout_ms)
    : rank_(rank), nranks_(nranks), timeout_ms_(timeout_ms), tag_(tag) {
  int fd = ::socket(AF_UNIX, SOCK_STREAM | SOCK_CLOEXEC, 0);
  if (fd < 0) {
    err_ = std::string("socket: ") + strerror(errno);
    return;
  }
  sockaddr_un a;
  socklen_t len = make_addr(&a, tag_, rank_);
  if (::bind(fd, reinterpret_cast<sockaddr*>(&a), len) != 0) {
    err_ = std::string("bind ccb.") + tag_ + ": " + strerror(errno);
    ::close(fd);
    return;
  }
  if (::listen(fd, 4 * nranks_ + 16) != 0) {
    err_ = std::string("listen: ") + strerror(errno);
    ::close(fd);
    return;
  }
  listen_fd_ = fd;
}

Bootstrap::~Bootstrap() {
  if (listen_fd_ >= 0) ::close(listen_fd_);
  for (auto& m : inbox_)
    if (m.fd >= 0) ::close(m.fd);
}

bool Bootstrap::send(int peer, int type, int seq, const void* data, size_t len, int fd) {
  sockaddr_un a;
  socklen_t alen = make_addr(&a, tag_, peer);
  const double deadline = now_s() + timeout_ms_ * 1e-3;
  int s = -1;
  for (;;) {
    s = ::socket(AF_UNIX, SOCK_STREAM | SOCK_CLOEXEC, 0);
    if (s < 0) {
      err_ = std::string("socket: ") + strerror(errno);
      return false;
    }
    if (::connect(s, reinterpret_cast<sockaddr*>(&a), alen) == 0) break;
    int e = errno;
    ::close(s);
    if ((e != ECONNREFUSED && e != ENOENT && e != EAGAIN) || now_s() > deadline) {
      err_ = "connect to rank " + std::to_string(peer) + ": " + strerror(e);
      return false;
    }
    usleep(2000);
  }
  WireHeader h{type, rank_, seq, fd >= 0 ? 1 : 0, (uint32_t)len};
  msghdr msg;
  memset(&msg, 0, sizeof(msg));
  iovec iov{&h, sizeof(h)};
  msg.msg_iov = &iov;
  msg.msg_iovlen = 1;
  alignas(cmsghdr) char ctrl[CMSG_SPACE(sizeof(int))];
  if (fd >= 0) {
    memset(ctrl, 0, sizeof(ctrl));
    msg.msg_control = ctrl;
    msg.msg_controllen = sizeof(ctrl);
    cmsghdr* cm = CMSG_FIRSTHDR(&msg);
    cm->cmsg_level = SOL_SOCKET;
    cm->cmsg_type = SCM_RIGHTS;
    cm->cmsg_len = CMSG_LEN(sizeof(int));
    memcpy(CMSG_DATA(cm), &fd, sizeof(int));
  }
  bool good = ::sendmsg(s, &msg, MSG_NOSIGNAL) == (ssize_t)sizeof(h);
  if (good && len) good = write_all(s, data, len);
  if (!good) err_ = std::string("sendmsg: ") + strerror(errno);
  ::close(s);
  return good;
}

// Accept and read at most one connection; false on timeout or error.
bool Bootstrap::pump(int timeout_ms) {
  pollfd p{listen_fd_, POLLIN, 0};
  int pr = ::poll(&p, 1, timeout_ms);
  if (pr <= 0) {
    if (pr == 0) err_ = "rendezvous timed out waiting for a peer";
    else err_ = std::string("poll: ") + strerror(errno);
    return pr < 0 && errno == EINTR;
  }
  int s = ::accept4(listen_fd_, nullptr, nullptr, SOCK_CLOEXEC);
  if (s < 0) {
    err_ = std::string("accept: ") + strerror(errno);
    return false;
  }
  WireHeader h;
  msghdr msg;
  memset(&msg, 0, sizeof(msg));
  iovec iov{&h, sizeof(h)};
  msg.msg_iov = &iov;
  msg.msg_iovlen = 1;
  alignas(cmsghdr) char ctrl[CMSG_SPACE(sizeof(int))];
  msg.msg_control = ctrl;
  msg.msg_controllen = sizeof(ctrl);
  ssize_t r = ::recvmsg(s, &msg, MSG_WAITALL | MSG_CMSG_CLOEXEC);
  if (r != (ssize_t)sizeof(h)) {
    err_ = "short rendezvous header";
    ::close(s);
    return false;
  }
  BootMsg m;
  m.type = h.type;
  m.rank = h.rank;
  m.seq = h.seq;
  for (cmsghdr* cm = CMSG_FIRSTHDR(&msg); cm; cm = CMSG_NXTHDR(&msg, cm))
    if (cm->cmsg_level == SOL_SOCKET && cm->cmsg_type == SCM_RIGHTS) memcpy(&m.fd, CMSG_DATA(cm), sizeof(int));
  if (h.len > (1u << 20)) {
    err_ = "oversized rendezvous message";
    ::close(s);
    return false;
  }
  m.payload.resize(h.len);
  if (h.len && !read_all(s, m.payload.data(), h.len)) {
    err_ = "short rendezvous payload";
    ::close(s);
    return false;
  }
  ::close(s);
  inbox_.push_back(std::move(m));
  return true;
}

bool Bootstrap::recv(int type, int seq, int src, BootMsg* out) {
  const double deadline = now_s() + timeout_ms_ * 1e-3;
  for (;;) {
    for (size_t i = 0; i < inbox_.size(); ++i) {
      const BootMsg& m = inbox_[i];
      if (m.type == type && m.seq == seq && (src < 0 || m.rank == src)) {
        *out = std::move(inbox_[i]);
        inbox_.erase(inbox_.begin() + (long)i);
        return true;
      }
    }
    double left = deadline - now_s();
    if (left <= 0) {
      err_ = "rendezvous timed out (type " + std::to_string(type) + ", seq " + std::to_string(seq) + ")";
      return false;
    }
    if (!pump((int)(left * 1000) + 1)) {
      if (now_s() > deadline) return false;
    }
  }
}

bool Bootstrap::all_gather(int type, int seq, const void* data, size_t len, int fd, std::vector<BootMsg>* out) {
  out->assign((size_t)nranks_, BootMsg());
  for (int j = 1; j < nranks_; ++j)
    if (!send((rank_ + j) % nranks_, type, seq, data, len, fd)) return false;
  for (int j = 1; j < nranks_; ++j) {
    BootMsg m;
    if (!recv(type, seq, -1, &m)) return false;
    if (m.rank < 0 || m.rank >= nranks_) {
      err_ = "rendezvous message from an unknown rank";
      return false;
    }
    (*out)[(size_t)m.rank] = std::move(m);
  }
  return true;
}

bool Bootstrap::barrier(int seq) {
  std::vector<BootMsg> tmp;
  return all_gather(0x7fff, seq, nullptr, 0, -1, &tmp);
}

}  // namespace ccb

// Test hook (host only, no CUDA call): one rendezvous as the communicator set-up does
// it. Every rank all-gathers its rank number together with a descriptor of an anonymous file that
// holds one byte (its rank), reads the byte through each received descriptor, then
// passes the barrier unless `skip_barrier` is set (a rank that leaves between the two
// steps). Returns 0 and the sum of the bytes read, or 1 with the reason in `err`
// when a step ran out of `timeout_ms`: how a rank that never joins, or that dies
// half-way, shows up on the others, on the host, before any kernel is launched.
extern "C" int ccb_test_bootstrap_exchange(int rank, int nranks, const char* tag, int timeout_ms, int skip_barrier,
                                           int* sum_out, char* err, int err_len) {
  auto fail = [&](const std::string& why) {
    if (err && err_len > 0) snprintf(err, (size_t)err_len, "%s", why.c_str());
    return 1;
  };
  ccb::Bootstrap b(rank, nranks, tag ? tag : "test", timeout_ms);
  if (!b.ok()) return fail("listen: " + b.error());
  const int mfd = memfd_create("ccb_test", MFD_CLOEXEC);
  if (mfd < 0) return fail("memfd_create");
  const unsigned char mine = (unsigned char)rank;
  if (write(mfd, &mine, 1) != 1) return fail("write");
  std::vector<ccb::BootMsg> all;
  const int32_t me = rank;
  const bool ok = b.all_gather(1, 0, &me, sizeof(me), mfd, &all);
  close(mfd);
  if (!ok) return fail("all_gather: " + b.error());
  int sum = rank;
  for (int r = 0; r < nranks; ++r) {
    if (r == rank) continue;
    const ccb::BootMsg& m = all[(size_t)r];
    int32_t who = -1;
    if (m.payload.size() == sizeof(who)) memcpy(&who, m.payload.data(), sizeof(who));
    unsigned char byte = 0xff;
    if (who != r || m.fd < 0 || pread(m.fd, &byte, 1, 0) != 1 || byte != (unsigned char)r) return fail("bad message from a peer");
    close(m.fd);
    sum += byte;
  }
  if (sum_out) *sum_out = sum;
  if (skip_barrier) return 0;
  if (!b.barrier(1)) return fail("barrier: " + b.error());
  return 0;
}

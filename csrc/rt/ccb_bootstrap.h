// Rendezvous between the ranks of one host: small messages, optionally carrying a
// file descriptor (SCM_RIGHTS), over abstract-namespace Unix sockets. Used once per
// communicator to exchange CUDA VMM handles; no MPI and no NCCL call is needed, so
// it also works inside an LD_PRELOAD library.
//
// The reference bootstraps through files in a shared directory plus a TCP star
// (run_codes/benchmark-core/src/nccl/nccl_utils.c:71-115, :222-327) and needs no
// handle exchange because it owns no peer memory.
#pragma once
#include <stdint.h>

#include <string>
#include <vector>

namespace ccb {

struct BootMsg {
  int type = 0;
  int rank = 0;
  int seq = 0;
  int fd = -1;  // received descriptor, or -1
  std::vector<uint8_t> payload;
};

class Bootstrap {
 public:
  Bootstrap(int rank, int nranks, const std::string& tag, int timeout_ms);
  ~Bootstrap();
  bool ok() const { return listen_fd_ >= 0; }
  const std::string& error() const { return err_; }

  // Send one message to `peer` (connect, retrying until the peer is listening).
  bool send(int peer, int type, int seq, const void* data, size_t len, int fd);
  // Block until a message of (type, seq) from `src` (or any rank if src < 0) is
  // here; earlier messages of other kinds are kept for later calls.
  bool recv(int type, int seq, int src, BootMsg* out);
  // Everybody sends `len` bytes (and optionally a descriptor) to everybody.
  bool all_gather(int type, int seq, const void* data, size_t len, int fd, std::vector<BootMsg>* out);
  bool barrier(int seq);

 private:
  bool pump(int timeout_ms);
  int rank_, nranks_, timeout_ms_;
  std::string tag_, err_;
  int listen_fd_ = -1;
  std::vector<BootMsg> inbox_;
};

}  // namespace ccb

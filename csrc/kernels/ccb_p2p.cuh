// Point-to-point transfers over peer memory: ncclSend / ncclRecv without NCCL.
//
// The reference's wrapper that replaces NCCL altogether does its sends and receives with
// an RDMA engine (userconfig/wrapper_code_examples/communication/nccl_via_uccl/
// nccl_via_uccl.cu:751-790: register the buffer, send_async / recv_async, busy poll). Inside
// an NVSwitch node the transport is the peer arena: the sender stores into a mailbox in the
// receiver's arena and bumps a counter there; the receiver copies out and bumps an
// acknowledgement counter in the sender's arena.
//
// One launch carries up to kP2pMaxOps operations of one rank (the sends and receives of an
// ncclGroupStart/End, or a single call): blockIdx.y selects the operation, the kP2pLanes
// CTAs of an operation are lanes that each move their own strip of every round, so the two
// ends synchronise lane by lane and never grid-wide. A round moves kP2pLanes * lane_bytes
// bytes; the mailbox of a (source, lane) pair has two halves, so the sender may run one
// round ahead of the receiver. Counters count rounds since the communicator was made and
// never reset; both ends derive the same numbers from the message size. Every wait is
// bounded (communicator time limit) and reports through the status words.
#pragma once
#include "ccb_reduce.cuh"

namespace ccb {

constexpr int kP2pLanes = 16;
constexpr int kP2pMaxOps = 16;
constexpr int kP2pCtrlData = 256;                              // ctrl words [256, 256 + 8*16): rounds delivered by (source, lane)
constexpr int kP2pCtrlAck = kP2pCtrlData + CCB_MAX_RANKS * kP2pLanes;  // rounds consumed by (destination, lane), in the SENDER's arena

struct P2pOp {
  void* buf;                 // user buffer (source of a send, destination of a receive)
  unsigned long long bytes;
  unsigned int first_round;  // rounds this (me -> peer) or (peer -> me) direction carried before this message
  int peer;
  int is_recv;
};
struct P2pArgs {
  CommDev c;
  P2pOp op[kP2pMaxOps];
  unsigned long long box_offset;  // arena offset of the mailboxes: [source][lane][half][lane_bytes]
  unsigned int lane_bytes;        // multiple of 16
  int rank, nops;
};

__device__ __forceinline__ bool p2p_wait(const uint32_t* ctr, uint32_t target, const CommDev& c, char* my, int where) {
  uint64_t t0 = 0;
  uint32_t polls = 0;
  for (;;) {
    const uint32_t v = ld_acquire_sys(ctr);
    if ((int32_t)(v - target) >= 0) return true;
    if ((++polls & 0x3f) == 0) {
      if (t0 == 0) t0 = globaltimer_ns();
      if ((globaltimer_ns() - t0) > c.timeout_ns || polls > (1u << 30)) {
        if (c.status) {
          atomicOr(c.status + CCB_STATUS_FLAGS, CCB_ST_TIMEOUT);
          if (atomicCAS(c.status + CCB_STATUS_WHERE, 0u, (uint32_t)where | 0x80000000u) == 0u) {
            c.status[CCB_STATUS_EPOCH] = target;
            c.status[CCB_STATUS_SEEN] = v;
          }
        }
        return false;
      }
    }
    __nanosleep(100);
  }
}

__global__ void __launch_bounds__(kThreads, 2) p2p_kernel(const __grid_constant__ P2pArgs a) {
  __shared__ int ok;
  const CommDev& c = a.c;
  const P2pOp& op = a.op[blockIdx.y];
  const int lane = blockIdx.x, r = a.rank, p = op.peer;
  char* my = c.arena[r];
  const size_t round_bytes = (size_t)kP2pLanes * a.lane_bytes;
  const uint32_t rounds = (uint32_t)((op.bytes + round_bytes - 1) / round_bytes);
  // mailbox of (source s, lane) in the arena of the receiver
  auto box = [&](char* arena, int s, uint32_t g) {
    return arena + a.box_offset + (((size_t)s * kP2pLanes + lane) * 2 + (g & 1u)) * a.lane_bytes;
  };
  for (uint32_t k = 0; k < rounds; ++k) {
    const uint32_t g = op.first_round + k;                      // round number of this direction since the start
    const size_t off = (size_t)k * round_bytes + (size_t)lane * a.lane_bytes;
    const size_t n = off >= op.bytes ? 0 : (op.bytes - off < a.lane_bytes ? op.bytes - off : a.lane_bytes);
    if (!op.is_recv) {
      // the half is free once the receiver has consumed round g - 2
      if (threadIdx.x == 0) ok = g < 2 || p2p_wait(ctrl_ptr(my, kP2pCtrlAck + p * kP2pLanes + lane), g - 1, c, my, 0xC0 | (p << 8));
      __syncthreads();
      if (!ok) return;
      const char* src = static_cast<const char*>(op.buf) + off;
      char* dst = box(c.arena[p], r, g);
      if ((reinterpret_cast<uintptr_t>(src) & 15) == 0) {
        for (size_t i = (size_t)threadIdx.x * 16; i + 16 <= n; i += (size_t)kThreads * 16) stg(dst + i, ldg_stream(src + i));
        for (size_t i = (n & ~(size_t)15) + threadIdx.x; i < n; i += kThreads) dst[i] = src[i];
      } else {
        for (size_t i = threadIdx.x; i < n; i += kThreads) dst[i] = src[i];
      }
      __syncthreads();
      if (threadIdx.x == 0) signal_flag(ctrl_ptr(c.arena[p], kP2pCtrlData + r * kP2pLanes + lane), g + 1);
    } else {
      if (threadIdx.x == 0) ok = p2p_wait(ctrl_ptr(my, kP2pCtrlData + p * kP2pLanes + lane), g + 1, c, my, 0xD0 | (p << 8));
      __syncthreads();
      if (!ok) return;
      const char* src = box(my, p, g);
      char* dst = static_cast<char*>(op.buf) + off;
      if ((reinterpret_cast<uintptr_t>(dst) & 15) == 0) {
        for (size_t i = (size_t)threadIdx.x * 16; i + 16 <= n; i += (size_t)kThreads * 16) stg_stream(dst + i, ldg_cg(src + i));
        for (size_t i = (n & ~(size_t)15) + threadIdx.x; i < n; i += kThreads) dst[i] = src[i];
      } else {
        for (size_t i = threadIdx.x; i < n; i += kThreads) dst[i] = src[i];
      }
      __syncthreads();  // every thread has read the half before it is handed back
      if (threadIdx.x == 0) signal_flag(ctrl_ptr(c.arena[p], kP2pCtrlAck + r * kP2pLanes + lane), g + 1);
    }
  }
}

}  // namespace ccb

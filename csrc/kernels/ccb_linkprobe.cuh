// Link probe: how fast can this GPU write into a peer's arena, by store method?
//
// The fused collectives move every byte with stores issued by SMs, so the rate of such
// stores is their roofline; a copy-engine transfer (cudaMemcpyPeer) is only the reference.
// The probe writes `bytes` of register-generated data from this rank into the data area of
// one peer's arena (no collective may be in flight) with one of:
//   method 0   st.global.v4 per lane: a warp stores 512 contiguous bytes per instruction
//   method 1   the same bytes staged in shared memory and sent by the TMA unit as untiled
//              bulk copies (cp.async.bulk.global.shared::cta) of 512 bytes per warp
//   method 2   bulk copies of 2 KB per warp (two stages per warp: 128 KB of shared memory)
// The bulk copy is a store from this CTA's shared memory: no multicast, no load from a peer.
// Completion is awaited with cp.async.bulk.wait_group by the lane that issued the copies.
#pragma once
#include "ccb_device.cuh"

namespace ccb {

struct LinkProbeArgs {
  char* dst;                 // peer arena + data offset
  unsigned long long bytes;  // multiple of 8192
  int method;
};

__device__ __forceinline__ void bulk_store(void* gdst, const void* ssrc, unsigned int bytes) {
  asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(gdst),
               "r"((unsigned)__cvta_generic_to_shared(ssrc)), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void bulk_wait_read() { asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory"); }
__device__ __forceinline__ void bulk_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }
__device__ __forceinline__ void fence_proxy_async_shared() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

constexpr int kProbeThreads = 1024;
constexpr int kProbeStages = 2;

__global__ void __launch_bounds__(kProbeThreads, 1) link_probe_kernel(const LinkProbeArgs a) {
  extern __shared__ __align__(128) char probe_smem[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const size_t nwarps = (size_t)gridDim.x * (kProbeThreads / 32), gw = (size_t)blockIdx.x * (kProbeThreads / 32) + warp;
  const uint4 v = make_uint4(threadIdx.x, blockIdx.x, 0x3f800000u, lane);
  if (a.method == 0) {
    for (size_t off = gw * 512; off < a.bytes; off += nwarps * 512) stg(a.dst + off + lane * 16, v);
    return;
  }
  const unsigned int chunk = a.method == 1 ? 512u : 2048u;
  char* stage = probe_smem + (size_t)warp * kProbeStages * chunk;
  int s = 0;
  for (size_t off = gw * chunk; off < a.bytes; off += nwarps * chunk) {
    // the stage is reused once the copy that read it has read it
    if (lane == 0) bulk_wait_read<kProbeStages - 1>();
    __syncwarp();
    char* buf = stage + (size_t)s * chunk;
    for (unsigned int o = lane * 16; o < chunk; o += 512) *reinterpret_cast<uint4*>(buf + o) = v;
    fence_proxy_async_shared();
    __syncwarp();
    if (lane == 0) {
      bulk_store(a.dst + off, buf, chunk);
      bulk_commit();
    }
    s = (s + 1) % kProbeStages;
  }
  if (lane == 0) bulk_wait_all();
}

}  // namespace ccb

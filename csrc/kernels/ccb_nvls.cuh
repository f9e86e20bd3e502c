// Uncompressed AllReduce through the NVSwitch's in-fabric reduction (NVLS):
// stage the input in the symmetric arena, have each rank pull the switch-reduced
// values of its own shard with multimem.ld_reduce and push them to every arena
// with multimem.st, then copy out. These are plain loads and stores on a multicast
// mapping issued from the SMs; no TMA and no cluster multicast is involved.
//
// This is the uncompressed baseline path (the reference's wrapper mode 0 is bare
// ncclAllReduce: userconfig/config_in_jsonc/communication_lib_selection.jsonc:5-7).
#pragma once
#include "ccb_reduce.cuh"

namespace ccb {

template <class T> struct Multimem;
template <> struct Multimem<float> {
  static __device__ __forceinline__ uint4 ld_reduce(const void* p) {
    uint4 v;
    asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
    return v;
  }
};
template <> struct Multimem<__nv_bfloat16> {
  static __device__ __forceinline__ uint4 ld_reduce(const void* p) {
    uint4 v;
    asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
    return v;
  }
};
template <> struct Multimem<__half> {
  static __device__ __forceinline__ uint4 ld_reduce(const void* p) {
    uint4 v;
    asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.f16x2 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
    return v;
  }
};
__device__ __forceinline__ void multimem_st(void* p, uint4 v) {
  asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}

// count is a multiple of 16 bytes' worth of elements per shard (the host pads the
// staging extent); shard_pad elements per shard, areas: in = half, out = half + n*slot.
template <class T>
__global__ void __launch_bounds__(kThreads, 2) nvls_allreduce_kernel(const __grid_constant__ ReduceArgs a) {
  __shared__ CtaSync sync;
  const CommDev& c = a.c;
  const int r = a.rank0, n = c.nranks;  // one rank per launch: multicast needs real peers
  const int b = blockIdx.x, G = gridDim.x;
  const T* send = static_cast<const T*>(a.send[0]);
  T* recv = static_cast<T*>(a.recv[0]);
  char* my = c.arena[r];
  const size_t half = CCB_DATA_OFFSET + (size_t)(c.epoch & 1u) * c.half_bytes;
  const size_t area_in = half, area_out = half + (size_t)n * a.slot_bytes;
  constexpr int kVec = 16 / sizeof(T);                 // elements per 16-byte vector
  constexpr size_t kTileVecs = kThreads * 4;           // vectors per tile
  const size_t shard_vecs = a.shard_pad / kVec;
  if (threadIdx.x == 0) sync.fail = 0;
  __syncthreads();

  auto shard_valid = [&](int s) -> size_t {
    const size_t beg = (size_t)s * a.shard_elems;
    if (beg >= a.count) return 0;
    const size_t left = a.count - beg;
    return left < a.shard_elems ? left : a.shard_elems;
  };

  // 1. stage: send -> own arena (zero-filled past the end so the switch adds zeros)
  for (int s = 0; s < n; ++s) {
    const size_t valid = shard_valid(s);
    const T* src = send + (size_t)s * a.shard_elems;
    char* dst = my + area_in + (size_t)s * a.slot_bytes;
    for (size_t t = b; t * kTileVecs < shard_vecs; t += G) {
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const size_t vi = t * kTileVecs + (size_t)u * kThreads + threadIdx.x;
        if (vi >= shard_vecs) continue;
        const size_t e0 = vi * kVec;
        uint4 x = make_uint4(0, 0, 0, 0);
        if (e0 + kVec <= valid && ((reinterpret_cast<uintptr_t>(src + e0) & 15) == 0)) {
          x = ldg_stream(src + e0);
        } else {
          T* h = reinterpret_cast<T*>(&x);
          for (int i = 0; i < kVec; ++i)
            if (e0 + i < valid) h[i] = src[e0 + i];
        }
        stg(dst + vi * 16, x);
      }
    }
  }
  // the barrier orders every thread's stores before thread 0's single fence
  __syncthreads();
  if (threadIdx.x == 0) signal_peers(c, ((1u << n) - 1u) & ~(1u << r), 0, r, b);
  if (!cta_wait_sources(sync, c, my, 0, r, 0xffu, 0x80)) return;

  // 2. own shard: reduce in the switch, broadcast through the switch
  {
    const char* mc_in = c.mc_arena + area_in + (size_t)r * a.slot_bytes;
    char* mc_out = c.mc_arena + area_out + (size_t)r * a.slot_bytes;
    for (size_t t = b; t * kTileVecs < shard_vecs; t += G) {
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const size_t vi = t * kTileVecs + (size_t)u * kThreads + threadIdx.x;
        if (vi >= shard_vecs) continue;
        uint4 x = Multimem<T>::ld_reduce(mc_in + vi * 16);
        multimem_st(mc_out + vi * 16, x);
      }
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) signal_peers(c, ((1u << n) - 1u) & ~(1u << r), 1, r, b);
  if (!cta_wait_sources(sync, c, my, 1, r, 0xffu, 0x90)) return;

  // 3. copy out of the own arena
  for (int s = 0; s < n; ++s) {
    const size_t valid = shard_valid(s);
    T* dst = recv + (size_t)s * a.shard_elems;
    const char* src = my + area_out + (size_t)s * a.slot_bytes;
    for (size_t t = b; t * kTileVecs < shard_vecs; t += G) {
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const size_t vi = t * kTileVecs + (size_t)u * kThreads + threadIdx.x;
        if (vi >= shard_vecs) continue;
        const size_t e0 = vi * kVec;
        if (e0 >= valid) continue;
        uint4 x = ldg_cg(src + vi * 16);
        if (e0 + kVec <= valid && ((reinterpret_cast<uintptr_t>(dst + e0) & 15) == 0)) {
          stg_stream(dst + e0, x);
        } else {
          const T* h = reinterpret_cast<const T*>(&x);
          for (int i = 0; i < kVec; ++i)
            if (e0 + i < valid) dst[e0 + i] = h[i];
        }
      }
    }
  }
}

// The same reduction IN PLACE on buffers that live inside the symmetric arena (allocated
// with ccb_comm_symm_alloc at the same offset on every rank): no staging copy in, no copy
// out. Each rank pulls the switch-reduced values of its own 1/n of the vectors straight
// from everybody's input (multimem.ld_reduce) and pushes them into everybody's output
// (multimem.st). Two all-rank flag rounds bracket it: inputs complete before anyone
// reads, outputs complete before anyone returns. send_off == recv_off is allowed: the
// vectors a rank reads and writes belong to no other rank's share.
template <class T>
__global__ void __launch_bounds__(kThreads, 2) nvls_inplace_kernel(const __grid_constant__ ReduceArgs a) {
  __shared__ CtaSync sync;
  const CommDev& c = a.c;
  const int r = a.rank0, n = c.nranks;
  const int b = blockIdx.x, G = gridDim.x;
  char* my = c.arena[r];
  const size_t send_off = (size_t)a.shard_elems, recv_off = (size_t)a.shard_pad;  // byte offsets inside the arena
  const size_t vecs = (a.count * sizeof(T) + 15) / 16;                            // the host pads allocations to 16 bytes
  const size_t per = (vecs + n - 1) / n, lo = (size_t)r * per, hi = lo + per < vecs ? lo + per : vecs;
  if (threadIdx.x == 0) sync.fail = 0;
  __syncthreads();
  const uint32_t peers = ((1u << n) - 1u) & ~(1u << r);
  // first flag exchange: what earlier kernels of this stream wrote into the input is visible everywhere
  if (threadIdx.x == 0) signal_peers(c, peers, 0, r, b);
  if (!cta_wait_sources(sync, c, my, 0, r, 0xffu, 0x88)) return;
  const char* mc_in = c.mc_arena + send_off;
  char* mc_out = c.mc_arena + recv_off;
  constexpr size_t kTileVecs = kThreads * 4;
  for (size_t t0 = lo + (size_t)b * kTileVecs; t0 < hi; t0 += (size_t)G * kTileVecs) {
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const size_t vi = t0 + (size_t)u * kThreads + threadIdx.x;
      if (vi >= hi) continue;
      const uint4 x = Multimem<T>::ld_reduce(mc_in + vi * 16);
      multimem_st(mc_out + vi * 16, x);
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) signal_peers(c, peers, 1, r, b);
  if (!cta_wait_sources(sync, c, my, 1, r, 0xffu, 0x98)) return;
}

}  // namespace ccb

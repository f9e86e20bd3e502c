// Warp-specialised, software-pipelined two-shot AllReduce / ReduceScatter for large
// messages: the same wire protocol as reduce_kernel (ccb_reduce.cuh), but the three
// phases of a wave run on different warps of a CTA, so the NVLink-bound phases and
// the HBM-bound decode overlap instead of alternating.
//
//   link warps    P1(w+1): quantise, store lanes into the owners' arenas     (NVLink out)
//                 P2(w)  : reduce own shard, requantise once, store to peers (NVLink out;
//                          ONE multimem.st per lane where the arenas have an NVLS mapping)
//   decode warps  P3(w)  : decode the reduced shards into recv               (HBM only)
//                 (ReduceScatter: they run the reduction P2 instead; there is no P3)
//   signal warp   (the last of the CTA's 32) owns every fence.acq_rel.sys + flag store: the link warps hand a phase
//                 over through a shared-memory counter and go on storing, so the
//                 20 us a system fence costs under store load is off their path.
//
// Flag row 2w carries phase 1 of wave w, row 2w+1 phase 2, as in reduce_kernel. Inside a
// role group the first warp polls the peers' flags and publishes "wave w is ready" in
// shared memory; the other warps of the group spin there, not on global memory.
//
// The reference does this job as 2(n-1) host-driven hops of quantize kernel, ncclSend,
// ncclRecv, dequantize kernel, cudaStreamSynchronize, reduce kernel
// (userconfig/wrapper_code_examples/communication/plain_nccl_compress/
// plain_nccl_compress.cu:682-773 AllReduce, :970-1076 ReduceScatter).
#pragma once
#include "ccb_reduce.cuh"

namespace ccb {

constexpr int kPipeChunkShift = 3;                    // a CTA owns runs of 8 units (4096 elements)
constexpr int kPipeChunkUnits = 1 << kPipeChunkShift;

struct PipeShared {
  // Warp arrivals after phase 1 / phase 2 of each wave. One counter per wave: warps drift
  // apart by more than a wave, so a running total would mix arrivals of different waves.
  unsigned int p1_done[CCB_MAX_SLOTS / 2];
  unsigned int p2_done[CCB_MAX_SLOTS / 2];
  unsigned int p1_ready;   // waves whose phase-1 flags from all peers have been seen
  unsigned int p2_ready;   // the same for phase 2
  int fail;
  // kb[s][w]: first chunk (of this CTA's chunks of shard s) that belongs to wave w; computed
  // once per launch, so that the phases do no division (a 64-bit division per phase, peer
  // and wave cost more instructions than the data loops of a warp)
  unsigned int kb[CCB_MAX_RANKS][CCB_MAX_SLOTS / 2 + 1];
};

__device__ __forceinline__ unsigned int ld_acquire_cta_shared(const unsigned int* p) {
  unsigned int v;
  asm volatile("ld.acquire.cta.shared.u32 %0, [%1];" : "=r"(v) : "r"((unsigned)__cvta_generic_to_shared(p)) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_cta_shared(unsigned int* p, unsigned int v) {
  asm volatile("st.release.cta.shared.u32 [%0], %1;" ::"r"((unsigned)__cvta_generic_to_shared(p)), "r"(v) : "memory");
}
__device__ __forceinline__ void red_release_cta_shared_add(unsigned int* p, unsigned int v) {
  asm volatile("red.release.cta.shared.add.u32 [%0], %1;" ::"r"((unsigned)__cvta_generic_to_shared(p)), "r"(v) : "memory");
}
__device__ __forceinline__ int ld_volatile_shared_int(const int* p) {
  int v;
  asm volatile("ld.volatile.shared.s32 %0, [%1];" : "=r"(v) : "r"((unsigned)__cvta_generic_to_shared(p)) : "memory");
  return v;
}
__device__ __forceinline__ void st_volatile_shared_int(int* p, int v) {
  asm volatile("st.volatile.shared.s32 [%0], %1;" ::"r"((unsigned)__cvta_generic_to_shared(p)), "r"(v) : "memory");
}

// Lane 0 of the calling warp waits until the shared counter reaches `target`; the whole
// warp learns the verdict. Gives up when another warp of the CTA failed, when the abort
// word carries this epoch, or after the communicator's time limit; never traps.
__device__ __forceinline__ bool warp_wait_counter(const unsigned int* ctr, unsigned int target, PipeShared& sh,
                                                  const CommDev& c, char* my_arena, int where) {
  int ok = 1;
  if ((threadIdx.x & 31) == 0) {
    uint64_t t0 = 0;
    uint32_t polls = 0;
    while ((int)(ld_acquire_cta_shared(ctr) - target) < 0) {
      if (ld_volatile_shared_int(&sh.fail)) { ok = 0; break; }
      if ((++polls & 0x3f) == 0) {
        if (t0 == 0) t0 = globaltimer_ns();
        const bool aborted = ld_relaxed_sys(ctrl_ptr(my_arena, CCB_CTRL_ABORT)) == c.epoch;
        const bool late = (globaltimer_ns() - t0) > c.timeout_ns || polls > (1u << 30);
        if (aborted || late) {
          if (c.status) {
            atomicOr(c.status + CCB_STATUS_FLAGS, aborted ? CCB_ST_ABORTED : CCB_ST_TIMEOUT);
            if (!aborted && atomicCAS(c.status + CCB_STATUS_WHERE, 0u, (uint32_t)where | 0x80000000u) == 0u) {
              c.status[CCB_STATUS_EPOCH] = c.epoch;
              c.status[CCB_STATUS_SEEN] = ld_acquire_cta_shared(ctr);
            }
          }
          st_volatile_shared_int(&sh.fail, 1);
          if (!aborted) broadcast_abort(c, c.epoch);
          ok = 0;
          break;
        }
      }
      __nanosleep(64);
    }
  }
  return __shfl_sync(0xffffffffu, ok, 0) != 0;
}

// The polling warp of a role group: lanes < n wait for flag (row, source = lane, this CTA).
__device__ __forceinline__ bool warp_wait_sources(const CommDev& c, char* my_arena, int row, int self, PipeShared& sh,
                                                  int where) {
  const int lane = threadIdx.x & 31;
  int ok = 1;
  if (lane < c.nranks && lane != self) {
    const uint32_t* flag = flag_ptr(my_arena, row, lane, blockIdx.x);
    uint64_t t0 = 0;
    uint32_t polls = 0;
    for (;;) {
      const uint32_t v = ld_acquire_sys(flag);
      if ((int32_t)(v - c.epoch) >= 0) break;
      if ((++polls & 0x3f) == 0) {
        if (t0 == 0) t0 = globaltimer_ns();
        const bool aborted = ld_relaxed_sys(ctrl_ptr(my_arena, CCB_CTRL_ABORT)) == c.epoch || ld_volatile_shared_int(&sh.fail);
        const bool late = (globaltimer_ns() - t0) > c.timeout_ns || polls > (1u << 30);
        if (aborted || late) {
          if (c.status) {
            atomicOr(c.status + CCB_STATUS_FLAGS, aborted ? CCB_ST_ABORTED : CCB_ST_TIMEOUT);
            if (!aborted && atomicCAS(c.status + CCB_STATUS_WHERE, 0u, (uint32_t)(where | (lane << 8)) | 0x80000000u) == 0u) {
              c.status[CCB_STATUS_EPOCH] = c.epoch;
              c.status[CCB_STATUS_SEEN] = v;
            }
          }
          ok = 0;
          break;
        }
      }
      __nanosleep(100);
    }
  }
  const bool all = __all_sync(0xffffffffu, ok);
  if (!all && lane == 0) {
    st_volatile_shared_int(&sh.fail, 1);
    broadcast_abort(c, c.epoch);
  }
  return all;
}

// Group-wide wait for "the flags of `row` have arrived" (wave number `w`): the group's
// first warp polls global memory and publishes w + 1 in `ready`; the others wait there.
__device__ __forceinline__ bool group_wait(bool leader, unsigned int* ready, int w, int row, const CommDev& c,
                                           char* my_arena, int self, PipeShared& sh, int where) {
  if (leader) {
    const bool ok = warp_wait_sources(c, my_arena, row, self, sh, where);
    if (ok && (threadIdx.x & 31) == 0) st_release_cta_shared(ready, (unsigned int)(w + 1));
    return ok;
  }
  return warp_wait_counter(ready, (unsigned int)(w + 1), sh, c, my_arena, where | 0x8000);
}

// A finished phase handed to the signal warp: every lane's stores are ordered before
// lane 0's release by the warp barrier.
__device__ __forceinline__ void warp_arrive(unsigned int* ctr) {
  __syncwarp();
  if ((threadIdx.x & 31) == 0) red_release_cta_shared_add(ctr, 1u);
}

// 1024 threads: 32 warps per SM at 64 registers. The phases are bound by instruction issue
// as much as by memory (about 25 instructions per element over the three phases), so the
// kernel needs the occupancy; the loops below therefore keep one item per warp in flight
// and leave latency hiding to the 32 resident warps.
constexpr int kPipeThreads = 1024;
constexpr int kPipeWarps = kPipeThreads / 32;

template <class T, class C>
__global__ void __launch_bounds__(kPipeThreads, 1) pipe_kernel(const __grid_constant__ ReduceArgs a) {
  __shared__ PipeShared sh;
  const CommDev& c = a.c;
  const int lr = blockIdx.y, r = a.rank0 + lr, n = c.nranks;
  const size_t b = blockIdx.x, G = gridDim.x;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int L = a.link_warps, D = kPipeWarps - 1 - L;  // the last warp signals
  const int W = a.waves;
  // Two calls of this rank may be on the device at once when calls overlap (a late CTA of call
  // k beside an early CTA of call k + 1 with the same index): they use different flag rows, or
  // the late one could put an older epoch over a newer one in a peer's flag word.
  const int rb = a.row_base;
  const bool ar = (a.mode == CCB_MODE_ALLREDUCE);
  const T* send = static_cast<const T*>(a.send[lr]);
  T* recv = static_cast<T*>(a.recv[lr]);
  float* ef = a.ef[lr];
  char* my = c.arena[r];
  const size_t half = CCB_DATA_OFFSET + (size_t)(c.epoch & 1u) * c.half_bytes;
  const size_t area1 = half, area2 = half + (size_t)n * a.slot_bytes;
  const size_t pad = a.shard_pad;
  const bool use_mc = a.use_mc && c.mc_arena != nullptr;
  const uint32_t peers = ((1u << n) - 1u) & ~(1u << r);
  auto shard_valid = [&](int s) -> size_t {
    const size_t beg = (size_t)s * a.shard_elems;
    if (beg >= a.count) return 0;
    const size_t left = a.count - beg;
    return left < a.shard_elems ? left : a.shard_elems;
  };
  if (threadIdx.x == 0) {
    for (int w = 0; w < CCB_MAX_SLOTS / 2; ++w) sh.p1_done[w] = sh.p2_done[w] = 0u;
    sh.p1_ready = sh.p2_ready = 0u;
    sh.fail = 0;
  }
  // Items are 512-element units; the CTA owns chunks b, b + G, b + 2G, ... of 8 units of every
  // shard, and wave w takes the slice [kb[s][w], kb[s][w + 1]) of them. 32-bit arithmetic: a
  // shard has fewer than 2^32 units.
  if (threadIdx.x >= 32 && threadIdx.x < 32 + (unsigned)n) {
    const int s = threadIdx.x - 32;
    const unsigned int units = (unsigned int)((shard_valid(s) + kWarpElems - 1) / kWarpElems);
    const unsigned int nch = (units + kPipeChunkUnits - 1) >> kPipeChunkShift;
    const unsigned int K = nch > (unsigned int)b ? (nch - (unsigned int)b + (unsigned int)G - 1u) / (unsigned int)G : 0u;
    for (int w = 0; w <= W; ++w) sh.kb[s][w] = (unsigned int)((unsigned long long)K * (unsigned)w / (unsigned)W);
  }
  __syncthreads();  // the only CTA-wide barrier: the roles part ways here
  // The next call of the stream may start on the SMs that this grid's CTAs leave (when it was
  // launched with the programmatic-serialisation attribute; a no-op otherwise). Nothing here
  // waits for the grid before this one: see the launch in the runtime.
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

  auto wave_items = [&](int s, int w, unsigned int& kb) -> unsigned int {
    kb = sh.kb[s][w];
    return (sh.kb[s][w + 1] - kb) << kPipeChunkShift;
  };
  auto item_elem = [&](unsigned int kb, unsigned int i) -> size_t {
    const unsigned int ch = (unsigned int)b + (kb + (i >> kPipeChunkShift)) * (unsigned int)G;
    return (size_t)((ch << kPipeChunkShift) + (i & (kPipeChunkUnits - 1))) * kWarpElems;
  };

  const bool sum = (a.op == CCB_OP_SUM);
  auto accumulate = [&](float (&acc)[16], const float (&d)[16]) {
    if (sum) {
#pragma unroll
      for (int k = 0; k < 16; ++k) acc[k] += d[k];
    } else {
#pragma unroll
      for (int k = 0; k < 16; ++k) acc[k] = apply_op(a.op, acc[k], d[k]);
    }
  };

  // ---- phase 1 of wave w: this rank's lanes of every peer's shard, to the owner ----
  auto phase1 = [&](int w, int gw, int gn) {
    for (int j = 1; j < n; ++j) {
      const int p = r + j < n ? r + j : r + j - n;
      const size_t valid = shard_valid(p);
      const T* src = send + (size_t)p * a.shard_elems;
      float* efs = ef ? ef + (size_t)p * a.shard_elems : nullptr;
      char* dst = c.arena[p] + area1 + (size_t)r * a.slot_bytes;
      unsigned int kb;
      const unsigned int items = wave_items(p, w, kb);
      // The raw elements of the next item are requested before the current one is encoded,
      // so a warp has two loads in flight instead of a load and then an idle wait.
      Raw16<T> raw;
      unsigned int i = gw;
      size_t e0 = i < items ? item_elem(kb, i) : valid;
      if (e0 < valid) load16_raw<T>(src, e0 + lane * kLaneElems, valid, raw);
      while (e0 < valid) {
        const size_t idx = e0 + lane * kLaneElems;
        float v[16];
        raw16_to_f<T>(raw, v);
        i += gn;
        e0 = i < items ? item_elem(kb, i) : valid;
        if (e0 < valid) load16_raw<T>(src, e0 + lane * kLaneElems, valid, raw);
        if (efs) {
          float e[16];
          load16f_plain(efs, idx, valid, e);
#pragma unroll
          for (int q = 0; q < 16; ++q) v[q] += e[q];
        }
        typename C::Packet pk;
        C::encode(v, pk);
        C::store(dst, pad, idx, pk);
        if (efs) {
          float d[16];
          C::decode(pk, d);
#pragma unroll
          for (int q = 0; q < 16; ++q) d[q] = v[q] - d[q];
          store16f_plain(efs, idx, valid, d);
        }
      }
    }
  };

  // ---- phase 2 of wave w: reduce the own shard; AllReduce requantises and sends it ----
  auto phase2 = [&](int w, int gw, int gn) {
    const size_t valid = shard_valid(r);
    const T* src = send + (size_t)r * a.shard_elems;
    float* efs = (ef && ar) ? ef + (size_t)r * a.shard_elems : nullptr;
    T* out = ar ? recv + (size_t)r * a.shard_elems : recv;
    unsigned int kb;
    const unsigned int items = wave_items(r, w, kb);
    for (unsigned int i = gw; i < items; i += gn) {
      const size_t e0 = item_elem(kb, i);
      if (e0 >= valid) continue;
      const size_t idx = e0 + lane * kLaneElems;
      // The packet of the next source is requested before the current one is decoded.
      typename C::Packet nxt;
      int q = (r == 0) ? 1 : 0;
      C::load(my + area1 + (size_t)q * a.slot_bytes, pad, idx, nxt);
      float acc[16];
      load16<T>(src, idx, valid, acc);
      while (q < n) {  // increasing rank order, as in reduce_kernel
        const typename C::Packet pk = nxt;
        q += (q + 1 == r) ? 2 : 1;
        if (q < n) C::load(my + area1 + (size_t)q * a.slot_bytes, pad, idx, nxt);
        float d[16];
        C::decode(pk, d);
        accumulate(acc, d);
      }
      if (!ar) {  // ReduceScatter delivers the fp32 sum without a second quantisation
        store16<T>(out, idx, valid, acc);
        continue;
      }
      if (efs) {
        float e[16];
        load16f_plain(efs, idx, valid, e);
#pragma unroll
        for (int k = 0; k < 16; ++k) acc[k] += e[k];
      }
      typename C::Packet pk;
      C::encode(acc, pk);
      if (use_mc) {
        C::store_mc(c.mc_arena + area2 + (size_t)r * a.slot_bytes, pad, idx, pk);
      } else {
        for (int j = 1; j < n; ++j) C::store(c.arena[r + j < n ? r + j : r + j - n] + area2 + (size_t)r * a.slot_bytes, pad, idx, pk);
      }
      float d[16];
      C::decode(pk, d);
      if (efs) {
        float e[16];
#pragma unroll
        for (int k = 0; k < 16; ++k) e[k] = acc[k] - d[k];
        store16f_plain(efs, idx, valid, e);
      }
      store16<T>(out, idx, valid, d);
    }
  };

  // ---- phase 3 of wave w: decode the peers' reduced shards ----
  auto phase3 = [&](int w, int gw, int gn) {
    for (int j = 1; j < n; ++j) {
      const int q = r + j < n ? r + j : r + j - n;
      const size_t valid = shard_valid(q);
      const char* slot = my + area2 + (size_t)q * a.slot_bytes;
      T* out = recv + (size_t)q * a.shard_elems;
      unsigned int kb;
      const unsigned int items = wave_items(q, w, kb);
      typename C::Packet nxt;
      unsigned int i = gw;
      size_t e0 = i < items ? item_elem(kb, i) : valid;
      if (e0 < valid) C::load(slot, pad, e0 + lane * kLaneElems, nxt);
      while (e0 < valid) {
        const size_t idx = e0 + lane * kLaneElems;
        const typename C::Packet pk = nxt;
        i += gn;
        e0 = i < items ? item_elem(kb, i) : valid;
        if (e0 < valid) C::load(slot, pad, e0 + lane * kLaneElems, nxt);
        float d[16];
        C::decode(pk, d);
        store16<T>(out, idx, valid, d);
      }
    }
  };

  const bool tr = c.trace != nullptr && lane == 0;
  auto mark = [&](int k) {
    if (tr) c.trace[((size_t)blockIdx.y * gridDim.x + blockIdx.x) * CCB_TRACE_SLOTS + k] = globaltimer_ns();
  };

  // Ramp-up and ramp-down: before the first phase-2 flags can arrive the decode warps have
  // nothing to do, and after the last phase 2 the link warps have nothing left, so in an
  // AllReduce all 31 data warps share phase 1 of wave 0 and phase 3 of the last wave.
  const int kData = kPipeWarps - 1;
  if (warp < L) {
    // ------------------------------------------------------------ link warps ----
    const bool leader = (warp == 0);
    uint64_t waited = 0;  // trace slot 6: ns the link leader spent waiting for phase-1 flags
    if (leader) mark(0);
    if (ar) phase1(0, warp, kData); else phase1(0, warp, L);
    warp_arrive(&sh.p1_done[0]);
    if (leader) mark(1);
    if (ar) {
      for (int w = 0; w < W; ++w) {
        if (w + 1 < W) {
          phase1(w + 1, warp, L);
          warp_arrive(&sh.p1_done[w + 1]);
        }
        const uint64_t tw0 = tr ? globaltimer_ns() : 0;
        if (!group_wait(leader, &sh.p1_ready, w, rb + 2 * w, c, my, r, sh, 0x10 | (w << 16))) return;
        if (tr) waited += globaltimer_ns() - tw0;
        phase2(w, warp, L);
        warp_arrive(&sh.p2_done[w]);
        if (leader && w == 0) mark(2);
      }
      if (leader) mark(3);
      if (leader && tr) c.trace[((size_t)blockIdx.y * gridDim.x + blockIdx.x) * CCB_TRACE_SLOTS + 6] = waited;
      // the last wave's decode, shared with the decode warps (whose leader polls the flags)
      if (!warp_wait_counter(&sh.p2_ready, (unsigned)W, sh, c, my, 0x20 | ((W - 1) << 16) | 0x8000)) return;
      phase3(W - 1, warp, kData);
    } else {
      for (int w = 1; w < W; ++w) {
        phase1(w, warp, L);
        warp_arrive(&sh.p1_done[w]);
      }
      if (leader) mark(3);
    }
  } else if (warp < L + D) {
    // ---------------------------------------------------------- decode warps ----
    const int gw = warp - L;
    const bool leader = (gw == 0);
    if (ar) {
      phase1(0, warp, kData);
      warp_arrive(&sh.p1_done[0]);
    }
    for (int w = 0; w < W; ++w) {
      if (ar) {
        if (!group_wait(leader, &sh.p2_ready, w, rb + 2 * w + 1, c, my, r, sh, 0x20 | (w << 16))) return;
        if (w + 1 < W) phase3(w, gw, D); else phase3(w, warp, kData);
      } else {
        if (!group_wait(leader, &sh.p1_ready, w, rb + 2 * w, c, my, r, sh, 0x10 | (w << 16))) return;
        phase2(w, gw, D);
      }
      if (leader && w == 0) mark(5);
    }
    if (leader) mark(4);
  } else {
    // ----------------------------------------------------------- signal warp ----
    // Events in the order the link warps produce them: P1(0), then per wave P1(w+1), P2(w).
    // Phase 1 of wave 0 has kData arrivals in an AllReduce (everybody helps), L otherwise.
    const unsigned first = ar ? (unsigned)kData : (unsigned)L;
    uint64_t fenced = 0;  // trace slot 7: ns spent in fences and flag stores
    auto publish = [&](int row) {
      const uint64_t t0 = tr ? globaltimer_ns() : 0;
      if (lane == 0) signal_peers(c, peers, row, r, (int)b);
      __syncwarp();
      if (tr) fenced += globaltimer_ns() - t0;
    };
    if (!warp_wait_counter(&sh.p1_done[0], first, sh, c, my, 0xA0)) return;
    publish(rb);
    for (int w = 0; w < W; ++w) {
      if (w + 1 < W) {
        if (!warp_wait_counter(&sh.p1_done[w + 1], (unsigned)L, sh, c, my, 0xA0 | ((w + 1) << 16))) return;
        publish(rb + 2 * (w + 1));
      }
      if (ar) {
        if (!warp_wait_counter(&sh.p2_done[w], (unsigned)L, sh, c, my, 0xB0 | (w << 16))) return;
        publish(rb + 2 * w + 1);
      }
    }
    if (tr) c.trace[((size_t)blockIdx.y * gridDim.x + blockIdx.x) * CCB_TRACE_SLOTS + 7] = fenced;
  }
}

}  // namespace ccb

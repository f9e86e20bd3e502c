// Fused codec + reduction collectives over peer memory: two-shot AllReduce,
// one-shot AllReduce, ReduceScatter and Reduce in ONE kernel per call.
//
// The reference performs the same job as 2(n-1) host-driven hops, each one a
// quantize kernel, ncclSend, ncclRecv, dequantize kernel, cudaStreamSynchronize and
// reduce kernel (userconfig/wrapper_code_examples/communication/plain_nccl_compress/
// plain_nccl_compress.cu:654-774 AllReduce, :970-1076 ReduceScatter, :839-912 Reduce).
// On an NVSwitch box every peer is one hop away at full bandwidth, so the native
// shape is: quantise in registers, store the compressed lane straight into the
// owner's arena, flag; the owner dequantises and reduces in fp32, requantises ONCE,
// stores the result into every peer's arena, flag; everybody dequantises into recv.
// Two quantisation hops instead of n-1, no host involvement, no separate codec pass.
#pragma once
#include "ccb_codec.cuh"

namespace ccb {

struct CtaSync {
  int fail;
};

// Threads [0, n) each wait for one source's flag; the whole CTA learns the verdict.
// Returns false (uniformly) when any wait gave up; the caller must then return.
__device__ __forceinline__ bool cta_wait_sources(CtaSync& s, const CommDev& c, char* my_arena, int slot,
                                                 int self, uint32_t srcmask, int where) {
  const int t = threadIdx.x;
  if (t < c.nranks && t != self && ((srcmask >> t) & 1u)) {
    if (!wait_flag(flag_ptr(my_arena, slot, t, blockIdx.x), c.epoch, c, my_arena, where | (t << 8))) s.fail = 1;
  }
  __syncthreads();
  if (s.fail) {
    if (t == 0) broadcast_abort(c, c.epoch);
    return false;
  }
  return true;
}

// End-of-call handshake for rooted patterns, where some ranks wait on nobody and
// could otherwise run two calls ahead and overwrite staging that is still being
// read. The last CTA of each rank to finish tells every peer, then waits for all.
__device__ __forceinline__ void end_handshake(CtaSync& s, const CommDev& c, int r) {
  __shared__ int last;
  char* my = c.arena[r];
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    uint32_t done = atomicAdd(ctrl_ptr(my, CCB_CTRL_BARRIER + CCB_MAX_RANKS), 1u);
    last = (done == gridDim.x - 1);
    if (last) *ctrl_ptr(my, CCB_CTRL_BARRIER + CCB_MAX_RANKS) = 0u;
  }
  __syncthreads();
  if (!last) return;
  const int t = threadIdx.x;
  if (t < c.nranks && t != r) signal_flag(ctrl_ptr(c.arena[t], CCB_CTRL_BARRIER + r), c.epoch);
  if (t < c.nranks && t != r) {
    if (!wait_flag(ctrl_ptr(my, CCB_CTRL_BARRIER + t), c.epoch, c, my, 0xE0 | (t << 8))) s.fail = 1;
  }
  __syncthreads();
}

enum { kTwoShot = 0, kOneShot = 1 };

// SHAPE == kOneShot: every rank stores its whole (compressed) message into every
// arena and reduces all n copies itself: one exchange, n times the bytes; for
// latency-bound sizes.
// SHAPE == kTwoShot: shard s is owned by rank s (or the whole message by `root` for
// Reduce). The CTA's tiles of a shard are cut into `waves` consecutive groups and
// the three phases are software-pipelined over them,
//     P1(w+1): compress and store to the owners      (HBM read, NVLink write)
//     P2(w)  : owner reduces, requantises, stores    (HBM read, NVLink write)
//     P3(w-1): everybody decodes the reduced shards  (HBM read and write only)
// so that, across the CTAs of a GPU, link-bound and memory-bound work overlap
// instead of alternating. Flag row 2w carries phase 1 of wave w, row 2w+1 phase 2.
template <class T, class C, int SHAPE>
__global__ void __launch_bounds__(kThreads, 2) reduce_kernel(const __grid_constant__ ReduceArgs a) {
  __shared__ CtaSync sync;
  const CommDev& c = a.c;
  const int lr = blockIdx.y, r = a.rank0 + lr, n = c.nranks;
  const int b = blockIdx.x, G = gridDim.x;
  const int lane_off = (threadIdx.x >> 5) * kWarpElems + (threadIdx.x & 31) * kLaneElems;
  const int warp_off = (threadIdx.x >> 5) * kWarpElems;
  // A tile is tile_warps x 512 elements: mid-size messages use narrow tiles so that they
  // still spread over all CTAs; warps beyond tile_warps only take part in the barriers.
  const size_t tile_elems = (size_t)a.tile_warps * kWarpElems;
  const bool active_warp = (int)(threadIdx.x >> 5) < a.tile_warps;
  const T* send = static_cast<const T*>(a.send[lr]);
  T* recv = static_cast<T*>(a.recv[lr]);
  float* ef = a.ef[lr];
  char* my = c.arena[r];
  const size_t half = CCB_DATA_OFFSET + (size_t)(c.epoch & 1u) * c.half_bytes;
  const size_t area1 = half, area2 = half + (size_t)n * a.slot_bytes;
  const size_t pad = a.shard_pad;
  const bool rooted = (a.mode == CCB_MODE_REDUCE);
  if (threadIdx.x == 0) sync.fail = 0;
  __syncthreads();

  auto shard_valid = [&](int s) -> size_t {
    const size_t beg = (size_t)s * a.shard_elems;
    if (beg >= a.count) return 0;
    const size_t left = a.count - beg;
    return left < a.shard_elems ? left : a.shard_elems;
  };

  if constexpr (SHAPE == kOneShot) {
    const size_t valid = shard_valid(0);
    for (size_t t = b; t * tile_elems < valid; t += G) {
      if (!active_warp || t * tile_elems + warp_off >= valid) continue;
      const size_t idx = t * tile_elems + lane_off;
      float v[16];
      load16<T>(send, idx, valid, v);
      if (ef) {
        float e[16];
        load16f_plain(ef, idx, a.count, e);
#pragma unroll
        for (int i = 0; i < 16; ++i) v[i] += e[i];
      }
      typename C::Packet pk;
      C::encode(v, pk);
      for (int j = 0; j < n; ++j) {
        const int p = r + j < n ? r + j : r + j - n;
        C::store(c.arena[p] + area1 + (size_t)r * a.slot_bytes, pad, idx, pk);
      }
      if (ef) {
        float d[16];
        C::decode(pk, d);
#pragma unroll
        for (int i = 0; i < 16; ++i) d[i] = v[i] - d[i];
        store16f_plain(ef, idx, a.count, d);
      }
    }
    __syncthreads();
    if (threadIdx.x < n && threadIdx.x != r) signal_flag(flag_ptr(c.arena[threadIdx.x], 0, r, b), c.epoch);
    if (!cta_wait_sources(sync, c, my, 0, r, 0xffu, 0x10)) return;
    for (size_t t = b; t * tile_elems < valid; t += G) {
      if (!active_warp || t * tile_elems + warp_off >= valid) continue;
      const size_t idx = t * tile_elems + lane_off;
      // Every rank sums the same n decoded contributions in the same order, its own
      // included, so all ranks end with bit-identical results.
      float acc[16];
      for (int q = 0; q < n; ++q) {
        typename C::Packet pk;
        C::load(my + area1 + (size_t)q * a.slot_bytes, pad, idx, pk);
        float d[16];
        C::decode(pk, d);
        if (q == 0) {
#pragma unroll
          for (int i = 0; i < 16; ++i) acc[i] = d[i];
        } else {
#pragma unroll
          for (int i = 0; i < 16; ++i) acc[i] = apply_op(a.op, acc[i], d[i]);
        }
      }
      store16<T>(recv, idx, valid, acc);
    }
    return;
  } else {
    const int W = a.waves < 1 ? 1 : a.waves;
    // k-range of this CTA's tiles (t = b + k*G) of a shard that belong to wave w
    // 32-bit arithmetic (a shard has fewer than 2^32 tiles): a 64-bit division costs about a
    // hundred instructions, and this runs per phase, peer and wave
    auto wave_range = [&](size_t valid, int w, size_t& kb, size_t& ke) {
      const unsigned int units = (unsigned int)((valid + kWarpElems - 1) / kWarpElems);  // constant divisor: a shift
      const unsigned int nt = (units + (unsigned int)a.tile_warps - 1u) / (unsigned int)a.tile_warps;
      const unsigned int K = nt > (unsigned int)b ? (nt - (unsigned int)b + (unsigned int)G - 1u) / (unsigned int)G : 0u;
      if (W == 1) {
        kb = 0;
        ke = K;
      } else {
        kb = K * (unsigned int)w / (unsigned int)W;
        ke = K * (unsigned int)(w + 1) / (unsigned int)W;
      }
    };

    auto phase1 = [&](int w) {
      for (int j = 1; j < n; ++j) {
        const int p = r + j < n ? r + j : r + j - n;
        if (rooted && p != a.root) continue;
        const int s = rooted ? 0 : p;
        const size_t valid = shard_valid(s);
        const T* src = send + (size_t)s * a.shard_elems;
        float* efs = ef ? ef + (size_t)s * a.shard_elems : nullptr;
        char* dst = c.arena[p] + area1 + (size_t)r * a.slot_bytes;
        size_t kb, ke;
        wave_range(valid, w, kb, ke);
        for (size_t k = kb; k < ke; ++k) {
          const size_t t = b + k * G;
          if (!active_warp || t * tile_elems + warp_off >= valid) continue;
          const size_t idx = t * tile_elems + lane_off;
          float v[16];
          load16<T>(src, idx, valid, v);
          if (efs) {
            float e[16];
            load16f_plain(efs, idx, valid, e);
#pragma unroll
            for (int i = 0; i < 16; ++i) v[i] += e[i];
          }
          typename C::Packet pk;
          C::encode(v, pk);
          C::store(dst, pad, idx, pk);
          if (efs) {
            float d[16];
            C::decode(pk, d);
#pragma unroll
            for (int i = 0; i < 16; ++i) d[i] = v[i] - d[i];
            store16f_plain(efs, idx, valid, d);
          }
        }
      }
      // one barrier and ONE fence for all destinations: a fence per destination costs a
      // round trip each, seven in a row at eight ranks
      __syncthreads();
      if (threadIdx.x == 0) signal_peers(c, rooted ? ((r != a.root) ? (1u << a.root) : 0u) : (((1u << n) - 1u) & ~(1u << r)), 2 * w, r, b);
    };

    auto phase2 = [&](int w) -> bool {
      if (rooted && r != a.root) return true;
      if (!cta_wait_sources(sync, c, my, 2 * w, r, 0xffu, 0x10 | (w << 16))) return false;
      const int s = rooted ? 0 : r;
      const size_t valid = shard_valid(s);
      const T* src = send + (size_t)s * a.shard_elems;
      float* efs = (ef && a.mode == CCB_MODE_ALLREDUCE) ? ef + (size_t)s * a.shard_elems : nullptr;
      size_t kb, ke;
      wave_range(valid, w, kb, ke);
      for (size_t k = kb; k < ke; ++k) {
        const size_t t = b + k * G;
        if (!active_warp || t * tile_elems + warp_off >= valid) continue;
        const size_t idx = t * tile_elems + lane_off;
        float acc[16];
        load16<T>(src, idx, valid, acc);
        for (int q = 0; q < n; ++q) {
          if (q == r) continue;
          typename C::Packet pk;
          C::load(my + area1 + (size_t)q * a.slot_bytes, pad, idx, pk);
          float d[16];
          C::decode(pk, d);
#pragma unroll
          for (int i = 0; i < 16; ++i) acc[i] = apply_op(a.op, acc[i], d[i]);
        }
        if (a.mode == CCB_MODE_ALLREDUCE) {
          if (efs) {
            float e[16];
            load16f_plain(efs, idx, valid, e);
#pragma unroll
            for (int i = 0; i < 16; ++i) acc[i] += e[i];
          }
          typename C::Packet pk;
          C::encode(acc, pk);
          for (int j = 1; j < n; ++j) {
            const int p = r + j < n ? r + j : r + j - n;
            C::store(c.arena[p] + area2 + (size_t)r * a.slot_bytes, pad, idx, pk);
          }
          float d[16];
          C::decode(pk, d);
          if (efs) {
            float e[16];
#pragma unroll
            for (int i = 0; i < 16; ++i) e[i] = acc[i] - d[i];
            store16f_plain(efs, idx, valid, e);
          }
          store16<T>(recv + (size_t)s * a.shard_elems, idx, valid, d);
        } else {  // ReduceScatter and Reduce deliver the fp32 sum without a second quantisation
          store16<T>(recv, idx, valid, acc);
        }
      }
      if (a.mode == CCB_MODE_ALLREDUCE) {
        __syncthreads();
        if (threadIdx.x == 0) signal_peers(c, ((1u << n) - 1u) & ~(1u << r), 2 * w + 1, r, b);
      }
      return true;
    };

    auto phase3 = [&](int w) -> bool {
      if (!cta_wait_sources(sync, c, my, 2 * w + 1, r, 0xffu, 0x20 | (w << 16))) return false;
      for (int j = 1; j < n; ++j) {
        const int q = r + j < n ? r + j : r + j - n;
        const size_t valid = shard_valid(q);
        size_t kb, ke;
        wave_range(valid, w, kb, ke);
        for (size_t k = kb; k < ke; ++k) {
          const size_t t = b + k * G;
          if (!active_warp || t * tile_elems + warp_off >= valid) continue;
          const size_t idx = t * tile_elems + lane_off;
          typename C::Packet pk;
          C::load(my + area2 + (size_t)q * a.slot_bytes, pad, idx, pk);
          float d[16];
          C::decode(pk, d);
          store16<T>(recv + (size_t)q * a.shard_elems, idx, valid, d);
        }
      }
      return true;
    };

    const bool ar = (a.mode == CCB_MODE_ALLREDUCE);
    trace_mark(c, 0);
    phase1(0);
    trace_mark(c, 1);
    for (int w = 0; w < W; ++w) {
      if (w + 1 < W) phase1(w + 1);
      if (!phase2(w)) return;
      if (w == 0) trace_mark(c, 2);
      if (ar && w >= 1 && !phase3(w - 1)) return;
    }
    trace_mark(c, 3);
    if (ar && !phase3(W - 1)) return;
    trace_mark(c, 4);
    if (rooted) end_handshake(sync, c, r);
  }
}

}  // namespace ccb

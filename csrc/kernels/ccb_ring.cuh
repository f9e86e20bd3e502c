// Ring and binomial-tree AllReduce with per-hop requantisation, each as ONE kernel.
//
// These are the algorithms of the reference wrappers: ring reduce-scatter + ring
// all-gather that re-quantises at every hop (plain_nccl_compress.cu:682-773,
// plain_mpi_compress.c:163-273) and binomial trees for Reduce / Broadcast
// (plain_nccl_compress.cu:808-831, :869-909). There every hop is a host-driven
// sequence of kernels, NCCL p2p calls and a stream synchronisation. Here a hop is a
// flag wait inside the kernel: CTA b of rank r only depends on CTA b of its
// neighbour, so the hops of different CTAs overlap and the ring pipelines itself.
// The all-gather half forwards the compressed lanes verbatim (no decode/encode
// round trip), and every rank decodes the same bytes, so results are bit-identical
// on all ranks.
//
// Slot numbering (one slot = one compressed shard for the ring, the whole message
// for the tree): ring reduce-scatter step s -> slot s, all-gather step s -> slot
// n-1+s; tree reduce round k -> slot k, broadcast -> slot L (L = ceil(log2 n)).
// Flags use source column 0 because each slot has exactly one writer.
#pragma once
#include "ccb_reduce.cuh"

namespace ccb {

__device__ __forceinline__ bool cta_wait_slot(CtaSync& s, const CommDev& c, char* my, int slot, int where) {
  if (threadIdx.x == 0) {
    if (!wait_flag(flag_ptr(my, slot, 0, blockIdx.x), c.epoch, c, my, where | (slot << 8))) s.fail = 1;
  }
  __syncthreads();
  if (s.fail) {
    if (threadIdx.x == 0) broadcast_abort(c, c.epoch);
    return false;
  }
  return true;
}

template <class T, class C>
__global__ void __launch_bounds__(kThreads, 2) ring_kernel(const __grid_constant__ ReduceArgs a) {
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
  const int next = (r + 1) % n;
  char* nx = c.arena[next];
  const size_t half = CCB_DATA_OFFSET + (size_t)(c.epoch & 1u) * c.half_bytes;
  const size_t pad = a.shard_pad;
  if (threadIdx.x == 0) sync.fail = 0;
  __syncthreads();

  auto shard_valid = [&](int s) -> size_t {
    const size_t beg = (size_t)s * a.shard_elems;
    if (beg >= a.count) return 0;
    const size_t left = a.count - beg;
    return left < a.shard_elems ? left : a.shard_elems;
  };
  auto slot = [&](int k) -> size_t { return half + (size_t)k * a.slot_bytes; };

  // ---- reduce-scatter: n-1 hops, each one adds this rank's chunk and requantises
  // ---- (the last iteration, s == n-1, produces the fully reduced chunk r+1).
  for (int s = 0; s < n; ++s) {
    const int cs = ((r - s) % n + n) % n;
    const bool last = (s == n - 1);
    if (s > 0 && !cta_wait_slot(sync, c, my, s - 1, 0x40)) return;
    const size_t valid = shard_valid(cs);
    const T* src = send + (size_t)cs * a.shard_elems;
    float* efs = ef ? ef + (size_t)cs * a.shard_elems : nullptr;
    for (size_t t = b; t * tile_elems < valid; t += G) {
      if (!active_warp || t * tile_elems + warp_off >= valid) continue;
      const size_t idx = t * tile_elems + lane_off;
      float v[16];
      load16<T>(src, idx, valid, v);
      if (s > 0) {
        typename C::Packet in;
        C::load(my + slot(s - 1), pad, idx, in);
        float d[16];
        C::decode(in, d);
#pragma unroll
        for (int i = 0; i < 16; ++i) v[i] = apply_op(a.op, v[i], d[i]);
      }
      if (efs) {
        float e[16];
        load16f_plain(efs, idx, valid, e);
#pragma unroll
        for (int i = 0; i < 16; ++i) v[i] += e[i];
      }
      typename C::Packet pk;
      C::encode(v, pk);
      if (n > 1) C::store(nx + slot(last ? n - 1 : s), pad, idx, pk);
      if (efs || last) {
        float d[16];
        C::decode(pk, d);
        if (last) store16<T>(recv + (size_t)cs * a.shard_elems, idx, valid, d);
        if (efs) {
#pragma unroll
          for (int i = 0; i < 16; ++i) d[i] = v[i] - d[i];
          store16f_plain(efs, idx, valid, d);
        }
      }
    }
    if (n > 1) {
      __syncthreads();
      if (threadIdx.x == 0) signal_flag(flag_ptr(nx, last ? n - 1 : s, 0, b), c.epoch);
    }
    if (n == 1) break;
  }
  // With n ranks the loop above ran s = 0..n-1: the iteration s == n-1 wrote the
  // first all-gather slot (n-1). Remaining all-gather hops: receive slot n-1+k-1,
  // decode into recv, forward verbatim unless the next rank is the chunk's origin.
  for (int k = 1; k < n - 1 + 1 && n > 1; ++k) {
    if (k > n - 1) break;
    const int in_slot = n - 1 + (k - 1);
    if (!cta_wait_slot(sync, c, my, in_slot, 0x50)) return;
    const int cg = ((r + 1 - k) % n + n) % n;  // chunk that arrives at all-gather hop k
    const bool forward = (k < n - 1);
    const size_t valid = shard_valid(cg);
    for (size_t t = b; t * tile_elems < valid; t += G) {
      if (!active_warp || t * tile_elems + warp_off >= valid) continue;
      const size_t idx = t * tile_elems + lane_off;
      typename C::Packet pk;
      C::load(my + slot(in_slot), pad, idx, pk);
      if (forward) C::store(nx + slot(in_slot + 1), pad, idx, pk);
      float d[16];
      C::decode(pk, d);
      store16<T>(recv + (size_t)cg * a.shard_elems, idx, valid, d);
    }
    if (forward) {
      __syncthreads();
      if (threadIdx.x == 0) signal_flag(flag_ptr(nx, in_slot + 1, 0, b), c.epoch);
    }
  }
}

template <class T, class C>
__global__ void __launch_bounds__(kThreads, 2) tree_kernel(const __grid_constant__ ReduceArgs a) {
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
  const size_t pad = a.shard_pad;
  const size_t valid = a.count;
  if (threadIdx.x == 0) sync.fail = 0;
  __syncthreads();
  int L = 0;
  while ((1 << L) < n) ++L;
  // Rounds in which this rank receives: k below its lowest set bit (all for rank 0).
  const int tz = r == 0 ? L : (__ffs(r) - 1);
  auto slot = [&](int k) -> size_t { return half + (size_t)k * a.slot_bytes; };
  uint32_t kids = 0;
  for (int k = 0; k < tz; ++k)
    if (r + (1 << k) < n) kids |= 1u << k;

  // ---- up: wait for every child, add, requantise once, hand to the parent ------
  if (threadIdx.x < L && ((kids >> threadIdx.x) & 1u)) {
    if (!wait_flag(flag_ptr(my, threadIdx.x, 0, b), c.epoch, c, my, 0x60 | (threadIdx.x << 8))) sync.fail = 1;
  }
  __syncthreads();
  if (sync.fail) {
    if (threadIdx.x == 0) broadcast_abort(c, c.epoch);
    return;
  }
  char* parent = r == 0 ? nullptr : c.arena[r - (1 << tz)];
  for (size_t t = b; t * tile_elems < valid; t += G) {
    if (!active_warp || t * tile_elems + warp_off >= valid) continue;
    const size_t idx = t * tile_elems + lane_off;
    float v[16];
    load16<T>(send, idx, valid, v);
    for (int k = 0; k < tz; ++k) {
      if (!((kids >> k) & 1u)) continue;
      typename C::Packet in;
      C::load(my + slot(k), pad, idx, in);
      float d[16];
      C::decode(in, d);
#pragma unroll
      for (int i = 0; i < 16; ++i) v[i] = apply_op(a.op, v[i], d[i]);
    }
    if (ef) {
      float e[16];
      load16f_plain(ef, idx, valid, e);
#pragma unroll
      for (int i = 0; i < 16; ++i) v[i] += e[i];
    }
    typename C::Packet pk;
    C::encode(v, pk);
    if (parent) {
      C::store(parent + slot(tz), pad, idx, pk);
    } else {
      // Root: the encoded total goes down the same tree; the root's own result is
      // the decoded packet so that it matches what every other rank will decode.
      for (int k = 0; k < L; ++k)
        if ((kids >> k) & 1u) C::store(c.arena[r + (1 << k)] + slot(L), pad, idx, pk);
    }
    if (ef || !parent) {
      float d[16];
      C::decode(pk, d);
      if (!parent) store16<T>(recv, idx, valid, d);
      if (ef) {
#pragma unroll
        for (int i = 0; i < 16; ++i) d[i] = v[i] - d[i];
        store16f_plain(ef, idx, valid, d);
      }
    }
  }
  __syncthreads();
  if (parent) {
    if (threadIdx.x == 0) signal_flag(flag_ptr(parent, tz, 0, b), c.epoch);
  } else {
    if (threadIdx.x < L && ((kids >> threadIdx.x) & 1u))
      signal_flag(flag_ptr(c.arena[r + (1 << threadIdx.x)], L, 0, b), c.epoch);
    return;
  }

  // ---- down: take the encoded total from the parent, pass it on verbatim -------
  if (!cta_wait_slot(sync, c, my, L, 0x70)) return;
  for (size_t t = b; t * tile_elems < valid; t += G) {
    if (!active_warp || t * tile_elems + warp_off >= valid) continue;
    const size_t idx = t * tile_elems + lane_off;
    typename C::Packet pk;
    C::load(my + slot(L), pad, idx, pk);
    for (int k = 0; k < tz; ++k)
      if ((kids >> k) & 1u) C::store(c.arena[r + (1 << k)] + slot(L), pad, idx, pk);
    float d[16];
    C::decode(pk, d);
    store16<T>(recv, idx, valid, d);
  }
  __syncthreads();
  if (threadIdx.x < L && ((kids >> threadIdx.x) & 1u))
    signal_flag(flag_ptr(c.arena[r + (1 << threadIdx.x)], L, 0, b), c.epoch);
}

}  // namespace ccb

// Fused codec + data-movement collectives over peer memory: AllGather(v),
// Broadcast, Scatter(v), Gather and AlltoAll(v) are all one "exchange": rank r
// compresses cnt[r][p] elements for peer p in registers, stores them into p's
// arena, flags; p decompresses every slot it was sent into its receive buffer.
//
// The reference builds each of these from per-peer quantize kernel + ncclSend /
// ncclRecv + dequantize kernel sequences with a host sync per step
// (plain_nccl_compress.cu:779-834 Broadcast, :917-965 AllGather, :1081-1147
// AllToAll; run_codes/wrappers/src/nccl/nccl_extensions.c:28-250 Scatter, Gather,
// AllGatherv, Scatterv as uncompressed byte-typed send/recv loops).
#pragma once
#include "ccb_reduce.cuh"

namespace ccb {

template <class T, class C>
__global__ void __launch_bounds__(kThreads, 2) exchange_kernel(const __grid_constant__ ExchangeArgs a) {
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
  char* my = c.arena[r];
  const size_t area = CCB_DATA_OFFSET + (size_t)(c.epoch & 1u) * c.half_bytes;
  const size_t pad = a.slot_pad;
  if (threadIdx.x == 0) sync.fail = 0;
  __syncthreads();

  // Same block for every destination (AllGather, Broadcast): encode once, store n times.
  bool same = true;
  uint32_t dstmask = 0;
  for (int p = 0; p < n; ++p) {
    if (a.cnt[r][p] == 0) continue;
    dstmask |= 1u << p;
    const int f = __ffs(dstmask) - 1;
    if (a.cnt[r][p] != a.cnt[r][f] || a.send_off[r][p] != a.send_off[r][f]) same = false;
  }

  if (dstmask && same) {
    const int f = __ffs(dstmask) - 1;
    const size_t valid = a.cnt[r][f];
    const T* src = send + a.send_off[r][f];
    for (size_t t = b; t * tile_elems < valid; t += G) {
      if (!active_warp || t * tile_elems + warp_off >= valid) continue;
      const size_t idx = t * tile_elems + lane_off;
      float v[16];
      load16<T>(src, idx, valid, v);
      typename C::Packet pk;
      C::encode(v, pk);
      for (int j = 0; j < n; ++j) {
        const int p = (r + j) % n;
        if ((dstmask >> p) & 1u) C::store(c.arena[p] + area + (size_t)r * a.slot_bytes, pad, idx, pk);
      }
    }
  } else if (dstmask) {
    for (int j = 0; j < n; ++j) {
      const int p = (r + j) % n;
      const size_t valid = a.cnt[r][p];
      if (valid == 0) continue;
      const T* src = send + a.send_off[r][p];
      char* dst = c.arena[p] + area + (size_t)r * a.slot_bytes;
      for (size_t t = b; t * tile_elems < valid; t += G) {
        if (!active_warp || t * tile_elems + warp_off >= valid) continue;
        const size_t idx = t * tile_elems + lane_off;
        float v[16];
        load16<T>(src, idx, valid, v);
        typename C::Packet pk;
        C::encode(v, pk);
        C::store(dst, pad, idx, pk);
      }
    }
  }
  __syncthreads();
  if (threadIdx.x < n && threadIdx.x != r && ((dstmask >> threadIdx.x) & 1u))
    signal_flag(flag_ptr(c.arena[threadIdx.x], 0, r, b), c.epoch);

  uint32_t srcmask = 0;
  for (int q = 0; q < n; ++q)
    if (a.cnt[q][r]) srcmask |= 1u << q;
  if (!cta_wait_sources(sync, c, my, 0, r, srcmask, 0x30)) return;
  for (int j = 0; j < n; ++j) {
    const int q = (r + j) % n;
    const size_t valid = a.cnt[q][r];
    if (valid == 0) continue;
    T* dst = recv + a.recv_off[r][q];
    for (size_t t = b; t * tile_elems < valid; t += G) {
      if (!active_warp || t * tile_elems + warp_off >= valid) continue;
      const size_t idx = t * tile_elems + lane_off;
      typename C::Packet pk;
      C::load(my + area + (size_t)q * a.slot_bytes, pad, idx, pk);
      float d[16];
      C::decode(pk, d);
      store16<T>(dst, idx, valid, d);
    }
  }
  if (a.ack) end_handshake(sync, c, r);
}

}  // namespace ccb

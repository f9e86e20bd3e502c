// MoE dispatch and combine over peer memory with per-destination compression
// (fp8 e4m3 + ue8m0 block scales by default): see include/ccb/ccb_moe.h.
//
// Work unit = 512 consecutive elements of one row (a warp); a CTA tile = 16 units.
// Unit u of the block (src -> dst) is always handled by CTA ((u / 16) mod G) on both
// sides, so dispatch needs only per-CTA flags. The combine's receive side gathers
// rows by token, which may have been written by any CTA of the source, so it waits
// for ALL CTA flags of every source before reading.
#include <cuda_runtime.h>
#include <string.h>

#include "../rt/ccb_rt_internal.h"
#include "ccb/ccb_moe.h"
#include "ccb_reduce.cuh"

namespace ccb {

struct MoeArgs {
  CommDev c;
  const void* src[CCB_MAX_RANKS];        // x (dispatch) or y (combine), per local rank
  void* dst[CCB_MAX_RANKS];              // recv rows (dispatch) or out tokens (combine)
  const int32_t* perm[CCB_MAX_RANKS];    // dispatch: send order -> token row
  const int32_t* dest_rank[CCB_MAX_RANKS];
  const int32_t* pos[CCB_MAX_RANKS];
  const float* gate[CCB_MAX_RANKS];
  uint64_t cnt[CCB_MAX_RANKS][CCB_MAX_RANKS];   // rows [src][dst] (dispatch direction)
  uint64_t hidden, tokens;
  uint64_t slot_pad, slot_bytes;          // per (src,dst) slot, elements / bytes
  int topk, combine;
  int rank0, nlocal;
};

template <class T, class C>
__global__ void __launch_bounds__(kThreads, 2) moe_kernel(const __grid_constant__ MoeArgs a) {
  __shared__ CtaSync sync;
  const CommDev& c = a.c;
  const int lr = blockIdx.y, r = a.rank0 + lr, n = c.nranks;
  const int b = blockIdx.x, G = gridDim.x;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const T* src = static_cast<const T*>(a.src[lr]);
  T* dst = static_cast<T*>(a.dst[lr]);
  char* my = c.arena[r];
  const size_t area = CCB_DATA_OFFSET + (size_t)(c.epoch & 1u) * c.half_bytes;
  const size_t H = a.hidden;
  const unsigned int upr = (unsigned int)(H / kWarpElems);  // units per row (constant divisor above: a shift)
  // unit -> (row, column) without a 64-bit division per unit: a shift when a row is a power
  // of two of units (the usual hidden sizes), else a 32-bit division
  const int upr_shift = (upr & (upr - 1u)) == 0 ? __ffs((int)upr) - 1 : -1;
  auto row_of = [&](size_t u, size_t& col) -> size_t {
    const unsigned int u32 = (unsigned int)u;
    const unsigned int j = upr_shift >= 0 ? (u32 >> upr_shift) : (u32 / upr);
    col = (size_t)(u32 - j * upr) * kWarpElems + (size_t)lane * kLaneElems;
    return j;
  };
  const size_t pad = a.slot_pad;
  if (threadIdx.x == 0) sync.fail = 0;
  __syncthreads();

  // ---- send: block (r -> p). Dispatch gathers rows through perm; combine sends the
  // ---- contiguous block of rows that came from origin p (transposed counts).
  // Destinations are visited starting with the next rank, (r + 1) % n, ..., r: at any moment
  // every rank stores to a different peer, so no inbound link takes all the traffic.
  for (int jd = 1; jd <= n; ++jd) {
    const int p = r + jd < n ? r + jd : r + jd - n;
    const size_t rows = a.combine ? a.cnt[p][r] : a.cnt[r][p];
    size_t base_row = 0, send_row_off = 0;  // combine: first row of origin p; dispatch: offset into perm
    for (int s = 0; s < p; ++s) {
      base_row += a.cnt[s][r];
      send_row_off += a.cnt[r][s];
    }
    char* slot = c.arena[p] + area + (size_t)r * a.slot_bytes;
    const size_t units = rows * upr;
    for (size_t t = b; t * kWarps < units; t += G) {
      const size_t u = t * kWarps + warp;
      if (u >= units) continue;
      size_t col;
      const size_t j = row_of(u, col);
      const size_t srow = a.combine ? base_row + j : (size_t)a.perm[lr][send_row_off + j];
      float v[16];
      load16<T>(src + srow * H, col, H, v);
      typename C::Packet pk;
      C::encode(v, pk);
      C::store(slot, pad, j * H + col, pk);
    }
  }
  __syncthreads();
  // the combine's receiver gathers rows written by any CTA, its own rank's included,
  // so there the flag goes to this rank's own arena as well
  if (threadIdx.x < n && (a.combine || threadIdx.x != r)) signal_flag(flag_ptr(c.arena[threadIdx.x], 0, r, b), c.epoch);

  if (!a.combine) {
    // ---- dispatch receive: rows of source q land at recv row (sum_{s<q} cnt[s][r]) + j
    // own rows first (nothing to wait for), then each source as its flag arrives, in the
    // order in which the sources reach this rank
    for (int jq = 0; jq < n; ++jq) {
      const int q = (r - jq + n) % n;
      if (q != r && !cta_wait_sources(sync, c, my, 0, r, 1u << q, 0xB0)) return;
      size_t row0 = 0;
      for (int s = 0; s < q; ++s) row0 += a.cnt[s][r];
      const size_t units = a.cnt[q][r] * upr;
      const char* slot = my + area + (size_t)q * a.slot_bytes;
      for (size_t t = b; t * kWarps < units; t += G) {
        const size_t u = t * kWarps + warp;
        if (u >= units) continue;
        size_t col;
        const size_t j = row_of(u, col);
        typename C::Packet pk;
        C::load(slot, pad, j * H + col, pk);
        float d[16];
        C::decode(pk, d);
        store16<T>(dst + (row0 + j) * H, col, H, d);
      }
    }
    return;
  }

  // ---- combine receive: wait for every CTA of every source, then gather per token
  for (int i = threadIdx.x; i < n * G; i += kThreads) {
    const int q = i / G, cb = i % G;
    if (!wait_flag(flag_ptr(my, 0, q, cb), c.epoch, c, my, 0xC0 | (q << 8))) sync.fail = 1;
  }
  __syncthreads();
  if (sync.fail) {
    if (threadIdx.x == 0) broadcast_abort(c, c.epoch);
    return;
  }
  const size_t units = a.tokens * upr;
  for (size_t t = b; t * kWarps < units; t += G) {
    const size_t u = t * kWarps + warp;
    if (u >= units) continue;
    size_t col;
    const size_t tok = row_of(u, col);
    float acc[16];
#pragma unroll
    for (int i = 0; i < 16; ++i) acc[i] = 0.f;
    for (int k = 0; k < a.topk; ++k) {
      const int q = a.dest_rank[lr][tok * a.topk + k];
      const size_t j = (size_t)a.pos[lr][tok * a.topk + k];
      const float g = a.gate[lr][tok * a.topk + k];
      typename C::Packet pk;
      C::load(my + area + (size_t)q * a.slot_bytes, pad, j * H + col, pk);
      float d[16];
      C::decode(pk, d);
#pragma unroll
      for (int i = 0; i < 16; ++i) acc[i] += g * d[i];
    }
    store16<T>(dst + tok * H, col, H, acc);
  }
}

static const void* moe_fn(int dtype, int codec) {
#define CCB_MOE_CODEC(T)                                                                              \
  switch (codec) {                                                                                    \
    case CCB_CODEC_NONE: return reinterpret_cast<const void*>(&moe_kernel<T, CodecNone<T>>);          \
    case CCB_CODEC_INT8: return reinterpret_cast<const void*>(&moe_kernel<T, CodecInt8<128>>);        \
    case CCB_CODEC_INT8_G256: return reinterpret_cast<const void*>(&moe_kernel<T, CodecInt8<256>>);   \
    case CCB_CODEC_FP8: return reinterpret_cast<const void*>(&moe_kernel<T, CodecFp8>);               \
    case CCB_CODEC_INT4: return reinterpret_cast<const void*>(&moe_kernel<T, CodecInt4>);             \
    default: return nullptr;                                                                          \
  }
  switch (dtype) {
    case CCB_F32: CCB_MOE_CODEC(float)
    case CCB_BF16: CCB_MOE_CODEC(__nv_bfloat16)
    case CCB_F16: CCB_MOE_CODEC(__half)
  }
#undef CCB_MOE_CODEC
  return nullptr;
}

static int moe_launch(ccb_comm* c, MoeArgs& a, int dtype, int codec, uint64_t max_rows, uint64_t work_rows, cudaStream_t stream) {
  const void* fn = moe_fn(dtype, codec);
  if (!fn) {
    set_error("unsupported dtype %d / codec %d", dtype, codec);
    return CCB_ERR_UNSUPPORTED;
  }
  if (a.hidden == 0 || a.hidden % kWarpElems) {
    set_error("hidden size must be a multiple of %d", kWarpElems);
    return CCB_ERR_ARG;
  }
  const int n = ccb_comm_nranks(c);
  a.slot_pad = (max_rows ? max_rows : 1) * a.hidden;
  a.slot_bytes = codec_slot_bytes(codec, dtype, a.slot_pad);
  a.c = comm_dev(c, 0);
  if ((uint64_t)n * a.slot_bytes > a.c.half_bytes) {
    set_error("arena too small: MoE blocks of %llu rows need %llu bytes of staging", (unsigned long long)max_rows,
              (unsigned long long)((uint64_t)n * a.slot_bytes * 2));
    return CCB_ERR_CAPACITY;
  }
  a.c = comm_dev(c, next_epoch(c));
  a.rank0 = ccb_comm_rank(c);
  a.nlocal = ccb_comm_nlocal(c);
  const size_t units = (size_t)work_rows * (a.hidden / kWarpElems);
  if (units >> 32 || ((uint64_t)max_rows * (a.hidden / kWarpElems)) >> 32) {  // the kernel indexes units with 32 bits
    set_error("MoE block too large: %llu rows of %llu elements", (unsigned long long)work_rows, (unsigned long long)a.hidden);
    return CCB_ERR_CAPACITY;
  }
  size_t tiles = (units + kWarps - 1) / kWarps;
  int cap = grid_cap(c, fn);
  if (tiles < 1) tiles = 1;
  return launch(c, fn, tiles < (size_t)cap ? (int)tiles : cap, &a, stream);
}

}  // namespace ccb

using namespace ccb;

extern "C" int ccb_moe_dispatch(ccb_comm* c, const void* const* x, void* const* recv, const int32_t* const* perm,
                                const uint64_t* counts, uint64_t hidden, int dtype, int codec, ccb_stream_t stream) {
  int rc = check_alive(c);
  if (rc) return rc;
  const int n = ccb_comm_nranks(c), nl = ccb_comm_nlocal(c);
  MoeArgs a;
  memset(&a, 0, sizeof(a));
  uint64_t mx = 0;
  for (int s = 0; s < n; ++s)
    for (int d = 0; d < n; ++d) {
      a.cnt[s][d] = counts[s * n + d];
      if (a.cnt[s][d] > mx) mx = a.cnt[s][d];
    }
  for (int i = 0; i < nl; ++i) {
    a.src[i] = x[i];
    a.dst[i] = recv[i];
    a.perm[i] = perm[i];
  }
  a.hidden = hidden;
  a.combine = 0;
  return moe_launch(c, a, dtype, codec, mx, mx, static_cast<cudaStream_t>(stream));
}

extern "C" int ccb_moe_combine(ccb_comm* c, const void* const* y, void* const* out, const int32_t* const* dest_rank,
                               const int32_t* const* pos, const float* const* gate, const uint64_t* counts, uint64_t tokens,
                               int topk, uint64_t hidden, int dtype, int codec, ccb_stream_t stream) {
  int rc = check_alive(c);
  if (rc) return rc;
  const int n = ccb_comm_nranks(c), nl = ccb_comm_nlocal(c);
  MoeArgs a;
  memset(&a, 0, sizeof(a));
  uint64_t mx = 0;
  for (int s = 0; s < n; ++s)
    for (int d = 0; d < n; ++d) {
      a.cnt[s][d] = counts[s * n + d];
      if (a.cnt[s][d] > mx) mx = a.cnt[s][d];
    }
  for (int i = 0; i < nl; ++i) {
    a.src[i] = y[i];
    a.dst[i] = out[i];
    a.dest_rank[i] = dest_rank[i];
    a.pos[i] = pos[i];
    a.gate[i] = gate[i];
  }
  a.hidden = hidden;
  a.tokens = tokens;
  a.topk = topk;
  a.combine = 1;
  return moe_launch(c, a, dtype, codec, mx, tokens > mx ? tokens : mx, static_cast<cudaStream_t>(stream));
}

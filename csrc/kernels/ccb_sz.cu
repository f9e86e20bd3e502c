// SZ-style error-bounded lossy codec for 3-D fp32 fields, and its fusion with
// AllGather / Broadcast over peer memory.
//
// Codec (format "ccb-sz v2"):
//   1. pre-quantisation   q = rint(x / step), step = 2 eb (1 - 2^-10), corrected by +-1
//                         where fp32 rounding picked the farther grid point; the bound
//                         |x - q * step| <= eb is then checked on the very product the
//                         decoder computes, and a tile that fails it is stored raw;
//   2. 3-D Lorenzo        d = q - (prediction from the 7 already-coded neighbours),
//                         computed on the integers, inside a 32 x 8 x 8 tile (values
//                         outside the tile predict as 0), hence lossless and parallel:
//                         the decoder undoes it with prefix sums along x, y and z;
//   3. bit-packing        zig-zag to unsigned, then per packing row of 32 values the
//                         minimum width w (0..32) and w bit-planes of 32 bits. A row is
//                         element e of the eight consecutive x that each of the 32 threads
//                         of a z plane owns (thread = 4 y + x / 8): row index 8 z + e, bit
//                         t of a plane belongs to thread t. Planes come out of a 32 x 32
//                         bit-matrix transpose across the warp (five shuffle steps), one
//                         transpose for FOUR rows when their widths are at most 8 bits.
// A tile is  [64 row widths (1 B each)][bit-planes of row 0][row 1]...  padded to
// 16 B; a tile whose values do not fit the integer range (or are not finite) is
// stored raw (width byte 0 = 255, then 8 KiB of fp32). Eight consecutive tiles form a
// group that owns a fixed-capacity slot of kGroupStride bytes:
//   [8 x u32 tile sizes][tile 0][tile 1]...
// so a receiver finds every tile without any size exchange, while only the used
// bytes are ever written (and cross NVLink).
//
// Kernel shape: one thread-block cluster of 8 CTAs per group. Each CTA fetches its
// tile with ONE 3-D TMA copy (cp.async.bulk.tensor, no multicast) tracked by an
// mbarrier, packs it in shared memory, the cluster exchanges the 8 sizes through
// distributed shared memory to place the tiles back to back, and the packed tile is
// copied out with 16-byte stores, to local memory (ccb_sz_compress) or straight
// into every peer's arena (ccb_sz_all_gather), where the same CTAs decode what
// arrives. Fields whose x extent is not a multiple of 4 elements (TMA needs 16-byte
// row strides) take a plain-load path.
//
// The reference has no GPU error-bounded codec: it reaches SZ3 through dlopen on the
// CPU (userconfig/wrapper_code_examples/compression/sz3/mpi_sz3_wrapper.c:57-101,
// :138-218) and cuZFP as a library call (zfp_for_gpu_nvidia.cu:130, :179).
#include <cooperative_groups.h>
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdlib.h>
#include <string.h>

#include "../rt/ccb_rt_internal.h"
#include "ccb/ccb_sz.h"
#include "ccb_fastdiv.h"
#include "ccb_reduce.cuh"

namespace cg = cooperative_groups;

namespace ccb {

constexpr int kTX = 32, kTY = 8, kTZ = 8;
constexpr int kTileVals = kTX * kTY * kTZ;        // 2048
constexpr int kRows = kTY * kTZ;                  // 64
constexpr int kSzThreads = 256;                   // warp = z plane, lane = x
constexpr int kClusterSize = 8;
constexpr int kTileCap = kRows + kTileVals * 4;   // 8256 bytes, worst case (w = 32 everywhere)
constexpr int kGroupHeader = 32;
constexpr int kGroupStride = kGroupHeader + kClusterSize * kTileCap + 32;  // 66112, multiple of 16
static_assert(kGroupStride % 16 == 0, "slots must keep 16-byte alignment");
constexpr float kQMax = 4194304.f;                // 2^22: |q| beyond this stores the tile raw

struct SzField {
  const float* in;   // compress source (or 0)
  float* out;        // decompress destination (or 0)
};

struct SzArgs {
  CommDev c;
  CUtensorMap tmap[CCB_MAX_RANKS];   // one per local rank, over `in`
  SzField f[CCB_MAX_RANKS];          // per local rank
  unsigned long long* used_bytes;    // per local rank: compressed bytes produced (atomicAdd), or 0
  char* local_out;                   // compress-only: destination buffer (rank-less)
  const char* local_in;              // decompress-only: source buffer
  int nx, ny, nz;
  int tiles_x, tiles_y, tiles_z;
  unsigned int ngroups;
  float eb, two_eb, inv_two_eb;
  int use_tma;
  int mode;                          // 0 compress to local_out, 1 decompress from local_in, 2 all-gather, 3 broadcast
  int root;
  int rank0, nlocal;
  unsigned int bcast_waves;          // progress steps a broadcast root publishes (1..kMaxBcastWaves)
  unsigned long long slot_bytes;     // arena bytes of one source's slot (ngroups * kGroupStride, rounded)
  // Division of a tile index by tiles_x and by tiles_x * tiles_y as a multiplication:
  // (ccb_fastdiv.h; exact for tile < 2^22 and d < 2^18, which the host checks: 0 = use the
  // division). An integer division by a run-time value
  // costs about 25 instructions, and every thread needs three per tile.
  unsigned long long magic_x, magic_xy;
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, int count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
// Bounded wait on an mbarrier phase: false when the copy never completed.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity) {
  for (uint32_t spin = 0; spin < (1u << 26); ++spin) {
    uint32_t done;
    asm volatile(
        "{\n.reg .pred p;\n"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
        "selp.u32 %0, 1, 0, p;\n}\n"
        : "=r"(done) : "r"(smem_u32(bar)), "r"(parity) : "memory");
    if (done) return true;
  }
  return false;
}
__device__ __forceinline__ void tma_load_3d(void* smem_dst, const CUtensorMap* map, int x, int y, int z, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];"
      ::"r"(smem_u32(smem_dst)), "l"(map), "r"(x), "r"(y), "r"(z), "r"(smem_u32(bar)) : "memory");
}

struct TileCoord { int x0, y0, z0; };
__device__ __forceinline__ TileCoord tile_coord(const SzArgs& a, unsigned int tile) {
  TileCoord t;
  unsigned int tx, ty, tz;
  if (a.magic_x) {
    const unsigned int txy = a.tiles_x * a.tiles_y;
    tz = ccb_fastdiv(tile, a.magic_xy);
    const unsigned int rem = tile - tz * txy;
    ty = ccb_fastdiv(rem, a.magic_x);
    tx = rem - ty * a.tiles_x;
  } else {
    tx = tile % a.tiles_x, ty = (tile / a.tiles_x) % a.tiles_y, tz = tile / (a.tiles_x * a.tiles_y);
  }
  t.x0 = tx * kTX; t.y0 = ty * kTY; t.z0 = tz * kTZ;
  return t;
}

// Thread mapping of both directions: warp = z plane of the tile, lane = 4 y + xq, and the
// thread owns the eight consecutive values x = 8 xq .. 8 xq + 7 of line (y, z), which sit at
// words 8 * threadIdx.x .. +7 of the tile in shared memory (two 16-byte accesses). A packing
// row is element e of all 32 lanes of a warp: row index 8 z + e.

// Transposes the 32 x 32 bit matrix whose row i is the word held by lane i: afterwards
// lane j holds column j (bit i of the result = bit j of lane i's input). Five exchange steps.
__device__ __forceinline__ uint32_t transpose32(uint32_t x, int lane) {
#pragma unroll
  for (int s = 16; s >= 1; s >>= 1) {
    const uint32_t m = s == 16 ? 0x0000ffffu : s == 8 ? 0x00ff00ffu : s == 4 ? 0x0f0f0f0fu : s == 2 ? 0x33333333u : 0x55555555u;
    const uint32_t p = __shfl_xor_sync(0xffffffffu, x, s);
    const bool up = (lane & s) != 0;
    const uint32_t moved = up ? (p >> s) : (p << s);
    const uint32_t keep = up ? ~m : m;
    x = (x & keep) | (moved & ~keep);
  }
  return x;
}
__device__ __forceinline__ uint32_t bytesum(uint32_t v) { return __dp4a(v, 0x01010101u, 0u); }
// True when every byte of w (each at most 32) is at most 8 / at most 16.
__device__ __forceinline__ bool bytes_le8(uint32_t w) { return ((w + 0x77777777u) & 0x80808080u) == 0; }
__device__ __forceinline__ bool bytes_le16(uint32_t w) { return ((w + 0x6f6f6f6fu) & 0x80808080u) == 0; }

// Bit-planes of four rows: `W` holds their widths (one byte each), `off` is the word offset
// of the first row's planes. With all widths <= 8 the four rows share ONE bit-matrix
// transpose (lane 8 r + j ends up with plane j of row r); widths up to 16 take two, wider
// rows one transpose each. The byte layout does not depend on which way was taken.
template <bool kStore>
__device__ __forceinline__ void planes4(uint32_t (&u)[4], uint32_t W, uint32_t off, uint32_t* words, int lane) {
  auto pass = [&](int bits, int first_row, int rows) {   // rows * bits == 32
    const int rr = lane / bits, jj = lane % bits, row = first_row + rr;
    const uint32_t w = (W >> (8 * row)) & 0xffu;
    const uint32_t at = off + bytesum(W & ((1u << (8 * row)) - 1u)) + jj;
    if (kStore) {
      uint32_t U = 0;
      for (int r2 = 0; r2 < rows; ++r2) U |= u[first_row + r2] << (bits * r2);
      const uint32_t X = transpose32(U, lane);
      if ((uint32_t)jj < w) words[at] = X;
    } else {
      const uint32_t X = (uint32_t)jj < w ? ldg_cg_u32(words + at) : 0u;
      const uint32_t U = transpose32(X, lane);
      for (int r2 = 0; r2 < rows; ++r2) u[first_row + r2] = bits == 32 ? U : (U >> (bits * r2)) & ((1u << bits) - 1u);
    }
  };
  if (bytes_le8(W)) {
    pass(8, 0, 4);
  } else if (bytes_le16(W)) {
    pass(16, 0, 2);
    pass(16, 2, 2);
  } else {
#pragma unroll
    for (int r2 = 0; r2 < 4; ++r2) pass(32, r2, 1);
  }
}

constexpr float kRoundMagic = 12582912.f;   // 1.5 * 2^23: adding and subtracting it rounds to nearest even

// Packs the tile held in `vals` (fp32, [z][y][x]) into `pk`; returns its byte size.
// The codes overwrite the values in shared memory (each thread its own eight words).
// With `recon` set, the decoder's view of the tile (q * step, or the raw values of a raw
// tile) is also written to its place in that field: the sender's own copy of what every
// receiver will decode, without a decode pass.
__device__ __forceinline__ uint32_t pack_tile(float* vals, unsigned char* pk, int* s_tot, const SzArgs& a,
                                              float* recon = nullptr, TileCoord tc = TileCoord{0, 0, 0}) {
  const int lane = threadIdx.x & 31, z = threadIdx.x >> 5;
  int4* q4 = reinterpret_cast<int4*>(vals) + 2 * threadIdx.x;
  float x[8];
  {
    const float4 v0 = reinterpret_cast<const float4*>(q4)[0], v1 = reinterpret_cast<const float4*>(q4)[1];
    x[0] = v0.x; x[1] = v0.y; x[2] = v0.z; x[3] = v0.w; x[4] = v1.x; x[5] = v1.y; x[6] = v1.z; x[7] = v1.w;
  }
  int q[8];
  bool bad = false;
  const float half = 0.5f * a.two_eb;
#pragma unroll
  for (int e = 0; e < 8; ++e) {
    const float s = __fmul_rn(x[e], a.inv_two_eb);
    bad |= !(fabsf(s) < kQMax);  // also catches NaN / Inf
    float rf = __fadd_rn(__fadd_rn(s, kRoundMagic), -kRoundMagic);
    const float diff = __fsub_rn(x[e], __fmul_rn(rf, a.two_eb));  // against the decoder's own product (no FMA)
    // Nearly always |diff| <= step / 2 < eb: the value sits on the nearest grid point and the
    // bound holds, nothing to correct or to re-check. The correction runs only when some lane
    // of the warp needs it (NaN counts as needing it), with the same result either way.
    if (__any_sync(0xffffffffu, !(fabsf(diff) <= half))) {
      rf += diff > half ? 1.f : 0.f;                              // fp32 rounding picked the farther grid point
      rf -= -diff > half ? 1.f : 0.f;
      // The grid step is a shade under 2 eb, which absorbs the rounding of q * step for
      // |q| < 2^13. Beyond that a value can fall between two grid points that are both more
      // than eb away: such a tile is stored raw, so the bound always holds.
      bad |= fabsf(__fsub_rn(x[e], __fmul_rn(rf, a.two_eb))) > a.eb;
    }
    q[e] = (int)rf;
  }
  const bool raw_tile = __syncthreads_or(bad);
  if (recon) {
    const int gx = tc.x0 + 8 * (lane & 3), gy = tc.y0 + (lane >> 2), gz = tc.z0 + z;
    if (gy < a.ny && gz < a.nz) {
      float* row = recon + ((size_t)gz * a.ny + gy) * a.nx + gx;
      float o[8];
#pragma unroll
      for (int e = 0; e < 8; ++e) o[e] = raw_tile ? x[e] : __fmul_rn((float)q[e], a.two_eb);
      if (gx + 8 <= a.nx && (reinterpret_cast<uintptr_t>(row) & 15) == 0) {
        reinterpret_cast<float4*>(row)[0] = make_float4(o[0], o[1], o[2], o[3]);
        reinterpret_cast<float4*>(row)[1] = make_float4(o[4], o[5], o[6], o[7]);
      } else {
#pragma unroll
        for (int e = 0; e < 8; ++e)
          if (gx + e < a.nx) row[e] = o[e];
      }
    }
  }
  if (raw_tile) {  // raw tile: marker + the fp32 values
    for (int i = threadIdx.x; i < kRows; i += kSzThreads) pk[i] = (i == 0) ? 255 : 0;
    float* raw = reinterpret_cast<float*>(pk + kRows);
    for (int i = threadIdx.x; i < kTileVals; i += kSzThreads) raw[i] = vals[i];
    __syncthreads();
    return kRows + kTileVals * 4;
  }
  q4[0] = make_int4(q[0], q[1], q[2], q[3]);
  q4[1] = make_int4(q[4], q[5], q[6], q[7]);
  __syncthreads();
  // Lorenzo residual = the three first differences, in any order: z through shared memory
  // (plane z - 1 belongs to the warp below), y through the lane four below, x in registers.
  if (z > 0) {
    const int4 b0 = q4[-64], b1 = q4[-63];
    q[0] -= b0.x; q[1] -= b0.y; q[2] -= b0.z; q[3] -= b0.w; q[4] -= b1.x; q[5] -= b1.y; q[6] -= b1.z; q[7] -= b1.w;
  }
#pragma unroll
  for (int e = 0; e < 8; ++e) {
    const int up = __shfl_up_sync(0xffffffffu, q[e], 4);
    q[e] -= lane >= 4 ? up : 0;
  }
  int left = __shfl_up_sync(0xffffffffu, q[7], 1);
  if ((lane & 3) == 0) left = 0;
  uint32_t u[8], W[2] = {0u, 0u};
#pragma unroll
  for (int e = 7; e >= 0; --e) {
    const int d = q[e] - (e ? q[e - 1] : left);
    u[e] = ((uint32_t)d << 1) ^ (uint32_t)(d >> 31);
  }
#pragma unroll
  for (int e = 0; e < 8; ++e) {
    const uint32_t any = __reduce_or_sync(0xffffffffu, u[e]);
    W[e >> 2] |= (uint32_t)(32 - __clz(any)) << (8 * (e & 3));
  }
  const uint32_t tot_lo = bytesum(W[0]), tot = tot_lo + bytesum(W[1]);
  if (lane == 0) {
    reinterpret_cast<uint2*>(pk)[z] = make_uint2(W[0], W[1]);   // the eight width bytes of this plane
    s_tot[z] = (int)tot;
  }
  __syncthreads();
  uint32_t base = 0, total = 0;
#pragma unroll
  for (int zz = 0; zz < kTZ; ++zz) {
    const uint32_t t = (uint32_t)s_tot[zz];
    base += zz < z ? t : 0u;
    total += t;
  }
  uint32_t* words = reinterpret_cast<uint32_t*>(pk + kRows);
  uint32_t ua[4] = {u[0], u[1], u[2], u[3]}, ub[4] = {u[4], u[5], u[6], u[7]};
  planes4<true>(ua, W[0], base, words, lane);
  planes4<true>(ub, W[1], base + tot_lo, words, lane);
  const uint32_t bytes = kRows + 4u * total;
  const uint32_t padded = (bytes + 15u) & ~15u;
  for (uint32_t i = bytes + threadIdx.x; i < padded; i += kSzThreads) pk[i] = 0;
  __syncthreads();
  return padded;
}

// Decodes a packed tile at `src` (global or arena memory) and writes it to its place in `out`;
// `qs` is 8 KB of shared scratch.
__device__ __forceinline__ void unpack_tile(const unsigned char* src, int* qs, const SzArgs& a, float* out, const TileCoord& t) {
  const int lane = threadIdx.x & 31, z = threadIdx.x >> 5;
  // the 16 words of row widths, one per lane, and their running word count
  const uint32_t hw = lane < 16 ? ldg_cg_u32(src + 4 * lane) : 0u;
  if ((__shfl_sync(0xffffffffu, hw, 0) & 0xffu) == 255u) {
    const float* raw = reinterpret_cast<const float*>(src + kRows);
    for (int i = threadIdx.x; i < kTileVals; i += kSzThreads) {
      const int gx = t.x0 + (i % kTX), gy = t.y0 + (i / kTX) % kTY, gz = t.z0 + i / (kTX * kTY);
      if (gx < a.nx && gy < a.ny && gz < a.nz)
        out[((size_t)gz * a.ny + gy) * a.nx + gx] = __uint_as_float(ldg_cg_u32(raw + i));
    }
    return;
  }
  const uint32_t mine = bytesum(hw);
  uint32_t incl = mine;
#pragma unroll
  for (int d = 1; d < 16; d <<= 1) {
    const uint32_t v = __shfl_up_sync(0xffffffffu, incl, d);
    if (lane >= d) incl += v;
  }
  const uint32_t W0 = __shfl_sync(0xffffffffu, hw, 2 * z), W1 = __shfl_sync(0xffffffffu, hw, 2 * z + 1);
  const uint32_t base = __shfl_sync(0xffffffffu, incl - mine, 2 * z);
  uint32_t* words = reinterpret_cast<uint32_t*>(const_cast<unsigned char*>(src) + kRows);
  uint32_t ua[4], ub[4];
  planes4<false>(ua, W0, base, words, lane);
  planes4<false>(ub, W1, base + bytesum(W0), words, lane);
  int p[8];
#pragma unroll
  for (int e = 0; e < 8; ++e) {
    const uint32_t u = e < 4 ? ua[e & 3] : ub[e & 3];
    const int d = (int)(u >> 1) ^ -(int)(u & 1u);
    p[e] = e ? p[e - 1] + d : d;          // prefix along x inside the thread
  }
  {
    int sum = p[7];                         // then across the four threads of the line
    int v = __shfl_up_sync(0xffffffffu, sum, 1);
    if ((lane & 3) >= 1) sum += v;
    v = __shfl_up_sync(0xffffffffu, sum, 2);
    if ((lane & 3) >= 2) sum += v;
    const int before = sum - p[7];
#pragma unroll
    for (int e = 0; e < 8; ++e) p[e] += before;
  }
  int4* q4 = reinterpret_cast<int4*>(qs) + 2 * threadIdx.x;
  q4[0] = make_int4(p[0], p[1], p[2], p[3]);
  q4[1] = make_int4(p[4], p[5], p[6], p[7]);
  __syncthreads();
  // prefix along y: threads re-mapped to (x = lane, z = warp) walk the eight lines of their plane
  {
    int run = 0;
#pragma unroll
    for (int y = 0; y < kTY; ++y) {
      run += qs[(z * kTY + y) * kTX + lane];
      qs[(z * kTY + y) * kTX + lane] = run;
    }
  }
  __syncthreads();
  // prefix along z: threads re-mapped to (x = lane, y = warp) walk z with a running sum and
  // write each reconstructed row straight to the field (coalesced 128-byte row stores)
  {
    const int y = z;  // this warp now owns line y of every plane
    const int gx = t.x0 + lane, gy = t.y0 + y;
    const bool ok = gx < a.nx && gy < a.ny;
    int run = 0;
#pragma unroll
    for (int zz = 0; zz < kTZ; ++zz) {
      run += qs[(zz * kTY + y) * kTX + lane];
      const int gz = t.z0 + zz;
      if (ok && gz < a.nz) out[((size_t)gz * a.ny + gy) * a.nx + gx] = __fmul_rn((float)run, a.two_eb);
    }
  }
  __syncthreads();   // the scratch is free for the next tile
}

__device__ __forceinline__ void load_tile_plain(const float* in, float* vals, const TileCoord& t, const SzArgs& a) {
  const int lane = threadIdx.x & 31, z = threadIdx.x >> 5;
#pragma unroll
  for (int y = 0; y < kTY; ++y) {
    const int gx = t.x0 + lane, gy = t.y0 + y, gz = t.z0 + z;
    float v = 0.f;
    if (gx < a.nx && gy < a.ny && gz < a.nz) v = in[((size_t)gz * a.ny + gy) * a.nx + gx];
    vals[(z * kTY + y) * kTX + lane] = v;
  }
}
__device__ __forceinline__ void multimem_st(void* p, uint4 v) {
  asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}
__device__ __forceinline__ void multimem_st_u32(void* p, uint32_t v) {
  asm volatile("multimem.st.relaxed.sys.global.f32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ void cluster_arrive() { asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory"); }
__device__ __forceinline__ void cluster_wait() { asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory"); }
constexpr int kStage = kTileCap + 16;
constexpr unsigned int kMaxBcastWaves = 8;   // most progress steps of a broadcast (flag slots 0..7)   // one packed tile, 16-byte granular

// kKind: 0 compress into a local buffer, 1 decompress from one, 2 the collectives (mode 2
// all-gather, 3 broadcast). One body, three instantiations, so that each direction gets its
// own register allocation and occupancy.
template <int kKind>
__global__ void __launch_bounds__(kSzThreads, kKind == 1 ? 6 : kKind == 2 ? 5 : 4) sz_kernel(const __grid_constant__ SzArgs a) {
  const int mode = kKind == 2 ? a.mode : kKind;
  const unsigned int kBcastWaves = a.bcast_waves;
  // Two 8 KB buffers: compress lands the next tile in one while the other is packed;
  // decompress prefixes in vals2[0].
  __shared__ __align__(128) float vals2[2][kTileVals];
  __shared__ __align__(16) unsigned char pk2[2][kStage];
  __shared__ int s_tot[kTZ];
  __shared__ uint32_t s_size[2];         // this CTA's packed size per group parity, read by the cluster
  __shared__ __align__(8) uint64_t mbar[2];
  __shared__ CtaSync sync;

  cg::cluster_group cluster = cg::this_cluster();
  const int k = (int)cluster.block_rank();          // tile within the group
  const unsigned int cl = blockIdx.x / kClusterSize, ncl = gridDim.x / kClusterSize;
  const int lr = blockIdx.y, r = a.rank0 + lr, n = a.c.nranks;
  const int b = blockIdx.x;                         // flag column
  const unsigned int ntiles = (unsigned)a.tiles_x * a.tiles_y * a.tiles_z;
  const bool collective = mode >= 2;
  const bool i_send = mode == 0 || mode == 2 || (mode == 3 && r == a.root);
  const size_t area = CCB_DATA_OFFSET + (size_t)(a.c.epoch & 1u) * a.c.half_bytes;
  if (threadIdx.x == 0) {
    sync.fail = 0;
    mbar_init(&mbar[0], 1);
    mbar_init(&mbar[1], 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  uint32_t phases = 0u;     // bit s: parity the next wait on mbarrier s expects
  auto landed = [&](int slot) {   // bounded wait for the copy into buffer `slot`; reports a copy that never came
    const bool ok = mbar_wait(&mbar[slot], (phases >> slot) & 1u);
    phases ^= 1u << slot;
    if (!ok) {
      if (threadIdx.x == 0 && a.c.status) atomicOr(a.c.status + CCB_STATUS_FLAGS, CCB_ST_TIMEOUT);
      sync.fail = 1;
    }
  };

  if (collective) trace_mark(a.c, 0);
  // ------------------------------------------------------------- compress ----
  if (i_send && mode != 1) {
    const float* in = a.f[lr].in;
    unsigned long long produced = 0;
    // one thread starts the copy of this CTA's tile of group g into landing buffer `slot`
    auto prefetch = [&](unsigned int g, int slot) {
      const unsigned int tile = g * kClusterSize + k;
      if (!a.use_tma || g >= a.ngroups || tile >= ntiles || threadIdx.x != 0) return;
      const TileCoord t = tile_coord(a, tile);
      // earlier generic-proxy accesses to the buffer must be ordered before the TMA write
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      mbar_expect_tx(&mbar[slot], kTileVals * 4);
      tma_load_3d(vals2[slot], &a.tmap[lr], t.x0, t.y0, t.z0, &mbar[slot]);
    };
    // copies a packed tile out: to the local buffer, to every peer's arena one by one, or,
    // where the arenas are bound to an NVLink multicast object, ONCE to the multicast
    // address: the switch replicates it, the sender's link carries the bytes one time.
    // The sender keeps no packed copy of its own field (pack_tile wrote the reconstruction).
    const bool use_mc = kKind == 2 && a.c.mc_arena != nullptr && a.nlocal == 1;
    auto emit = [&](unsigned int g, uint32_t off, uint32_t size, const unsigned char* pk) {
      const uint4* s4 = reinterpret_cast<const uint4*>(pk);
      auto to = [&](char* slot_base) {
        char* grp = slot_base + (size_t)g * kGroupStride;
        if (threadIdx.x == 0) reinterpret_cast<uint32_t*>(grp)[k] = size;
        char* dst = grp + kGroupHeader + off;
        for (uint32_t i = threadIdx.x; i < size / 16; i += kSzThreads) stg(dst + 16 * i, s4[i]);
      };
      if (mode == 0) {
        to(a.local_out);
      } else if (use_mc) {
        char* grp = a.c.mc_arena + area + (size_t)r * a.slot_bytes + (size_t)g * kGroupStride;
        if (threadIdx.x == 0) multimem_st_u32(grp + 4 * k, size);
        char* dst = grp + kGroupHeader + off;
        for (uint32_t i = threadIdx.x; i < size / 16; i += kSzThreads) multimem_st(dst + 16 * i, s4[i]);
      } else {
        for (int j = 1; j < n; ++j) to(a.c.arena[(r + j) % n] + area + (size_t)r * a.slot_bytes);
      }
    };
    // broadcast: the root's CTAs publish their progress in kBcastWaves steps (flag slot =
    // wave), so that the receivers decode the first groups while the last are still packed
    const unsigned int my_iters = cl < a.ngroups ? (a.ngroups - cl + ncl - 1) / ncl : 0;
    auto wave_end = [&](unsigned int w) { return (unsigned int)(((unsigned long long)my_iters * (w + 1)) / kBcastWaves); };
    unsigned int wave = 0;
    float* own_out = kKind == 2 ? a.f[lr].out + (mode == 2 ? (size_t)r * a.nx * a.ny * a.nz : 0) : nullptr;
    prefetch(cl, 0);
    uint32_t it = 0, pend_size = 0, pend_off = 0;
    unsigned int pend_g = 0;
    bool pend = false;
    for (unsigned int g = cl; g < a.ngroups; g += ncl, ++it) {
      const int slot = it & 1;
      const unsigned int tile = g * kClusterSize + k;
      uint32_t size = 0;
      prefetch(g + ncl, slot ^ 1);   // that buffer was released by the __syncthreads ending the previous pack
      if (tile < ntiles) {
        float* cur = vals2[slot];
        if (a.use_tma) landed(slot);
        else load_tile_plain(in, cur, tile_coord(a, tile), a);
        __syncthreads();
        size = sync.fail ? 0 : pack_tile(cur, pk2[slot], s_tot, a, own_out, tile_coord(a, tile));
      } else {
        __syncthreads();   // keeps one CTA barrier per iteration between a copy-out and its signal
      }
      if (threadIdx.x == 0) s_size[slot] = size;
      // One cluster barrier per group, split in two so that the copy-out of the PREVIOUS
      // tile runs while the cluster gathers. s_size[slot] is rewritten two groups later,
      // after every CTA has passed the next barrier, when all reads of it are done.
      cluster_arrive();
      if (mode == 3 && it >= 1) {
        // Tiles 0 .. it-2 were copied out one iteration ago by every thread (the barriers of
        // the pack above order those copies before this point), so their stores have had
        // time to complete and the fence of the signal is short.
        while (wave < kBcastWaves && wave_end(wave) <= it - 1) {
          if (threadIdx.x == 0 && wave_end(wave) > (wave ? wave_end(wave - 1) : 0u))
            signal_peers(a.c, ((1u << n) - 1u) & ~(1u << r), (int)wave, r, b);
          ++wave;
        }
      }
      if (pend) emit(pend_g, pend_off, pend_size, pk2[slot ^ 1]);
      cluster_wait();
      uint32_t off = 0;
      for (int j = 0; j < k; ++j) off += *cluster.map_shared_rank(&s_size[slot], j);
      pend = true; pend_g = g; pend_off = off; pend_size = size;
      produced += size;
    }
    if (pend) emit(pend_g, pend_off, pend_size, pk2[(it - 1) & 1]);
    if (mode == 3) {     // the remaining waves (the last one always ends here)
      __syncthreads();
      if (threadIdx.x == 0)
        for (; wave < kBcastWaves; ++wave)
          if (wave_end(wave) > (wave ? wave_end(wave - 1) : 0u)) signal_peers(a.c, ((1u << n) - 1u) & ~(1u << r), (int)wave, r, b);
    }
    cluster.sync();      // nobody leaves while a neighbour may still read its sizes
    if (a.used_bytes && threadIdx.x == 0 && produced) atomicAdd(a.used_bytes + lr, produced + 0ull);
  }
  if (mode == 0) return;

  // --------------------------------------------------------------- signal ----
  if (collective) trace_mark(a.c, 1);
  if (collective) {
    __syncthreads();
    if (mode == 2 && threadIdx.x == 0) signal_peers(a.c, ((1u << n) - 1u) & ~(1u << r), 0, r, b);
    // All-gather waits source by source inside the decode loop; broadcast wave by wave.
  }

  // ------------------------------------------------------------ decompress ---
  // Work items (source, group) of this cluster, flattened; the size words of the next
  // item's group are fetched while this item is decoded.
  const int nsrc = mode == 2 ? n - 1 : (mode == 3 && r == a.root) ? 0 : 1;   // the sender's own copy is already written
  const unsigned int per_src = cl < a.ngroups ? (a.ngroups - cl + ncl - 1) / ncl : 0;
  const unsigned int nitems = per_src * nsrc;
  const int ln = threadIdx.x & 31;
  auto group_of = [&](unsigned int f) -> const char* {
    const int q = mode == 2 ? (r + 1 + (int)(f / per_src)) % n : a.root;
    const char* slot = mode == 1 ? a.local_in : a.c.arena[r] + area + (size_t)q * a.slot_bytes;
    return slot + (size_t)(cl + (f % per_src) * ncl) * kGroupStride;
  };
  auto valid = [&](unsigned int f) { return f < nitems && (cl + (f % per_src) * ncl) * kClusterSize + k < ntiles; };
  auto sizes_of = [&](unsigned int f) -> uint32_t {   // lane j < k gets the size of tile j of the group
    return (valid(f) && ln < k) ? ldg_cg_u32(group_of(f) + 4 * ln) : 0u;
  };
  if (collective) trace_mark(a.c, 2);
  auto dwave_end = [&](unsigned int w) { return (unsigned int)(((unsigned long long)per_src * (w + 1)) / kBcastWaves); };
  unsigned int dwave = 0;
  uint32_t sz_next = (mode == 1) ? sizes_of(0) : 0u;
  for (unsigned int f = 0; f < nitems; ++f) {
    if (collective && per_src && f == per_src) trace_mark(a.c, 3);   // first received field decoded
    if (mode == 2 && f % per_src == 0) {   // first item of the next source: its CTA of the same index must be done
      const int src = (r + 1 + (int)(f / per_src)) % n;
      if (!cta_wait_sources(sync, a.c, a.c.arena[r], 0, r, 1u << src, 0xA0)) return;
      sz_next = sizes_of(f);               // (re)read now that the source's bytes are visible
    }
    if (mode == 3) {                        // first item of the next wave of the root's CTA of the same index
      bool waited = false;
      while (dwave < kBcastWaves && (dwave ? dwave_end(dwave - 1) : 0u) <= f) {
        if (dwave_end(dwave) > (dwave ? dwave_end(dwave - 1) : 0u)) {
          if (!cta_wait_sources(sync, a.c, a.c.arena[r], (int)dwave, r, 1u << a.root, 0xA0)) return;
          waited = true;
        }
        ++dwave;
      }
      if (waited) sz_next = sizes_of(f);
    }
    const uint32_t sz = sz_next;
    // no prefetch across a source or wave boundary: those bytes may not have arrived yet
    const bool boundary = (mode == 2 && (f + 1) % per_src == 0) ||
                          (mode == 3 && dwave < kBcastWaves && (dwave ? dwave_end(dwave - 1) : 0u) <= f + 1);
    sz_next = boundary ? 0u : sizes_of(f + 1);
    if (!valid(f)) continue;
    uint32_t off = __reduce_add_sync(0xffffffffu, sz);
    if (off > (uint32_t)(kClusterSize * kTileCap)) {   // damaged size words: stay inside the slot and flag it
      off = 0;
      if (threadIdx.x == 0 && a.c.status) atomicOr(a.c.status + CCB_STATUS_FLAGS, CCB_ST_TIMEOUT);
    }
    const int q = mode == 2 ? (r + 1 + (int)(f / per_src)) % n : a.root;
    float* out = a.f[lr].out + (mode == 2 ? (size_t)q * a.nx * a.ny * a.nz : 0);
    unpack_tile(reinterpret_cast<const unsigned char*>(group_of(f)) + kGroupHeader + off, reinterpret_cast<int*>(vals2[0]), a,
                out, tile_coord(a, (cl + (f % per_src) * ncl) * kClusterSize + k));
  }
  if (collective) trace_mark(a.c, 4);
  if (mode == 3) end_handshake(sync, a.c, r);
}

// --------------------------------------------------------------------- host --
typedef CUresult (*encode_tiled_t)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                   const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                   CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static encode_tiled_t tensor_map_encoder() {
  static encode_tiled_t fn = nullptr;
  if (!fn) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess && q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<encode_tiled_t>(p);
    (void)cudaGetLastError();
  }
  return fn;
}

static bool make_tmap(CUtensorMap* m, const float* base, int nx, int ny, int nz) {
  encode_tiled_t enc = tensor_map_encoder();
  if (!enc || (nx % 4) != 0 || (reinterpret_cast<uintptr_t>(base) & 15) != 0) return false;
  cuuint64_t dims[3] = {(cuuint64_t)nx, (cuuint64_t)ny, (cuuint64_t)nz};
  cuuint64_t strides[2] = {(cuuint64_t)nx * 4, (cuuint64_t)nx * ny * 4};
  cuuint32_t box[3] = {kTX, kTY, kTZ};
  cuuint32_t estr[3] = {1, 1, 1};
  return enc(m, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3, const_cast<float*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
             CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

static void fill_geometry(SzArgs& a, int nx, int ny, int nz, float eb) {
  a.nx = nx; a.ny = ny; a.nz = nz;
  a.tiles_x = (nx + kTX - 1) / kTX;
  a.tiles_y = (ny + kTY - 1) / kTY;
  a.tiles_z = (nz + kTZ - 1) / kTZ;
  const unsigned long long tiles = (unsigned long long)a.tiles_x * a.tiles_y * a.tiles_z;
  a.ngroups = (unsigned int)((tiles + kClusterSize - 1) / kClusterSize);
  const unsigned long long txy = (unsigned long long)a.tiles_x * a.tiles_y;
  // tile indices run up to ngroups * kClusterSize (the last group may be partly empty)
  const unsigned long long max_tile = (unsigned long long)a.ngroups * kClusterSize;
  a.magic_x = ccb_fastdiv_magic(max_tile, (unsigned long long)a.tiles_x);
  a.magic_xy = ccb_fastdiv_magic(max_tile, txy);
  if (!a.magic_x || !a.magic_xy) a.magic_x = a.magic_xy = 0;
  a.eb = eb;
  a.two_eb = 2.f * eb * (1.f - 0.0009765625f);  // quantisation step: 2 eb (1 - 2^-10)
  a.inv_two_eb = 1.f / a.two_eb;
}

// How the last waiting launch went: 1 = cluster + cooperative accepted, 2 = refused and
// launched with the cluster attribute alone (co-residency then rests on the occupancy bound).
static int g_sz_launch_path = 0;

// Launch with a cluster of 8 CTAs; cooperative when the kernel waits on peers.
static int sz_launch(SzArgs& a, int nlocal, int num_sms, bool waits, cudaStream_t stream) {
  void (*kernel)(const SzArgs) = a.mode == 0 ? sz_kernel<0> : a.mode == 1 ? sz_kernel<1> : sz_kernel<2>;
  cudaLaunchConfig_t cfg;
  memset(&cfg, 0, sizeof(cfg));
  cudaLaunchAttribute attrs[2];
  attrs[0].id = cudaLaunchAttributeClusterDimension;
  attrs[0].val.clusterDim.x = kClusterSize;
  attrs[0].val.clusterDim.y = 1;
  attrs[0].val.clusterDim.z = 1;
  cfg.blockDim = dim3(kSzThreads, 1, 1);
  cfg.dynamicSmemBytes = 0;
  cfg.stream = stream;
  cfg.attrs = attrs;
  cfg.numAttrs = 1;
  cfg.gridDim = dim3(kClusterSize, 1, 1);
  int max_clusters = 0;
  if (cudaOccupancyMaxActiveClusters(&max_clusters, kernel, &cfg) != cudaSuccess || max_clusters < 1) {
    (void)cudaGetLastError();
    max_clusters = num_sms / kClusterSize;
  }
  // CTAs that wait on peers must all be resident: stay within the resident clusters
  unsigned int clusters = a.ngroups;
  const unsigned int cap = (unsigned)(max_clusters / nlocal > 0 ? max_clusters / nlocal : 1);
  if (clusters > cap) clusters = cap;
  if (clusters * kClusterSize > CCB_MAX_CTAS) clusters = CCB_MAX_CTAS / kClusterSize;
  cfg.gridDim = dim3(clusters * kClusterSize, (unsigned)nlocal, 1);
  if (waits) {
    attrs[1].id = cudaLaunchAttributeCooperative;
    attrs[1].val.cooperative = 1;
    cfg.numAttrs = 2;
  }
  cudaError_t e = cudaLaunchKernelEx(&cfg, kernel, a);
  if (waits) g_sz_launch_path = 1;
  if (e != cudaSuccess && waits) {  // some drivers refuse cluster + cooperative: the bounded grid still fits
    (void)cudaGetLastError();
    cfg.numAttrs = 1;
    g_sz_launch_path = 2;
    e = cudaLaunchKernelEx(&cfg, kernel, a);
  }
  if (e != cudaSuccess) {
    set_error("sz kernel launch failed: %s", cudaGetErrorString(e));
    return CCB_ERR_CUDA;
  }
  count_launch();
  return CCB_OK;
}

static int device_sms() {
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  return sms;
}

}  // namespace ccb

using namespace ccb;

extern "C" int ccb_sz_launch_path(void) { return g_sz_launch_path; }

extern "C" uint64_t ccb_sz_capacity(int nx, int ny, int nz) {
  SzArgs a;
  memset(&a, 0, sizeof(a));
  fill_geometry(a, nx, ny, nz, 1.f);
  return (uint64_t)a.ngroups * kGroupStride;
}

extern "C" int ccb_sz_compress(const float* in, int nx, int ny, int nz, float eb, void* out, unsigned long long* d_used,
                               ccb_stream_t stream) {
  if (!in || !out || nx < 1 || ny < 1 || nz < 1 || !(eb > 0.f)) {
    set_error("ccb_sz_compress: bad arguments");
    return CCB_ERR_ARG;
  }
  SzArgs a;
  memset(&a, 0, sizeof(a));
  fill_geometry(a, nx, ny, nz, eb);
  a.c.nranks = 1;
  a.f[0].in = in;
  a.local_out = static_cast<char*>(out);
  a.used_bytes = d_used;
  a.use_tma = make_tmap(&a.tmap[0], in, nx, ny, nz) ? 1 : 0;
  a.mode = 0;
  a.nlocal = 1;
  if (d_used) cudaMemsetAsync(d_used, 0, sizeof(unsigned long long), static_cast<cudaStream_t>(stream));
  return sz_launch(a, 1, device_sms(), false, static_cast<cudaStream_t>(stream));
}

extern "C" int ccb_sz_decompress(const void* in, int nx, int ny, int nz, float eb, float* out, ccb_stream_t stream) {
  if (!in || !out || nx < 1 || ny < 1 || nz < 1 || !(eb > 0.f)) {
    set_error("ccb_sz_decompress: bad arguments");
    return CCB_ERR_ARG;
  }
  SzArgs a;
  memset(&a, 0, sizeof(a));
  fill_geometry(a, nx, ny, nz, eb);
  a.c.nranks = 1;
  a.f[0].out = out;
  a.local_in = static_cast<const char*>(in);
  a.mode = 1;
  a.nlocal = 1;
  return sz_launch(a, 1, device_sms(), false, static_cast<cudaStream_t>(stream));
}

// Error-bounded AllGather (root < 0) or Broadcast (root >= 0) of one nx*ny*nz field per
// rank. AllGather: recv holds nranks fields in rank order. d_used (optional, one
// counter per local rank, device memory) receives the compressed bytes each rank sent
// to ONE destination.
extern "C" int ccb_sz_collective(ccb_comm* c, const float* const* send, float* const* recv, int nx, int ny, int nz, float eb,
                                 int root, unsigned long long* d_used, ccb_stream_t stream_) {
  int rc = check_alive(c);
  if (rc) return rc;
  if (!send || !recv || nx < 1 || ny < 1 || nz < 1 || !(eb > 0.f)) {
    set_error("ccb_sz_collective: bad arguments");
    return CCB_ERR_ARG;
  }
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  const int n = ccb_comm_nranks(c), nlocal = ccb_comm_nlocal(c);
  SzArgs a;
  memset(&a, 0, sizeof(a));
  fill_geometry(a, nx, ny, nz, eb);
  a.slot_bytes = ((unsigned long long)a.ngroups * kGroupStride + 255ull) & ~255ull;
  a.c = comm_dev(c, 0);
  const int nslots = n;
  if ((unsigned long long)nslots * a.slot_bytes > a.c.half_bytes) {
    set_error("arena too small: an error-bounded collective of %d x %d x %d needs %llu bytes of staging (CCB_ARENA_MB)", nx, ny, nz,
              (unsigned long long)nslots * a.slot_bytes * 2 + CCB_DATA_OFFSET);
    return CCB_ERR_CAPACITY;
  }
  a.c = comm_dev(c, next_epoch(c));
  bool tma = true;
  for (int i = 0; i < nlocal; ++i) {
    a.f[i].in = send[i];
    a.f[i].out = recv[i];
    const bool sender = root < 0 || (ccb_comm_rank(c) + i) == root;
    if (sender && !make_tmap(&a.tmap[i], send[i], nx, ny, nz)) tma = false;
  }
  a.use_tma = tma ? 1 : 0;
  a.used_bytes = d_used;
  a.mode = root < 0 ? 2 : 3;
  a.root = root < 0 ? 0 : root;
  a.rank0 = ccb_comm_rank(c);
  a.nlocal = nlocal;
  {  // progress steps of a broadcast: every step costs the root a system fence
    static int waves = 0;
    if (!waves) {
      const char* e = getenv("CCB_SZ_BCAST_WAVES");
      waves = e ? atoi(e) : 2;
      if (waves < 1) waves = 1;
      if (waves > (int)kMaxBcastWaves) waves = (int)kMaxBcastWaves;
    }
    a.bcast_waves = (unsigned int)waves;
  }
  if (d_used) cudaMemsetAsync(d_used, 0, sizeof(unsigned long long) * nlocal, stream);
  return sz_launch(a, nlocal, device_sms(), true, stream);
}

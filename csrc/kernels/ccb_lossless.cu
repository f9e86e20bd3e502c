// Lossless float codec (f32 / bf16 / f16) on local memory, for the compression-hook ABI.
//
// The reference reaches a lossless GPU codec only through the external DietGPU library
// (userconfig/wrapper_code_examples/compression/dietgpu/dietgpu.cu:32-103:
// floatCompress / floatDecompress, exponents entropy-coded, the rest stored raw). This is
// an own sm_100a codec of the same shape: the exponent field of every value is split from
// sign and mantissa; sign and mantissa are stored raw in byte planes; the exponents of a
// block of 512 values are stored as (exponent - block minimum) in as many bit planes as the
// block's exponent range needs (0 to 8). Gradient-like and activation data keep the
// exponents of neighbouring values within a few octaves, so 3 to 5 planes replace 8 bits.
//
// Work decomposition: a warp owns a block of 512 values (16 per lane, like the other
// codecs); the bit planes are built with warp ballots, one 32-bit word per (plane,
// element-of-lane), and read back with warp-uniform loads. A CTA of 8 warps owns a TILE of
// 8 blocks = 4096 values and packs the variable-length exponent planes of its blocks
// back to back inside the tile's fixed-capacity slot:
//
//   container = [32-byte header][slot 0][slot 1]...          slot stride = 32 + 4096 * sizeof(T)
//   header    = u32 magic "CCBL", u32 dtype, u64 count, u64 used bytes (sum over slots), u64 0
//   slot      = u32 used bytes, u8 width[8], u8 kmin[8], 12 bytes 0,
//               rest section (fixed size): f32 3 byte planes of 4096 B (low, middle, sign|high)
//                                          bf16 1 byte plane (sign << 7 | mantissa)
//                                          f16 1 byte plane (mantissa low 8) + 3 bit planes
//                                              (mantissa bits 8, 9 and the sign), 48 words per block
//               exponent section: for block b, width[b] planes of 16 words:
//                                 word[p * 16 + j] bit l = bit p of (exponent - kmin[b]) of value 16 l + j
//
// A slot is never larger than its stride (8 planes = 1 byte per value = the raw exponent),
// so compression needs no size negotiation: a transport that wants the gain sends the
// `used` prefix of every slot, one that cannot (fixed-stride hooks) sends the stride.
#include <cuda_runtime.h>

#include "../rt/ccb_rt_internal.h"
#include "ccb_device.cuh"

namespace ccb {

constexpr int kLlThreads = 256;
constexpr int kLlBlocksPerTile = kLlThreads / 32;          // 8
constexpr int kLlTileElems = kLlBlocksPerTile * kWarpElems;  // 4096
constexpr uint32_t kLlMagic = 0x4C424343u;                 // "CCBL"
constexpr int kLlHeader = 32;

template <class T> struct LlTraits;
template <> struct LlTraits<float> {
  static constexpr int kExpBits = 8, kRestBytesPerTile = 3 * kLlTileElems;
  static __device__ __forceinline__ uint32_t key(uint32_t b) { return (b >> 23) & 0xffu; }
  static __device__ __forceinline__ uint32_t rest(uint32_t b) { return (b & 0x7fffffu) | ((b >> 31) << 23); }
  static __device__ __forceinline__ uint32_t join(uint32_t k, uint32_t r) { return ((r >> 23) << 31) | (k << 23) | (r & 0x7fffffu); }
};
template <> struct LlTraits<__nv_bfloat16> {
  static constexpr int kExpBits = 8, kRestBytesPerTile = kLlTileElems;
  static __device__ __forceinline__ uint32_t key(uint32_t b) { return (b >> 7) & 0xffu; }
  static __device__ __forceinline__ uint32_t rest(uint32_t b) { return (b & 0x7fu) | ((b >> 15) << 7); }
  static __device__ __forceinline__ uint32_t join(uint32_t k, uint32_t r) { return ((r >> 7) << 15) | (k << 7) | (r & 0x7fu); }
};
template <> struct LlTraits<__half> {
  static constexpr int kExpBits = 5, kRestBytesPerTile = kLlTileElems + 3 * kLlTileElems / 8;
  static __device__ __forceinline__ uint32_t key(uint32_t b) { return (b >> 10) & 0x1fu; }
  static __device__ __forceinline__ uint32_t rest(uint32_t b) { return (b & 0x3ffu) | ((b >> 15) << 10); }
  static __device__ __forceinline__ uint32_t join(uint32_t k, uint32_t r) { return ((r >> 10) << 15) | (k << 10) | (r & 0x3ffu); }
};

template <class T> __host__ __device__ constexpr size_t ll_slot_bytes() { return 32 + (size_t)kLlTileElems * sizeof(T); }

// The 16 values of a lane as bit patterns (zero beyond `limit`), and back.
template <class T>
__device__ __forceinline__ void ll_load_bits(const T* base, size_t idx, size_t limit, uint32_t (&b)[16]) {
  Raw16<T> raw;
  load16_raw<T>(base, idx, limit, raw);
#pragma unroll
  for (int k = 0; k < (int)sizeof(T); ++k) {
    const uint32_t w[4] = {raw.q[k].x, raw.q[k].y, raw.q[k].z, raw.q[k].w};
    if constexpr (sizeof(T) == 4) {
#pragma unroll
      for (int i = 0; i < 4; ++i) b[4 * k + i] = w[i];
    } else {
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        b[8 * k + 2 * i] = w[i] & 0xffffu;
        b[8 * k + 2 * i + 1] = w[i] >> 16;
      }
    }
  }
}
template <class T>
__device__ __forceinline__ void ll_store_bits(T* base, size_t idx, size_t limit, const uint32_t (&b)[16]) {
  T* p = base + idx;
  if (idx + 16 <= limit && (reinterpret_cast<uintptr_t>(p) & 15) == 0) {
    if constexpr (sizeof(T) == 4) {
#pragma unroll
      for (int k = 0; k < 4; ++k) stg_stream(reinterpret_cast<char*>(p) + 16 * k, make_uint4(b[4 * k], b[4 * k + 1], b[4 * k + 2], b[4 * k + 3]));
    } else {
#pragma unroll
      for (int k = 0; k < 2; ++k)
        stg_stream(reinterpret_cast<char*>(p) + 16 * k,
                   make_uint4(b[8 * k] | (b[8 * k + 1] << 16), b[8 * k + 2] | (b[8 * k + 3] << 16),
                              b[8 * k + 4] | (b[8 * k + 5] << 16), b[8 * k + 6] | (b[8 * k + 7] << 16)));
    }
  } else {
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      if (idx + i < limit) {
        if constexpr (sizeof(T) == 4) reinterpret_cast<uint32_t*>(p)[i] = b[i];
        else reinterpret_cast<unsigned short*>(p)[i] = (unsigned short)b[i];
      }
    }
  }
}

__device__ __forceinline__ uint4 pack16_bytes(const uint32_t (&v)[16], int shift) {
  uint32_t w[4];
#pragma unroll
  for (int k = 0; k < 4; ++k)
    w[k] = ((v[4 * k] >> shift) & 0xffu) | (((v[4 * k + 1] >> shift) & 0xffu) << 8) | (((v[4 * k + 2] >> shift) & 0xffu) << 16) |
           (((v[4 * k + 3] >> shift) & 0xffu) << 24);
  return make_uint4(w[0], w[1], w[2], w[3]);
}
__device__ __forceinline__ void unpack16_bytes(uint4 q, int shift, uint32_t (&v)[16]) {
  const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
  for (int k = 0; k < 4; ++k)
#pragma unroll
    for (int i = 0; i < 4; ++i) v[4 * k + i] |= ((w[k] >> (8 * i)) & 0xffu) << shift;
}

// Word `idx` of a run of ballot words: every lane gets the same `word`; lane idx % 32
// keeps it in hold[idx / 32], so that the run is written with one coalesced store per 32 words.
template <int N>
__device__ __forceinline__ void keep_word(uint32_t (&hold)[N], int idx, uint32_t word, int lane) {
#pragma unroll
  for (int h = 0; h < N; ++h)
    if ((idx >> 5) == h && (idx & 31) == lane) hold[h] = word;
}

template <class T>
__global__ void __launch_bounds__(kLlThreads) lossless_encode_kernel(const T* __restrict__ in, size_t count, char* out, size_t ntiles) {
  using Tr = LlTraits<T>;
  __shared__ uint32_t widths[kLlBlocksPerTile], kmins[kLlBlocksPerTile];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  unsigned long long* total = reinterpret_cast<unsigned long long*>(out + 16);
  for (size_t t = blockIdx.x; t < ntiles; t += gridDim.x) {
    char* slot = out + kLlHeader + t * ll_slot_bytes<T>();
    const size_t idx = t * kLlTileElems + (size_t)warp * kWarpElems + (size_t)lane * kLaneElems;
    uint32_t b[16], key[16], rest[16];
    ll_load_bits<T>(in, idx, count, b);
    uint32_t kmin = 0xffu, kmax = 0u;
#pragma unroll
    for (int j = 0; j < 16; ++j) {
      key[j] = Tr::key(b[j]);
      rest[j] = Tr::rest(b[j]);
      kmin = min(kmin, key[j]);
      kmax = max(kmax, key[j]);
    }
    kmin = __reduce_min_sync(0xffffffffu, kmin);
    kmax = __reduce_max_sync(0xffffffffu, kmax);
    const int w = kmax == kmin ? 0 : 32 - __clz(kmax - kmin);
    if (lane == 0) {
      widths[warp] = (uint32_t)w;
      kmins[warp] = kmin;
    }
    // sign and mantissa: raw byte planes (and for f16 three ballot planes)
    char* restp = slot + 32;
    if constexpr (sizeof(T) == 4) {
#pragma unroll
      for (int p = 0; p < 3; ++p) stg(restp + (size_t)p * kLlTileElems + warp * kWarpElems + lane * 16, pack16_bytes(rest, 8 * p));
    } else {
      stg(restp + warp * kWarpElems + lane * 16, pack16_bytes(rest, 0));
      if constexpr (Tr::kExpBits == 5) {
        uint32_t hold[2] = {0u, 0u};
#pragma unroll
        for (int p = 0; p < 3; ++p)
#pragma unroll
          for (int j = 0; j < 16; ++j) keep_word(hold, p * 16 + j, __ballot_sync(0xffffffffu, (rest[j] >> (8 + p)) & 1u), lane);
        uint32_t* hp = reinterpret_cast<uint32_t*>(restp + kLlTileElems) + warp * 48;
        hp[lane] = hold[0];
        if (lane < 16) hp[32 + lane] = hold[1];
      }
    }
    __syncthreads();
    uint32_t off = 0, all = 0;
#pragma unroll
    for (int k = 0; k < kLlBlocksPerTile; ++k) {
      if (k < warp) off += widths[k];
      all += widths[k];
    }
    // exponent planes of this block, behind those of the blocks before it
    uint32_t* ep = reinterpret_cast<uint32_t*>(slot + 32 + Tr::kRestBytesPerTile) + off * 16;
    uint32_t hold[4] = {0u, 0u, 0u, 0u};
    for (int p = 0; p < w; ++p) {
#pragma unroll
      for (int j = 0; j < 16; ++j) keep_word(hold, p * 16 + j, __ballot_sync(0xffffffffu, ((key[j] - kmin) >> p) & 1u), lane);
    }
#pragma unroll
    for (int h = 0; h < 4; ++h)
      if (h * 32 + lane < w * 16) ep[h * 32 + lane] = hold[h];
    if (warp == 0) {
      const uint32_t used = 32u + (uint32_t)Tr::kRestBytesPerTile + all * 64u;
      if (lane == 0) {
        *reinterpret_cast<uint32_t*>(slot) = used;
        atomicAdd(total, (unsigned long long)used);
      }
      if (lane < kLlBlocksPerTile) {
        reinterpret_cast<unsigned char*>(slot)[4 + lane] = (unsigned char)widths[lane];
        reinterpret_cast<unsigned char*>(slot)[12 + lane] = (unsigned char)kmins[lane];
      }
      if (lane < 3) reinterpret_cast<uint32_t*>(slot)[5 + lane] = 0u;
    }
    __syncthreads();  // widths[] is rewritten by the next tile
  }
}

// MODE 0: out = decoded values; MODE 1: out += decoded values (in T, one rounding)
template <class T, int MODE>
__global__ void __launch_bounds__(kLlThreads) lossless_decode_kernel(const char* __restrict__ in, size_t count, T* out, size_t ntiles) {
  using Tr = LlTraits<T>;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (size_t t = blockIdx.x; t < ntiles; t += gridDim.x) {
    const char* slot = in + kLlHeader + t * ll_slot_bytes<T>();
    const size_t idx = t * kLlTileElems + (size_t)warp * kWarpElems + (size_t)lane * kLaneElems;
    if (t * kLlTileElems + (size_t)warp * kWarpElems >= count) continue;
    const unsigned char* hdr = reinterpret_cast<const unsigned char*>(slot);
    uint32_t off = 0;
    for (int k = 0; k < warp; ++k) off += hdr[4 + k];
    const int w = hdr[4 + warp];
    const uint32_t kmin = hdr[12 + warp];
    uint32_t rest[16], key[16];
#pragma unroll
    for (int j = 0; j < 16; ++j) rest[j] = 0u, key[j] = 0u;
    const char* restp = slot + 32;
    if constexpr (sizeof(T) == 4) {
#pragma unroll
      for (int p = 0; p < 3; ++p)
        unpack16_bytes(*reinterpret_cast<const uint4*>(restp + (size_t)p * kLlTileElems + warp * kWarpElems + lane * 16), 8 * p, rest);
    } else {
      unpack16_bytes(*reinterpret_cast<const uint4*>(restp + warp * kWarpElems + lane * 16), 0, rest);
      if constexpr (Tr::kExpBits == 5) {
        const uint32_t* hp = reinterpret_cast<const uint32_t*>(restp + kLlTileElems) + warp * 48;
#pragma unroll
        for (int p = 0; p < 3; ++p)
#pragma unroll
          for (int j = 0; j < 16; ++j) rest[j] |= ((hp[p * 16 + j] >> lane) & 1u) << (8 + p);
      }
    }
    const uint32_t* ep = reinterpret_cast<const uint32_t*>(slot + 32 + Tr::kRestBytesPerTile) + off * 16;
    for (int p = 0; p < w; ++p) {
#pragma unroll
      for (int j = 0; j < 16; ++j) key[j] |= ((ep[p * 16 + j] >> lane) & 1u) << p;
    }
    uint32_t b[16];
#pragma unroll
    for (int j = 0; j < 16; ++j) b[j] = Tr::join(key[j] + kmin, rest[j]);
    if constexpr (MODE == 1) {
      uint32_t have[16];
      ll_load_bits<T>(out, idx, count, have);
#pragma unroll
      for (int j = 0; j < 16; ++j) b[j] = elem_bits(Elem<T>::from_f(bits_to_f<T>(b[j]) + bits_to_f<T>(have[j])));
    }
    ll_store_bits<T>(out, idx, count, b);
  }
}

static size_t ll_tiles(size_t count) { return (count + kLlTileElems - 1) / kLlTileElems; }
static size_t ll_slot(int dtype) { return dtype == CCB_F32 ? ll_slot_bytes<float>() : ll_slot_bytes<__half>(); }
static int ll_grid(size_t ntiles) {
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const size_t cap = (size_t)sms * 8;
  return (int)(ntiles < cap ? (ntiles ? ntiles : 1) : cap);
}

}  // namespace ccb

using namespace ccb;

extern "C" uint64_t ccb_lossless_max_bytes(int dtype, uint64_t count) {
  if (dtype != CCB_F32 && dtype != CCB_BF16 && dtype != CCB_F16) return 0;
  return kLlHeader + ll_tiles(count) * ll_slot(dtype);
}

extern "C" int ccb_lossless_encode(int dtype, const void* in, uint64_t count, void* out, void* stream) {
  if (!in || !out || (reinterpret_cast<uintptr_t>(out) & 15)) {
    set_error("ccb_lossless_encode: null or misaligned buffer (the container must be 16-byte aligned)");
    return CCB_ERR_ARG;
  }
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  struct { uint32_t magic, dtype; uint64_t count, used, zero; } h = {kLlMagic, (uint32_t)dtype, count, (uint64_t)kLlHeader, 0};
  if (cudaMemcpyAsync(out, &h, sizeof(h), cudaMemcpyHostToDevice, s) != cudaSuccess) {
    set_error("ccb_lossless_encode: header copy failed: %s", cudaGetErrorString(cudaGetLastError()));
    return CCB_ERR_CUDA;
  }
  const size_t nt = ll_tiles(count);
  if (nt == 0) return CCB_OK;
  const int g = ll_grid(nt);
  if (dtype == CCB_F32) lossless_encode_kernel<float><<<g, kLlThreads, 0, s>>>((const float*)in, count, (char*)out, nt);
  else if (dtype == CCB_BF16) lossless_encode_kernel<__nv_bfloat16><<<g, kLlThreads, 0, s>>>((const __nv_bfloat16*)in, count, (char*)out, nt);
  else if (dtype == CCB_F16) lossless_encode_kernel<__half><<<g, kLlThreads, 0, s>>>((const __half*)in, count, (char*)out, nt);
  else return CCB_ERR_UNSUPPORTED;
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    set_error("ccb_lossless_encode: %s", cudaGetErrorString(e));
    return CCB_ERR_CUDA;
  }
  count_launch();
  return CCB_OK;
}

extern "C" int ccb_lossless_decode(int dtype, const void* in, uint64_t count, void* out, int accumulate, void* stream) {
  if (!in || !out || (reinterpret_cast<uintptr_t>(in) & 15)) {
    set_error("ccb_lossless_decode: null or misaligned buffer");
    return CCB_ERR_ARG;
  }
  const size_t nt = ll_tiles(count);
  if (nt == 0) return CCB_OK;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int g = ll_grid(nt);
#define CCB_LL_DEC(T)                                                                                          \
  do {                                                                                                         \
    if (accumulate) lossless_decode_kernel<T, 1><<<g, kLlThreads, 0, s>>>((const char*)in, count, (T*)out, nt); \
    else lossless_decode_kernel<T, 0><<<g, kLlThreads, 0, s>>>((const char*)in, count, (T*)out, nt);            \
  } while (0)
  if (dtype == CCB_F32) CCB_LL_DEC(float);
  else if (dtype == CCB_BF16) CCB_LL_DEC(__nv_bfloat16);
  else if (dtype == CCB_F16) CCB_LL_DEC(__half);
  else return CCB_ERR_UNSUPPORTED;
#undef CCB_LL_DEC
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    set_error("ccb_lossless_decode: %s", cudaGetErrorString(e));
    return CCB_ERR_CUDA;
  }
  count_launch();
  return CCB_OK;
}

// Bytes a transport has to move for this container: the header plus the used prefix of
// every slot. Reads 8 bytes back from the device after synchronising `stream`.
extern "C" int ccb_lossless_used_bytes(const void* comp, uint64_t* bytes, void* stream) {
  if (!comp || !bytes) return CCB_ERR_ARG;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  unsigned long long v = 0;
  if (cudaMemcpyAsync(&v, static_cast<const char*>(comp) + 16, sizeof(v), cudaMemcpyDeviceToHost, s) != cudaSuccess ||
      cudaStreamSynchronize(s) != cudaSuccess) {
    set_error("ccb_lossless_used_bytes: %s", cudaGetErrorString(cudaGetLastError()));
    return CCB_ERR_CUDA;
  }
  *bytes = v;
  return CCB_OK;
}

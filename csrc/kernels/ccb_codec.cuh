// Wire codecs used inside the fused collective kernels. A codec turns the 16 fp32
// values a lane holds into a Packet (payload registers + block scale) and back;
// `store`/`load` move a Packet to/from a wire slot laid out as
//     [payload: pad elements][scales: pad / kGroup entries]
// where `pad` (a multiple of 512) is the slot's element extent. `encode` is
// warp-collective (lanes of one quantisation group share an absmax by shuffle), so
// every lane of a warp must call it together.
//
//   CodecNone<T>   elements travel as T (exact for T, used for the uncompressed paths)
//   CodecInt8<G>   int8, fp32 scale = absmax/127 per G values (G = 128 or 256)
//   CodecFp8       fp8 e4m3, ue8m0 (power-of-two) scale byte per 32 values
//   CodecInt4      int4, fp32 scale = absmax/7 per 128 values
//
// The reference's only GPU codec is int8 with a per-group reciprocal scale
// (userconfig/wrapper_code_examples/communication/plain_nccl_compress/
// plain_nccl_compress.cu:141-191), run as separate quantize / dequantize kernels
// around ncclSend / ncclRecv; here the codec lives in registers of the kernel that
// also moves the bytes.
#pragma once
#include <cuda_fp8.h>

#include "ccb_device.cuh"

namespace ccb {

template <class T>
struct CodecNone {
  static constexpr int kId = CCB_CODEC_NONE;
  static constexpr int kQ = sizeof(T);  // uint4 registers per lane
  struct Packet { uint4 q[kQ]; };
  static __host__ __device__ size_t slot_bytes(size_t pad) { return pad * sizeof(T); }
  static __device__ __forceinline__ void encode(const float (&v)[16], Packet& pk) {
    if constexpr (sizeof(T) == 4) {
#pragma unroll
      for (int k = 0; k < 4; ++k)
        pk.q[k] = make_uint4(__float_as_uint(v[4 * k]), __float_as_uint(v[4 * k + 1]),
                             __float_as_uint(v[4 * k + 2]), __float_as_uint(v[4 * k + 3]));
    } else {
#pragma unroll
      for (int k = 0; k < 2; ++k) {
        T* h = reinterpret_cast<T*>(&pk.q[k]);
#pragma unroll
        for (int i = 0; i < 8; ++i) h[i] = Elem<T>::from_f(v[8 * k + i]);
      }
    }
  }
  static __device__ __forceinline__ void decode(const Packet& pk, float (&v)[16]) {
    if constexpr (sizeof(T) == 4) {
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        v[4 * k] = __uint_as_float(pk.q[k].x); v[4 * k + 1] = __uint_as_float(pk.q[k].y);
        v[4 * k + 2] = __uint_as_float(pk.q[k].z); v[4 * k + 3] = __uint_as_float(pk.q[k].w);
      }
    } else {
#pragma unroll
      for (int k = 0; k < 2; ++k) {
        const T* h = reinterpret_cast<const T*>(&pk.q[k]);
#pragma unroll
        for (int i = 0; i < 8; ++i) v[8 * k + i] = Elem<T>::to_f(h[i]);
      }
    }
  }
  // The wire order inside one 512-element warp unit is register-major: vector k of
  // lane l sits at ((k * 32 + l) * 16) bytes, so that each store instruction of a warp
  // writes 512 contiguous bytes (full NVLink packets) instead of 16-byte pieces at a
  // 16*kQ-byte stride. Only `load` below ever reads this layout back.
  static __device__ __forceinline__ size_t wire_off(size_t idx, int k) {
    const size_t unit = idx / kWarpElems;
    const size_t lane = (idx % kWarpElems) / kLaneElems;
    return unit * (kWarpElems * sizeof(T)) + ((size_t)k * 32 + lane) * 16;
  }
  static __device__ __forceinline__ void store(char* slot, size_t pad, size_t idx, const Packet& pk) {
#pragma unroll
    for (int k = 0; k < kQ; ++k) stg(slot + wire_off(idx, k), pk.q[k]);
  }
  static __device__ __forceinline__ void load(const char* slot, size_t pad, size_t idx, Packet& pk) {
#pragma unroll
    for (int k = 0; k < kQ; ++k) pk.q[k] = ldg_cg(slot + wire_off(idx, k));
  }
  // `slot` is an address inside an NVLS multicast mapping: one store reaches every arena.
  static __device__ __forceinline__ void store_mc(char* slot, size_t pad, size_t idx, const Packet& pk) {
#pragma unroll
    for (int k = 0; k < kQ; ++k) mc_st16(slot + wire_off(idx, k), pk.q[k]);
  }
};

__device__ __forceinline__ float absmax16(const float (&v)[16]) {
  float m = 0.f;
#pragma unroll
  for (int i = 0; i < 16; ++i) m = fmaxf(m, fabsf(v[i]));
  return m;
}

template <int G>
struct CodecInt8 {
  static_assert(G == 128 || G == 256, "group must be 128 or 256");
  static constexpr int kId = (G == 128) ? CCB_CODEC_INT8 : CCB_CODEC_INT8_G256;
  static constexpr int kLanes = G / 16;  // lanes sharing one scale
  struct Packet { uint4 q; float scale; };
  static __host__ __device__ size_t slot_bytes(size_t pad) { return pad + pad / G * 4; }
  static __device__ __forceinline__ void encode(const float (&v)[16], Packet& pk) {
    float m = absmax16(v);
#pragma unroll
    for (int d = 1; d < kLanes; d <<= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, d));
    const float inv = m > 0.f ? 127.f / m : 0.f;
    pk.scale = m / 127.f;
    // Round to nearest even without a float-to-int conversion: adding 1.5 * 2^23 leaves the
    // integer (|v * inv| <= 127) in the low mantissa bits, two's complement in the low byte;
    // the product is rounded to fp32 first (no fused multiply-add), so the code is the
    // same as round-half-even of the fp32 product, which is what the restatements compute.
    auto q8 = [&](float x) { return __float_as_uint(__fadd_rn(__fmul_rn(x, inv), 12582912.f)); };
    uint32_t w[4];
#pragma unroll
    for (int k = 0; k < 4; ++k)
      w[k] = __byte_perm(__byte_perm(q8(v[4 * k]), q8(v[4 * k + 1]), 0x0040), __byte_perm(q8(v[4 * k + 2]), q8(v[4 * k + 3]), 0x0040), 0x5410);
    pk.q = make_uint4(w[0], w[1], w[2], w[3]);
  }
  // Integer to float without a conversion instruction: the byte, biased by 128, is dropped
  // into the low mantissa bits of 1.5 * 2^23 (one permute), and subtracting 1.5 * 2^23 + 128
  // leaves the signed value exactly. Three plain instructions per value on the ALU and FMA
  // pipes instead of shift, sign extension, conversion and multiply.
  static __device__ __forceinline__ void decode(const Packet& pk, float (&v)[16]) {
    const uint32_t w[4] = {pk.q.x, pk.q.y, pk.q.z, pk.q.w};
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const uint32_t x = w[k] ^ 0x80808080u;
      v[4 * k + 0] = __fmul_rn(__fadd_rn(__uint_as_float(__byte_perm(x, 0x4B400000u, 0x7650)), -12583040.f), pk.scale);
      v[4 * k + 1] = __fmul_rn(__fadd_rn(__uint_as_float(__byte_perm(x, 0x4B400000u, 0x7651)), -12583040.f), pk.scale);
      v[4 * k + 2] = __fmul_rn(__fadd_rn(__uint_as_float(__byte_perm(x, 0x4B400000u, 0x7652)), -12583040.f), pk.scale);
      v[4 * k + 3] = __fmul_rn(__fadd_rn(__uint_as_float(__byte_perm(x, 0x4B400000u, 0x7653)), -12583040.f), pk.scale);
    }
  }
  static __device__ __forceinline__ void store(char* slot, size_t pad, size_t idx, const Packet& pk) {
    stg(slot + idx, pk.q);
    if ((idx & (G - 1)) == 0) reinterpret_cast<float*>(slot + pad)[idx / G] = pk.scale;
  }
  static __device__ __forceinline__ void load(const char* slot, size_t pad, size_t idx, Packet& pk) {
    pk.q = ldg_cg(slot + idx);
    pk.scale = __uint_as_float(ldg_cg_u32(slot + pad + (idx / G) * 4));
  }
  static __device__ __forceinline__ void store_mc(char* slot, size_t pad, size_t idx, const Packet& pk) {
    mc_st16(slot + idx, pk.q);
    if ((threadIdx.x & (kLanes - 1)) == 0) mc_st4(slot + pad + (idx / G) * 4, __float_as_uint(pk.scale));
  }
};

// Symmetric 4-bit integers, fp32 scale = absmax/7 per 128 values: 0.53 bytes per value,
// a quarter of bf16. The reference reaches 4 bits only through the SDP4Bit-style
// compression wrapper (userconfig/wrapper_code_examples/compression/sdp4bit/
// sdp4bit.cu:38-51); its NCCL wrapper accepts NCCL_COMPRESS_BITS=4 but implements 8.
struct CodecInt4 {
  static constexpr int kId = CCB_CODEC_INT4;
  static constexpr int kGroup = 128;
  static constexpr int kLanes = kGroup / 16;
  struct Packet { uint2 q; float scale; };
  static __host__ __device__ size_t slot_bytes(size_t pad) { return pad / 2 + pad / kGroup * 4; }
  static __device__ __forceinline__ void encode(const float (&v)[16], Packet& pk) {
    float m = absmax16(v);
#pragma unroll
    for (int d = 1; d < kLanes; d <<= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, d));
    const float inv = m > 0.f ? 7.f / m : 0.f;
    pk.scale = m / 7.f;
    uint32_t w[2] = {0u, 0u};
#pragma unroll
    for (int i = 0; i < 16; ++i) w[i >> 3] |= ((uint32_t)__float2int_rn(v[i] * inv) & 0xfu) << (4 * (i & 7));
    pk.q = make_uint2(w[0], w[1]);
  }
  static __device__ __forceinline__ void decode(const Packet& pk, float (&v)[16]) {
    const uint32_t w[2] = {pk.q.x, pk.q.y};
#pragma unroll
    for (int i = 0; i < 16; ++i) v[i] = (float)((int)(w[i >> 3] << (28 - 4 * (i & 7))) >> 28) * pk.scale;
  }
  static __device__ __forceinline__ void store(char* slot, size_t pad, size_t idx, const Packet& pk) {
    stg8(slot + idx / 2, pk.q);
    if ((threadIdx.x & (kLanes - 1)) == 0) reinterpret_cast<float*>(slot + pad / 2)[idx / kGroup] = pk.scale;
  }
  static __device__ __forceinline__ void load(const char* slot, size_t pad, size_t idx, Packet& pk) {
    pk.q = ldg_cg8(slot + idx / 2);
    pk.scale = __uint_as_float(ldg_cg_u32(slot + pad / 2 + (idx / kGroup) * 4));
  }
  static __device__ __forceinline__ void store_mc(char* slot, size_t pad, size_t idx, const Packet& pk) {
    mc_st8(slot + idx / 2, pk.q);
    if ((threadIdx.x & (kLanes - 1)) == 0) mc_st4(slot + pad / 2 + (idx / kGroup) * 4, __float_as_uint(pk.scale));
  }
};

struct CodecFp8 {
  static constexpr int kId = CCB_CODEC_FP8;
  static constexpr int kGroup = 32;
  struct Packet { uint4 q; uint32_t e; };  // e = biased exponent byte (ue8m0)
  static __host__ __device__ size_t slot_bytes(size_t pad) { return pad + pad / 32; }
  // Smallest power of two 2^e with absmax * 2^-e <= 448 (largest e4m3 value).
  static __device__ __forceinline__ uint32_t scale_byte(float m) {
    const uint32_t bits = __float_as_uint(m);
    int e = (int)(bits >> 23) - 127 - 8 + ((bits & 0x7fffffu) > 0x600000u ? 1 : 0);
    e = max(-126, min(126, e));
    return (uint32_t)(e + 127);
  }
  static __device__ __forceinline__ void encode(const float (&v)[16], Packet& pk) {
    float m = absmax16(v);
    m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 1));
    pk.e = scale_byte(m);
    const float inv = __uint_as_float((254u - pk.e) << 23);  // 2^-e
    uint32_t w[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      uint32_t lo = __nv_cvt_float2_to_fp8x2(make_float2(v[4 * k] * inv, v[4 * k + 1] * inv), __NV_SATFINITE, __NV_E4M3);
      uint32_t hi = __nv_cvt_float2_to_fp8x2(make_float2(v[4 * k + 2] * inv, v[4 * k + 3] * inv), __NV_SATFINITE, __NV_E4M3);
      w[k] = lo | (hi << 16);
    }
    pk.q = make_uint4(w[0], w[1], w[2], w[3]);
  }
  static __device__ __forceinline__ void decode(const Packet& pk, float (&v)[16]) {
    const float s = __uint_as_float(pk.e << 23);  // 2^e
    const uint32_t w[4] = {pk.q.x, pk.q.y, pk.q.z, pk.q.w};
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      __half2_raw lo = __nv_cvt_fp8x2_to_halfraw2((__nv_fp8x2_storage_t)(w[k] & 0xffffu), __NV_E4M3);
      __half2_raw hi = __nv_cvt_fp8x2_to_halfraw2((__nv_fp8x2_storage_t)(w[k] >> 16), __NV_E4M3);
      float2 a = __half22float2(*reinterpret_cast<__half2*>(&lo));
      float2 b = __half22float2(*reinterpret_cast<__half2*>(&hi));
      v[4 * k] = a.x * s; v[4 * k + 1] = a.y * s; v[4 * k + 2] = b.x * s; v[4 * k + 3] = b.y * s;
    }
  }
  static __device__ __forceinline__ void store(char* slot, size_t pad, size_t idx, const Packet& pk) {
    stg(slot + idx, pk.q);
    if ((threadIdx.x & 1) == 0) reinterpret_cast<uint8_t*>(slot + pad)[idx / 32] = (uint8_t)pk.e;
  }
  static __device__ __forceinline__ void load(const char* slot, size_t pad, size_t idx, Packet& pk) {
    pk.q = ldg_cg(slot + idx);
    uint32_t e;
    asm volatile("ld.global.cg.u8 %0, [%1];" : "=r"(e) : "l"(slot + pad + idx / 32));
    pk.e = e & 0xffu;
  }
  // Multicast stores have no byte form: the four scale bytes of eight neighbouring lanes
  // travel as one word. Warp-collective (every lane of the warp must call it, with the
  // 32 lanes on 512 consecutive elements).
  static __device__ __forceinline__ void store_mc(char* slot, size_t pad, size_t idx, const Packet& pk) {
    mc_st16(slot + idx, pk.q);
    const int lane = threadIdx.x & 31;
    uint32_t w = pk.e;
    w |= __shfl_down_sync(0xffffffffu, pk.e, 2) << 8;
    w |= __shfl_down_sync(0xffffffffu, pk.e, 4) << 16;
    w |= __shfl_down_sync(0xffffffffu, pk.e, 6) << 24;
    if ((lane & 7) == 0) mc_st4(slot + pad + idx / 32, w);
  }
};

}  // namespace ccb

// Stand-alone codec kernels on local memory: encode, decode, decode+add,
// decode+add+re-encode of several inputs. They back the COCCL-style hook ABI
// (ncclCompress / ncclDecompress / ncclDecompressReduce / ncclDecompReduceComp), the
// nccl_send_compressed / nccl_recv_decompress helpers and the point-to-point path of
// the interposer, and decode the reference wrapper's own int8 wire
// ([f32 127/absmax x groups][int8 x count], plain_nccl_compress.cu:123-129).
//
// Reference kernels replaced: quantize_{f32,f16,f64}_i8, dequantize_i8_* and
// reduce_* (plain_nccl_compress.cu:141-325: one element per thread, a shared-memory
// tree reduction per group, grids capped at 65535 blocks without a grid-stride loop)
// and add_*_kernel (coccl_wrapper_template.cu:258-272). Here a lane owns 16 elements,
// the group maximum is a few warp shuffles, and every kernel is grid-stride.
#include <cuda_runtime.h>

#include "../rt/ccb_rt_internal.h"
#include "ccb_codec.cuh"

namespace ccb {

constexpr int kSaThreads = 256;

// blockIdx.y selects one of several equal chunks: chunk c reads in + c * in_stride elements
// and writes wire + c * wire_stride bytes, so that a chunked buffer is one launch.
template <class T, class C>
__global__ void __launch_bounds__(kSaThreads) encode_kernel(const T* __restrict__ in, size_t count, char* wire, size_t pad,
                                                            size_t in_stride, size_t wire_stride) {
  in += (size_t)blockIdx.y * in_stride;
  wire += (size_t)blockIdx.y * wire_stride;
  const size_t units = pad / kWarpElems;
  const size_t warp = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5, nwarps = ((size_t)gridDim.x * blockDim.x) >> 5;
  const int lane = threadIdx.x & 31;
  for (size_t u = warp; u < units; u += nwarps) {
    const size_t idx = u * kWarpElems + (size_t)lane * kLaneElems;
    float v[16];
    load16<T>(in, idx, count, v);
    typename C::Packet pk;
    C::encode(v, pk);
    C::store(wire, pad, idx, pk);
  }
}

// MODE 0: out = decode(wire); MODE 1: out += decode(wire)
template <class T, class C, int MODE>
__global__ void __launch_bounds__(kSaThreads) decode_kernel(const char* wire, size_t count, T* out, size_t pad,
                                                            size_t wire_stride, size_t out_stride) {
  wire += (size_t)blockIdx.y * wire_stride;
  out += (size_t)blockIdx.y * out_stride;
  const size_t units = pad / kWarpElems;
  const size_t warp = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5, nwarps = ((size_t)gridDim.x * blockDim.x) >> 5;
  const int lane = threadIdx.x & 31;
  for (size_t u = warp; u < units; u += nwarps) {
    const size_t idx = u * kWarpElems + (size_t)lane * kLaneElems;
    if (idx >= count) continue;
    typename C::Packet pk;
    C::load(wire, pad, idx, pk);
    float d[16];
    C::decode(pk, d);
    if (MODE == 1) {
      float a[16];
      load16<T>(out, idx, count, a);
#pragma unroll
      for (int i = 0; i < 16; ++i) d[i] += a[i];
    }
    store16<T>(out, idx, count, d);
  }
}

// inout += src, element-wise in T (one rounding): the "reduce" of hook libraries whose codec
// decodes into a temporary (coccl_wrapper_template.cu:258-272 add_*_kernel in the reference).
template <class T>
__global__ void __launch_bounds__(kSaThreads) accumulate_kernel(const T* __restrict__ src, T* inout, size_t count) {
  const size_t units = (count + kWarpElems - 1) / kWarpElems;
  const size_t warp = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5, nwarps = ((size_t)gridDim.x * blockDim.x) >> 5;
  const int lane = threadIdx.x & 31;
  for (size_t u = warp; u < units; u += nwarps) {
    const size_t idx = u * kWarpElems + (size_t)lane * kLaneElems;
    if (idx >= count) continue;
    float a[16], b[16];
    load16<T>(src, idx, count, a);
    load16<T>(inout, idx, count, b);
#pragma unroll
    for (int i = 0; i < 16; ++i) b[i] += a[i];
    store16<T>(inout, idx, count, b);
  }
}

struct WireList {
  const char* w[16];
  int n;
};

// wire_out = encode(sum_k decode(wires[k]))
template <class C>
__global__ void __launch_bounds__(kSaThreads) reduce_recode_kernel(const __grid_constant__ WireList wl, size_t count, char* wire_out, size_t pad) {
  const size_t units = pad / kWarpElems;
  const size_t warp = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5, nwarps = ((size_t)gridDim.x * blockDim.x) >> 5;
  const int lane = threadIdx.x & 31;
  for (size_t u = warp; u < units; u += nwarps) {
    const size_t idx = u * kWarpElems + (size_t)lane * kLaneElems;
    float acc[16];
#pragma unroll
    for (int i = 0; i < 16; ++i) acc[i] = 0.f;
    for (int k = 0; k < wl.n; ++k) {
      typename C::Packet pk;
      C::load(wl.w[k], pad, idx, pk);
      float d[16];
      C::decode(pk, d);
#pragma unroll
      for (int i = 0; i < 16; ++i) acc[i] += d[i];
    }
    typename C::Packet out;
    C::encode(acc, out);
    C::store(wire_out, pad, idx, out);
  }
}

// Reference wire v0: scales[g] = 127/absmax (1.0 when absmax < 1e-10), then int8 payload.
template <class T>
__global__ void __launch_bounds__(kSaThreads) refwire_encode_kernel(const T* __restrict__ in, size_t count, int group, float* scales, int8_t* q) {
  // one warp per group; group <= 4096
  const size_t warp = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5, nwarps = ((size_t)gridDim.x * blockDim.x) >> 5;
  const int lane = threadIdx.x & 31;
  const size_t ngroups = (count + group - 1) / group;
  for (size_t g = warp; g < ngroups; g += nwarps) {
    const size_t lo = g * group, hi = lo + group < count ? lo + group : count;
    float m = 0.f;
    for (size_t i = lo + lane; i < hi; i += 32) m = fmaxf(m, fabsf(Elem<T>::to_f(in[i])));
#pragma unroll
    for (int d = 16; d; d >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, d));
    const float inv = m < 1e-10f ? 1.0f : 127.0f / m;
    if (lane == 0) scales[g] = inv;
    for (size_t i = lo + lane; i < hi; i += 32) {
      float r = rintf(Elem<T>::to_f(in[i]) * inv);
      q[i] = (int8_t)fminf(fmaxf(r, -128.f), 127.f);
    }
  }
}
template <class T>
__global__ void __launch_bounds__(kSaThreads) refwire_decode_kernel(const float* scales, const int8_t* q, size_t count, int group, T* out) {
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < count; i += (size_t)gridDim.x * blockDim.x)
    out[i] = Elem<T>::from_f((float)q[i] * (1.0f / scales[i / group]));
}

// out[i] = op over p of parts[p * stride + i], for the element types the fused collectives
// do not carry (integers, double): the reduce step of the NCCL-free provider, which gathers
// the ranks' buffers first. op: CCB_OP_*, 4 = average (sum, then divided by nparts).
template <class T>
__global__ void __launch_bounds__(kSaThreads) fold_kernel(const T* __restrict__ parts, size_t stride, int nparts, size_t count, int op,
                                                          T* __restrict__ out) {
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < count; i += (size_t)gridDim.x * blockDim.x) {
    T acc = parts[i];
    for (int p = 1; p < nparts; ++p) {
      const T v = parts[(size_t)p * stride + i];
      acc = op == CCB_OP_PROD ? (T)(acc * v) : op == CCB_OP_MAX ? (v > acc ? v : acc) : op == CCB_OP_MIN ? (v < acc ? v : acc) : (T)(acc + v);
    }
    if (op == 4) acc = (T)(acc / (T)nparts);
    out[i] = acc;
  }
}

static int sa_grid(size_t units) {
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  size_t blocks = (units + (kSaThreads / 32) - 1) / (kSaThreads / 32);
  size_t cap = (size_t)sms * 8;
  if (blocks < 1) blocks = 1;
  return (int)(blocks < cap ? blocks : cap);
}

// Grid of a chunked launch: x covers one chunk (at most `cap` blocks over all chunks), y the chunks.
static dim3 sa_grid2(size_t units, size_t nchunks) {
  int gx = sa_grid(units);
  const size_t cap = 148 * 8;
  if (nchunks > 1 && (size_t)gx * nchunks > cap) gx = (int)(cap / nchunks > 0 ? cap / nchunks : 1);
  return dim3((unsigned)gx, (unsigned)nchunks, 1);
}

template <class T>
static int encode_t(int codec, const void* in, size_t count, void* wire, size_t pad, cudaStream_t s, size_t nchunks = 1,
                    size_t in_stride = 0, size_t wire_stride = 0) {
  const dim3 g = sa_grid2(pad / kWarpElems, nchunks);
#define CCB_ENC(C) encode_kernel<T, C><<<g, kSaThreads, 0, s>>>((const T*)in, count, (char*)wire, pad, in_stride, wire_stride)
  switch (codec) {
    case CCB_CODEC_NONE: CCB_ENC(CodecNone<T>); break;
    case CCB_CODEC_INT8: CCB_ENC(CodecInt8<128>); break;
    case CCB_CODEC_INT8_G256: CCB_ENC(CodecInt8<256>); break;
    case CCB_CODEC_FP8: CCB_ENC(CodecFp8); break;
    case CCB_CODEC_INT4: CCB_ENC(CodecInt4); break;
    default: return CCB_ERR_UNSUPPORTED;
  }
#undef CCB_ENC
  return CCB_OK;
}
template <class T, int MODE>
static int decode_t(int codec, const void* wire, size_t count, void* out, size_t pad, cudaStream_t s, size_t nchunks = 1,
                    size_t wire_stride = 0, size_t out_stride = 0) {
  const dim3 g = sa_grid2(pad / kWarpElems, nchunks);
#define CCB_DEC(C) decode_kernel<T, C, MODE><<<g, kSaThreads, 0, s>>>((const char*)wire, count, (T*)out, pad, wire_stride, out_stride)
  switch (codec) {
    case CCB_CODEC_NONE: CCB_DEC(CodecNone<T>); break;
    case CCB_CODEC_INT8: CCB_DEC(CodecInt8<128>); break;
    case CCB_CODEC_INT8_G256: CCB_DEC(CodecInt8<256>); break;
    case CCB_CODEC_FP8: CCB_DEC(CodecFp8); break;
    case CCB_CODEC_INT4: CCB_DEC(CodecInt4); break;
    default: return CCB_ERR_UNSUPPORTED;
  }
#undef CCB_DEC
  return CCB_OK;
}

static int finish(const char* what) {
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    set_error("%s: %s", what, cudaGetErrorString(e));
    return CCB_ERR_CUDA;
  }
  count_launch();
  return CCB_OK;
}

}  // namespace ccb

using namespace ccb;

static size_t pad_of(uint64_t count) { return (count + kWarpElems - 1) / kWarpElems * kWarpElems; }

extern "C" int ccb_encode(int codec, int dtype, const void* in, uint64_t count, void* wire, void* stream) {
  if (!count) return CCB_OK;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  int rc = dtype == CCB_F32    ? encode_t<float>(codec, in, count, wire, pad_of(count), s)
           : dtype == CCB_BF16 ? encode_t<__nv_bfloat16>(codec, in, count, wire, pad_of(count), s)
           : dtype == CCB_F16  ? encode_t<__half>(codec, in, count, wire, pad_of(count), s)
                               : CCB_ERR_UNSUPPORTED;
  return rc ? rc : finish("ccb_encode");
}

extern "C" int ccb_decode(int codec, int dtype, const void* wire, uint64_t count, void* out, void* stream) {
  if (!count) return CCB_OK;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  int rc = dtype == CCB_F32    ? decode_t<float, 0>(codec, wire, count, out, pad_of(count), s)
           : dtype == CCB_BF16 ? decode_t<__nv_bfloat16, 0>(codec, wire, count, out, pad_of(count), s)
           : dtype == CCB_F16  ? decode_t<__half, 0>(codec, wire, count, out, pad_of(count), s)
                               : CCB_ERR_UNSUPPORTED;
  return rc ? rc : finish("ccb_decode");
}

extern "C" int ccb_decode_reduce(int codec, int dtype, const void* wire, uint64_t count, void* inout, void* stream) {
  if (!count) return CCB_OK;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  int rc = dtype == CCB_F32    ? decode_t<float, 1>(codec, wire, count, inout, pad_of(count), s)
           : dtype == CCB_BF16 ? decode_t<__nv_bfloat16, 1>(codec, wire, count, inout, pad_of(count), s)
           : dtype == CCB_F16  ? decode_t<__half, 1>(codec, wire, count, inout, pad_of(count), s)
                               : CCB_ERR_UNSUPPORTED;
  return rc ? rc : finish("ccb_decode_reduce");
}

// The same three operations on `nchunks` equal chunks in ONE launch: chunk c holds
// chunk_count elements at element offset c * chunk_count of the plain buffer and its wire at
// byte offset c * wire_stride (wire_stride >= ccb_wire_bytes(codec, dtype, chunk_count), a
// multiple of 16). chunk_count must keep every chunk 16-byte aligned for the fast path;
// other counts work through the element-wise path.
extern "C" int ccb_encode_chunks(int codec, int dtype, const void* in, uint64_t chunk_count, uint64_t nchunks, void* wire,
                                 uint64_t wire_stride, void* stream) {
  if (!chunk_count || !nchunks) return CCB_OK;
  if (nchunks > 65535) {
    set_error("at most 65535 chunks per call");
    return CCB_ERR_ARG;
  }
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const size_t pad = pad_of(chunk_count);
  int rc = dtype == CCB_F32    ? encode_t<float>(codec, in, chunk_count, wire, pad, s, nchunks, chunk_count, wire_stride)
           : dtype == CCB_BF16 ? encode_t<__nv_bfloat16>(codec, in, chunk_count, wire, pad, s, nchunks, chunk_count, wire_stride)
           : dtype == CCB_F16  ? encode_t<__half>(codec, in, chunk_count, wire, pad, s, nchunks, chunk_count, wire_stride)
                               : CCB_ERR_UNSUPPORTED;
  return rc ? rc : finish("ccb_encode_chunks");
}
extern "C" int ccb_decode_chunks(int codec, int dtype, const void* wire, uint64_t wire_stride, uint64_t chunk_count,
                                 uint64_t nchunks, void* out, int accumulate, void* stream) {
  if (!chunk_count || !nchunks) return CCB_OK;
  if (nchunks > 65535) {
    set_error("at most 65535 chunks per call");
    return CCB_ERR_ARG;
  }
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const size_t pad = pad_of(chunk_count);
  int rc;
  if (accumulate)
    rc = dtype == CCB_F32    ? decode_t<float, 1>(codec, wire, chunk_count, out, pad, s, nchunks, wire_stride, chunk_count)
         : dtype == CCB_BF16 ? decode_t<__nv_bfloat16, 1>(codec, wire, chunk_count, out, pad, s, nchunks, wire_stride, chunk_count)
         : dtype == CCB_F16  ? decode_t<__half, 1>(codec, wire, chunk_count, out, pad, s, nchunks, wire_stride, chunk_count)
                             : CCB_ERR_UNSUPPORTED;
  else
    rc = dtype == CCB_F32    ? decode_t<float, 0>(codec, wire, chunk_count, out, pad, s, nchunks, wire_stride, chunk_count)
         : dtype == CCB_BF16 ? decode_t<__nv_bfloat16, 0>(codec, wire, chunk_count, out, pad, s, nchunks, wire_stride, chunk_count)
         : dtype == CCB_F16  ? decode_t<__half, 0>(codec, wire, chunk_count, out, pad, s, nchunks, wire_stride, chunk_count)
                             : CCB_ERR_UNSUPPORTED;
  return rc ? rc : finish("ccb_decode_chunks");
}

extern "C" int ccb_accumulate(int dtype, const void* src, void* inout, uint64_t count, void* stream) {
  if (!count) return CCB_OK;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int g = sa_grid((count + kWarpElems - 1) / kWarpElems);
  if (dtype == CCB_F32) accumulate_kernel<float><<<g, kSaThreads, 0, s>>>((const float*)src, (float*)inout, count);
  else if (dtype == CCB_BF16) accumulate_kernel<__nv_bfloat16><<<g, kSaThreads, 0, s>>>((const __nv_bfloat16*)src, (__nv_bfloat16*)inout, count);
  else if (dtype == CCB_F16) accumulate_kernel<__half><<<g, kSaThreads, 0, s>>>((const __half*)src, (__half*)inout, count);
  else return CCB_ERR_UNSUPPORTED;
  return finish("ccb_accumulate");
}

extern "C" int ccb_reduce_recode(int codec, const void* const* wires, int nwires, uint64_t count, void* wire_out, void* stream) {
  if (!count) return CCB_OK;
  if (nwires < 1 || nwires > 16) {
    set_error("ccb_reduce_recode takes 1..16 inputs");
    return CCB_ERR_ARG;
  }
  WireList wl;
  wl.n = nwires;
  for (int i = 0; i < nwires; ++i) wl.w[i] = static_cast<const char*>(wires[i]);
  const size_t pad = pad_of(count);
  const int g = sa_grid(pad / kWarpElems);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  switch (codec) {
    case CCB_CODEC_INT8: reduce_recode_kernel<CodecInt8<128>><<<g, kSaThreads, 0, s>>>(wl, count, (char*)wire_out, pad); break;
    case CCB_CODEC_INT8_G256: reduce_recode_kernel<CodecInt8<256>><<<g, kSaThreads, 0, s>>>(wl, count, (char*)wire_out, pad); break;
    case CCB_CODEC_FP8: reduce_recode_kernel<CodecFp8><<<g, kSaThreads, 0, s>>>(wl, count, (char*)wire_out, pad); break;
    case CCB_CODEC_INT4: reduce_recode_kernel<CodecInt4><<<g, kSaThreads, 0, s>>>(wl, count, (char*)wire_out, pad); break;
    case CCB_CODEC_NONE: reduce_recode_kernel<CodecNone<float>><<<g, kSaThreads, 0, s>>>(wl, count, (char*)wire_out, pad); break;
    default: return CCB_ERR_UNSUPPORTED;
  }
  return finish("ccb_reduce_recode");
}

extern "C" int ccb_fold(int xtype, int op, const void* parts, uint64_t stride, int nparts, uint64_t count, void* out, void* stream) {
  if (!count) return CCB_OK;
  if (nparts < 1 || op < 0 || op > 4) return CCB_ERR_ARG;
  const int g = sa_grid((count + 31) / 32);  // one thread per element, grid-stride beyond the cap
  cudaStream_t s = static_cast<cudaStream_t>(stream);
#define CCB_FOLD(T) fold_kernel<T><<<g, kSaThreads, 0, s>>>((const T*)parts, stride, nparts, count, op, (T*)out)
  switch (xtype) {
    case CCB_X_I8: CCB_FOLD(int8_t); break;
    case CCB_X_U8: CCB_FOLD(uint8_t); break;
    case CCB_X_I32: CCB_FOLD(int32_t); break;
    case CCB_X_U32: CCB_FOLD(uint32_t); break;
    case CCB_X_I64: CCB_FOLD(long long); break;
    case CCB_X_U64: CCB_FOLD(unsigned long long); break;
    case CCB_X_F64: CCB_FOLD(double); break;
    default: return CCB_ERR_UNSUPPORTED;
  }
#undef CCB_FOLD
  return finish("ccb_fold");
}

// Reference wire v0 (see the file comment). `wire` holds ceil(count/group) floats then count int8.
extern "C" int ccb_refwire_encode(int dtype, const void* in, uint64_t count, int group, void* wire, void* stream) {
  if (!count) return CCB_OK;
  if (group < 1 || group > 4096) return CCB_ERR_ARG;
  const size_t ng = (count + group - 1) / group;
  float* scales = static_cast<float*>(wire);
  int8_t* q = reinterpret_cast<int8_t*>(scales + ng);
  const int g = sa_grid(ng);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (dtype == CCB_F32) refwire_encode_kernel<float><<<g, kSaThreads, 0, s>>>((const float*)in, count, group, scales, q);
  else if (dtype == CCB_F16) refwire_encode_kernel<__half><<<g, kSaThreads, 0, s>>>((const __half*)in, count, group, scales, q);
  else if (dtype == CCB_BF16) refwire_encode_kernel<__nv_bfloat16><<<g, kSaThreads, 0, s>>>((const __nv_bfloat16*)in, count, group, scales, q);
  else return CCB_ERR_UNSUPPORTED;
  return finish("ccb_refwire_encode");
}
extern "C" int ccb_refwire_decode(int dtype, const void* wire, uint64_t count, int group, void* out, void* stream) {
  if (!count) return CCB_OK;
  if (group < 1 || group > 4096) return CCB_ERR_ARG;
  const size_t ng = (count + group - 1) / group;
  const float* scales = static_cast<const float*>(wire);
  const int8_t* q = reinterpret_cast<const int8_t*>(scales + ng);
  const int g = sa_grid((count + 255) / 256);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (dtype == CCB_F32) refwire_decode_kernel<float><<<g, kSaThreads, 0, s>>>(scales, q, count, group, (float*)out);
  else if (dtype == CCB_F16) refwire_decode_kernel<__half><<<g, kSaThreads, 0, s>>>(scales, q, count, group, (__half*)out);
  else if (dtype == CCB_BF16) refwire_decode_kernel<__nv_bfloat16><<<g, kSaThreads, 0, s>>>(scales, q, count, group, (__nv_bfloat16*)out);
  else return CCB_ERR_UNSUPPORTED;
  return finish("ccb_refwire_decode");
}

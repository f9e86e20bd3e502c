// Group-wise symmetric 4-bit / 8-bit quantisation behind the four compression hooks
// (ncclCompress, ncclDecompress, ncclDecompressReduce, ncclDecompReduceComp), with the
// chunk layout of the reference's SDP4Bit example
// (userconfig/wrapper_code_examples/compression/sdp4bit/sdp4bit.cu:56-61, 97-105):
//
//   [ChunkHeader 16 B {groups, bits, elems_per_group, dtype}] [f32 scale x groups] [packed ints]
//
// so that a peer built from either tree decodes the other's chunks. What differs is how:
// the reference calls DeepSpeed-style quantise kernels, writes the header with a
// host-to-device copy and reads it back with a device-to-host copy and a stream
// synchronisation on every decompress (:125, :155-157). Here the kernels are in this file,
// the encoder writes the header itself and the decoders read it on the device, so no call
// ever synchronises; decode+add is one kernel.
//
// Environment: SDP4BIT_BITS = 4 (default) | 8, SDP4BIT_GROUP = elements per scale
// (default 256, a multiple of 32, at most 4096). Types: fp32, fp16, bf16.
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <nccl.h>
#include <stdint.h>
#include <stdlib.h>

typedef enum {
  AlltoAll = 0, AlltoAll_Inter = 1, AllReduce = 2, AllReduce_Inter = 3, AllGather = 4, AllGather_Inter = 5,
  ReduceScatter = 6, ReduceScatter_Inter = 7, SendRecv = 8, SendRecv_BWD = 9
} ncclCommOp_t;

struct ChunkHeader { int32_t groups, bits, elems_per_group, dtype; };

static int env_int(const char* name, int dflt) {
  const char* e = getenv(name);
  return e && *e ? atoi(e) : dflt;
}
static int cfg_bits() { static int b = 0; if (!b) b = env_int("SDP4BIT_BITS", 4) == 8 ? 8 : 4; return b; }
static int cfg_group() {
  static int g = 0;
  if (!g) {
    g = env_int("SDP4BIT_GROUP", 256);
    if (g < 32) g = 32;
    if (g > 4096) g = 4096;
    g -= g % 32;
  }
  return g;
}
static size_t type_size(ncclDataType_t t) { return t == ncclFloat32 ? 4 : (t == ncclFloat16 || (int)t == 9) ? 2 : 0; }
static size_t groups_of(size_t count) { return (count + cfg_group() - 1) / cfg_group(); }
static size_t packed_bytes(size_t count, int bits) { return bits == 8 ? count : (count + 1) / 2; }
// Bytes of one chunk of `count` elements, rounded so that consecutive chunks stay 16-byte aligned.
static size_t chunk_bytes(size_t count) {
  const size_t b = sizeof(ChunkHeader) + 4 * groups_of(count) + packed_bytes(count, cfg_bits());
  return (b + 15) & ~(size_t)15;
}

template <class T> __device__ __forceinline__ float to_f(T x);
template <> __device__ __forceinline__ float to_f<float>(float x) { return x; }
template <> __device__ __forceinline__ float to_f<__half>(__half x) { return __half2float(x); }
template <> __device__ __forceinline__ float to_f<__nv_bfloat16>(__nv_bfloat16 x) { return __bfloat162float(x); }
template <class T> __device__ __forceinline__ T from_f(float x);
template <> __device__ __forceinline__ float from_f<float>(float x) { return x; }
template <> __device__ __forceinline__ __half from_f<__half>(float x) { return __float2half_rn(x); }
template <> __device__ __forceinline__ __nv_bfloat16 from_f<__nv_bfloat16>(float x) { return __float2bfloat16_rn(x); }

// One warp per group, chunks along blockIdx.y. `in` is numChunks x count elements (or fp32
// when T = float is used for the re-encode), `out` numChunks x stride bytes.
template <class T>
__global__ void __launch_bounds__(256) quant_kernel(const T* in, size_t count, int group, int bits, int dtype, char* out, size_t stride) {
  const size_t chunk = blockIdx.y;
  const T* src = in + chunk * count;
  char* dst = out + chunk * stride;
  const size_t ngroups = (count + group - 1) / group;
  ChunkHeader* h = reinterpret_cast<ChunkHeader*>(dst);
  float* scales = reinterpret_cast<float*>(dst + sizeof(ChunkHeader));
  uint8_t* q = reinterpret_cast<uint8_t*>(scales + ngroups);
  if (blockIdx.x == 0 && threadIdx.x == 0) *h = ChunkHeader{(int32_t)ngroups, bits, group, dtype};
  const int lane = threadIdx.x & 31;
  const size_t warp = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5, nwarps = ((size_t)gridDim.x * blockDim.x) >> 5;
  const float qmax = bits == 8 ? 127.f : 7.f;
  for (size_t g = warp; g < ngroups; g += nwarps) {
    const size_t lo = g * group, hi = lo + group < count ? lo + group : count;
    float m = 0.f;
    for (size_t i = lo + lane; i < hi; i += 32) m = fmaxf(m, fabsf(to_f<T>(src[i])));
#pragma unroll
    for (int d = 16; d; d >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, d));
    const float scale = m / qmax, inv = m > 0.f ? qmax / m : 0.f;
    if (lane == 0) scales[g] = scale;
    if (bits == 8) {
      for (size_t i = lo + lane; i < hi; i += 32) q[i] = (uint8_t)(int8_t)__float2int_rn(to_f<T>(src[i]) * inv);
    } else {
      // two values per byte, low nibble first; a lane packs the pair (2j, 2j+1)
      for (size_t i = lo + 2 * lane; i < hi; i += 64) {
        const int a = __float2int_rn(to_f<T>(src[i]) * inv);
        const int b = i + 1 < hi ? __float2int_rn(to_f<T>(src[i + 1]) * inv) : 0;
        q[i >> 1] = (uint8_t)((a & 0xf) | ((b & 0xf) << 4));
      }
    }
  }
}

// kAdd: out += decode, else out = decode. The layout is read from the chunk's own header.
template <class T, bool kAdd>
__global__ void __launch_bounds__(256) dequant_kernel(const char* in, size_t stride, size_t count, T* out) {
  const size_t chunk = blockIdx.y;
  const char* src = in + chunk * stride;
  const ChunkHeader h = *reinterpret_cast<const ChunkHeader*>(src);
  if (h.groups <= 0 || h.elems_per_group <= 0 || (h.bits != 4 && h.bits != 8)) return;  // not a chunk of this format
  const float* scales = reinterpret_cast<const float*>(src + sizeof(ChunkHeader));
  const uint8_t* q = reinterpret_cast<const uint8_t*>(scales + h.groups);
  T* dst = out + chunk * count;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < count; i += (size_t)gridDim.x * blockDim.x) {
    const float s = scales[i / (size_t)h.elems_per_group];
    int v;
    if (h.bits == 8) v = (int8_t)q[i];
    else v = ((int)((uint32_t)(q[i >> 1] >> (4 * (i & 1))) << 28)) >> 28;  // sign-extend the nibble
    const float d = (float)v * s;
    dst[i] = kAdd ? from_f<T>(to_f<T>(dst[i]) + d) : from_f<T>(d);
  }
}

static dim3 grid_for(size_t units, size_t chunks) {
  size_t bx = (units + 7) / 8;  // 8 warps per block
  if (bx < 1) bx = 1;
  if (bx > 1184) bx = 1184;     // 8 blocks on each of 148 SMs
  return dim3((unsigned)bx, (unsigned)chunks, 1);
}

template <class T>
static ncclResult_t quant(const void* in, size_t count, size_t chunks, int dtype, void* out, cudaStream_t s) {
  quant_kernel<T><<<grid_for(groups_of(count), chunks), 256, 0, s>>>((const T*)in, count, cfg_group(), cfg_bits(), dtype, (char*)out, chunk_bytes(count));
  return cudaGetLastError() == cudaSuccess ? ncclSuccess : ncclUnhandledCudaError;
}
template <class T, bool kAdd>
static ncclResult_t dequant(const void* in, size_t stride, size_t count, size_t chunks, void* out, cudaStream_t s) {
  dequant_kernel<T, kAdd><<<grid_for((count + 255) / 256 * 8, chunks), 256, 0, s>>>((const char*)in, stride, count, (T*)out);
  return cudaGetLastError() == cudaSuccess ? ncclSuccess : ncclUnhandledCudaError;
}
#define BY_TYPE(dt, CALL)                                          \
  ((dt) == ncclFloat32 ? CALL(float) : (dt) == ncclFloat16 ? CALL(__half) : (int)(dt) == 9 ? CALL(__nv_bfloat16) : ncclInvalidArgument)

extern "C" {

size_t ncclCompressedChunkBytes(size_t chunkCount, ncclDataType_t datatype) { return type_size(datatype) ? chunk_bytes(chunkCount) : 0; }

ncclResult_t ncclCompress(const void* orgbuff, void** compbuff, const size_t orgChunkCount, ncclDataType_t orgDatatype,
                          size_t* compChunkCount, ncclDataType_t* compDatatype, const size_t numChunks, const int rank,
                          ncclCommOp_t commOp, cudaStream_t stream) {
  (void)rank; (void)commOp;
  if (!type_size(orgDatatype) || !compbuff || !numChunks) return ncclInvalidArgument;
  const size_t stride = chunk_bytes(orgChunkCount);
  *compChunkCount = stride;
  *compDatatype = ncclUint8;
  if (*compbuff == NULL && cudaMallocAsync(compbuff, stride * numChunks, stream) != cudaSuccess) return ncclUnhandledCudaError;
#define Q(T) quant<T>(orgbuff, orgChunkCount, numChunks, (int)orgDatatype, *compbuff, stream)
  return BY_TYPE(orgDatatype, Q);
#undef Q
}

ncclResult_t ncclDecompress(void* decompbuff, const void* compbuff, const size_t decompChunkCount, ncclDataType_t decompDatatype,
                            const size_t compChunkCount, ncclDataType_t compDatatype, const size_t numChunks,
                            ncclCommOp_t commOp, cudaStream_t stream) {
  (void)compDatatype; (void)commOp;
#define D(T) dequant<T, false>(compbuff, compChunkCount, decompChunkCount, numChunks, decompbuff, stream)
  return BY_TYPE(decompDatatype, D);
#undef D
}

ncclResult_t ncclDecompressReduce(void* reducebuff, const void* compbuff, const size_t compChunkCount, ncclDataType_t compDatatype,
                                  const size_t reduceChunkCount, ncclDataType_t reduceDataType, const size_t numChunks,
                                  ncclCommOp_t commOp, cudaStream_t stream) {
  (void)compDatatype; (void)commOp;
#define D(T) dequant<T, true>(compbuff, compChunkCount, reduceChunkCount, numChunks, reducebuff, stream)
  return BY_TYPE(reduceDataType, D);
#undef D
}

// *recompbuff = one chunk = encode(sum of the numChunks decoded chunks); the sum is kept in
// fp32 in a stream-ordered temporary.
ncclResult_t ncclDecompReduceComp(const void* compbuff, void** recompbuff, const size_t orgChunkCount, ncclDataType_t orgDatatype,
                                  const size_t compChunkCount, ncclDataType_t compDatatype, size_t* reCompChunkCount,
                                  ncclDataType_t* reCompDatatype, const size_t numChunks, ncclCommOp_t commOp, cudaStream_t stream) {
  (void)compDatatype; (void)commOp;
  if (!type_size(orgDatatype) || !recompbuff || !numChunks) return ncclInvalidArgument;
  const size_t stride = chunk_bytes(orgChunkCount);
  *reCompChunkCount = stride;
  *reCompDatatype = ncclUint8;
  if (*recompbuff == NULL && cudaMallocAsync(recompbuff, stride, stream) != cudaSuccess) return ncclUnhandledCudaError;
  float* acc = NULL;
  if (cudaMallocAsync((void**)&acc, orgChunkCount * sizeof(float), stream) != cudaSuccess) return ncclUnhandledCudaError;
  ncclResult_t rc = dequant<float, false>(compbuff, compChunkCount, orgChunkCount, 1, acc, stream);
  for (size_t c = 1; c < numChunks && rc == ncclSuccess; ++c)
    rc = dequant<float, true>((const char*)compbuff + c * compChunkCount, compChunkCount, orgChunkCount, 1, acc, stream);
  if (rc == ncclSuccess) rc = quant<float>(acc, orgChunkCount, 1, (int)orgDatatype, *recompbuff, stream);
  cudaFreeAsync(acc, stream);
  return rc;
}

}  // extern "C"

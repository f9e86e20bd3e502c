// Template for a GPU compression library behind the four hooks of a compressing transport:
// ncclCompress, ncclDecompress, ncclDecompressReduce, ncclDecompReduceComp.
//
// The reference ships a template of the same role and ABI at this path
// (userconfig/wrapper_code_examples/compression/coccl_wrapper_template.cu:64, 108, 141, 185):
// its hooks copy bytes per chunk and add with separate kernels (:258-279), and the user is
// meant to replace the copies by calls into a codec library. This template is organised the
// other way round: the user writes ONE small struct, a lane codec, and the four hooks come
// out as four kernels that each handle all chunks of a call in a single launch, including
// decode + add and decode + add over all chunks + re-encode fused into one pass.
//
//   struct MyCodec {
//     static constexpr int kGroup = ...;        // elements that share side information
//     static size_t chunk_bytes(size_t count);  // fixed stride of one compressed chunk
//     // one thread owns group g of a chunk: it reads kGroup floats and writes their code
//     static __device__ void encode(const float* v, int n, unsigned char* chunk, size_t count, size_t g);
//     static __device__ void decode(const unsigned char* chunk, size_t count, size_t g, float* v, int n);
//   };
//
// The example codec below keeps every value as a 16-bit float with one fp32 scale per group
// of 32 (2.06 x smaller than fp32): replace it, keep the rest. Element types: float, half,
// bfloat16. Build: nvcc -gencode arch=compute_100a,code=sm_100a -shared -Xcompiler -fPIC.
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <nccl.h>
#include <stdint.h>

typedef enum {
  AlltoAll = 0, AlltoAll_Inter = 1, AllReduce = 2, AllReduce_Inter = 3, AllGather = 4, AllGather_Inter = 5,
  ReduceScatter = 6, ReduceScatter_Inter = 7, SendRecv = 8, SendRecv_BWD = 9
} ncclCommOp_t;

// ------------------------------------------------------------------ USER SECTION --
struct ExampleCodec {
  static constexpr int kGroup = 32;
  // layout of a chunk: [fp32 scale per group][fp16 value per element], 16-byte granular
  static __host__ __device__ size_t groups(size_t count) { return (count + kGroup - 1) / kGroup; }
  static __host__ __device__ size_t chunk_bytes(size_t count) { return (groups(count) * 4 + count * 2 + 15) & ~(size_t)15; }
  static __device__ void encode(const float* v, int n, unsigned char* chunk, size_t count, size_t g) {
    float m = 0.f;
    for (int i = 0; i < n; ++i) m = fmaxf(m, fabsf(v[i]));
    const float scale = m > 0.f ? m : 1.f;   // values are stored relative to the group's absmax
    reinterpret_cast<float*>(chunk)[g] = scale;
    __half* q = reinterpret_cast<__half*>(chunk + groups(count) * 4) + g * kGroup;
    for (int i = 0; i < n; ++i) q[i] = __float2half_rn(v[i] / scale);
  }
  static __device__ void decode(const unsigned char* chunk, size_t count, size_t g, float* v, int n) {
    const float scale = reinterpret_cast<const float*>(chunk)[g];
    const __half* q = reinterpret_cast<const __half*>(chunk + groups(count) * 4) + g * kGroup;
    for (int i = 0; i < n; ++i) v[i] = __half2float(q[i]) * scale;
  }
};
using Codec = ExampleCodec;
// -------------------------------------------------------------- END USER SECTION --

namespace {

template <class T> __device__ __forceinline__ float to_f(T x);
template <> __device__ __forceinline__ float to_f<float>(float x) { return x; }
template <> __device__ __forceinline__ float to_f<__half>(__half x) { return __half2float(x); }
template <> __device__ __forceinline__ float to_f<__nv_bfloat16>(__nv_bfloat16 x) { return __bfloat162float(x); }
template <class T> __device__ __forceinline__ T from_f(float x);
template <> __device__ __forceinline__ float from_f<float>(float x) { return x; }
template <> __device__ __forceinline__ __half from_f<__half>(float x) { return __float2half_rn(x); }
template <> __device__ __forceinline__ __nv_bfloat16 from_f<__nv_bfloat16>(float x) { return __float2bfloat16_rn(x); }

constexpr int kThreads = 256;

// mode 0: comp[c] = encode(plain[c]); 1: plain[c] = decode(comp[c]); 2: plain[c] += decode(comp[c])
template <class T, int kMode>
__global__ void __launch_bounds__(kThreads) per_chunk_kernel(T* plain, unsigned char* comp, size_t count, size_t stride, size_t nchunks) {
  const size_t groups = Codec::groups(count), total = groups * nchunks;
  for (size_t w = (size_t)blockIdx.x * blockDim.x + threadIdx.x; w < total; w += (size_t)gridDim.x * blockDim.x) {
    const size_t c = w / groups, g = w - c * groups;
    const size_t first = g * Codec::kGroup;
    const int n = (int)(count - first < (size_t)Codec::kGroup ? count - first : Codec::kGroup);
    T* p = plain + c * count + first;
    unsigned char* ch = comp + c * stride;
    float v[Codec::kGroup];
    if (kMode == 0) {
      for (int i = 0; i < n; ++i) v[i] = to_f<T>(p[i]);
      Codec::encode(v, n, ch, count, g);
    } else {
      Codec::decode(ch, count, g, v, n);
      for (int i = 0; i < n; ++i) p[i] = from_f<T>(kMode == 2 ? to_f<T>(p[i]) + v[i] : v[i]);
    }
  }
}

// out = encode(sum over chunks of decode(comp[c])): the reduction step of a compressed ring,
// one pass, nothing decoded to memory
__global__ void __launch_bounds__(kThreads) sum_recode_kernel(const unsigned char* comp, size_t count, size_t stride, size_t nchunks,
                                                              unsigned char* out) {
  const size_t groups = Codec::groups(count);
  for (size_t g = (size_t)blockIdx.x * blockDim.x + threadIdx.x; g < groups; g += (size_t)gridDim.x * blockDim.x) {
    const size_t first = g * Codec::kGroup;
    const int n = (int)(count - first < (size_t)Codec::kGroup ? count - first : Codec::kGroup);
    float acc[Codec::kGroup], v[Codec::kGroup];
    for (int i = 0; i < n; ++i) acc[i] = 0.f;
    for (size_t c = 0; c < nchunks; ++c) {
      Codec::decode(comp + c * stride, count, g, v, n);
      for (int i = 0; i < n; ++i) acc[i] += v[i];
    }
    Codec::encode(acc, n, out, count, g);
  }
}

int grid_for(size_t work) {
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  size_t blocks = (work + kThreads - 1) / kThreads, cap = (size_t)sms * 8;
  return (int)(blocks < 1 ? 1 : blocks < cap ? blocks : cap);
}

template <int kMode>
ncclResult_t per_chunk(void* plain, void* comp, size_t count, ncclDataType_t dt, size_t stride, size_t nchunks, cudaStream_t s) {
  if (count == 0 || nchunks == 0) return ncclSuccess;
  const int g = grid_for(Codec::groups(count) * nchunks);
  unsigned char* c = static_cast<unsigned char*>(comp);
  if (dt == ncclFloat32) per_chunk_kernel<float, kMode><<<g, kThreads, 0, s>>>((float*)plain, c, count, stride, nchunks);
  else if (dt == ncclFloat16) per_chunk_kernel<__half, kMode><<<g, kThreads, 0, s>>>((__half*)plain, c, count, stride, nchunks);
  else if ((int)dt == 9) per_chunk_kernel<__nv_bfloat16, kMode><<<g, kThreads, 0, s>>>((__nv_bfloat16*)plain, c, count, stride, nchunks);
  else return ncclInvalidArgument;
  return cudaGetLastError() == cudaSuccess ? ncclSuccess : ncclUnhandledCudaError;
}

}  // namespace

extern "C" {

// Stride between compressed chunks: fixed, so that the transport needs no size exchange.
size_t ncclCompressedChunkBytes(size_t chunkCount, ncclDataType_t datatype) {
  (void)datatype;
  return Codec::chunk_bytes(chunkCount);
}

ncclResult_t ncclCompress(const void* orgbuff, void** compbuff, const size_t orgChunkCount, ncclDataType_t orgDatatype,
                          size_t* compChunkCount, ncclDataType_t* compDatatype, const size_t numChunks, const int rank,
                          ncclCommOp_t commOp, cudaStream_t stream) {
  (void)rank; (void)commOp;
  if (!compbuff || !compChunkCount || !compDatatype) return ncclInvalidArgument;
  const size_t stride = Codec::chunk_bytes(orgChunkCount);
  *compChunkCount = stride;
  *compDatatype = ncclUint8;
  if (*compbuff == nullptr && cudaMallocAsync(compbuff, stride * numChunks, stream) != cudaSuccess) return ncclUnhandledCudaError;
  return per_chunk<0>(const_cast<void*>(orgbuff), *compbuff, orgChunkCount, orgDatatype, stride, numChunks, stream);
}

ncclResult_t ncclDecompress(void* decompbuff, const void* compbuff, const size_t decompChunkCount, ncclDataType_t decompDatatype,
                            const size_t compChunkCount, ncclDataType_t compDatatype, const size_t numChunks, ncclCommOp_t commOp,
                            cudaStream_t stream) {
  (void)compDatatype; (void)commOp;
  return per_chunk<1>(decompbuff, const_cast<void*>(compbuff), decompChunkCount, decompDatatype, compChunkCount, numChunks, stream);
}

ncclResult_t ncclDecompressReduce(void* reducebuff, const void* compbuff, const size_t compChunkCount, ncclDataType_t compDatatype,
                                  const size_t reduceChunkCount, ncclDataType_t reduceDataType, const size_t numChunks,
                                  ncclCommOp_t commOp, cudaStream_t stream) {
  (void)compDatatype; (void)commOp;
  return per_chunk<2>(reducebuff, const_cast<void*>(compbuff), reduceChunkCount, reduceDataType, compChunkCount, numChunks, stream);
}

ncclResult_t ncclDecompReduceComp(const void* compbuff, void** recompbuff, const size_t orgChunkCount, ncclDataType_t orgDatatype,
                                  const size_t compChunkCount, ncclDataType_t compDatatype, size_t* reCompChunkCount,
                                  ncclDataType_t* reCompDatatype, const size_t numChunks, ncclCommOp_t commOp, cudaStream_t stream) {
  (void)orgDatatype; (void)compDatatype; (void)commOp;
  if (!recompbuff || !reCompChunkCount || !reCompDatatype || numChunks == 0) return ncclInvalidArgument;
  const size_t stride = Codec::chunk_bytes(orgChunkCount);
  *reCompChunkCount = stride;
  *reCompDatatype = ncclUint8;
  if (*recompbuff == nullptr && cudaMallocAsync(recompbuff, stride, stream) != cudaSuccess) return ncclUnhandledCudaError;
  if (orgChunkCount == 0) return ncclSuccess;
  sum_recode_kernel<<<grid_for(Codec::groups(orgChunkCount)), kThreads, 0, stream>>>(
      static_cast<const unsigned char*>(compbuff), orgChunkCount, compChunkCount, numChunks, static_cast<unsigned char*>(*recompbuff));
  return cudaGetLastError() == cudaSuccess ? ncclSuccess : ncclUnhandledCudaError;
}

}  // extern "C"

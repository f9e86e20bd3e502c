/* Error-bounded GPU compression behind the four compression hooks (ncclCompress,
 * ncclDecompress, ncclDecompressReduce, ncclDecompReduceComp), for float32.
 *
 * Role of the reference's cuZFP wrapper (userconfig/wrapper_code_examples/compression/
 * zfp_for_gpu_nvidia/zfp_for_gpu_nvidia.cu:46-71, 120-185: cuda_compress / cuda_decompress
 * of a 1-D field in fixed-precision mode, chunk layout [u32 stream_bytes][bitstream]).
 * cuZFP is an external library; the codec here is libccb.so's own error-bounded GPU codec
 * (csrc/kernels/ccb_sz.cu: quantise under an absolute bound, Lorenzo prediction inside
 * tiles, bit-plane packing), which makes the transport-independent codec of the fused
 * AllGather / Broadcast usable by an NCCL fork with compression hooks.
 *
 * Chunk layout (the reference's): [u32 stream_bytes][12 bytes 0][stream], at a fixed stride.
 * The header word is written on the device (no host synchronisation; the reference reads
 * it back with a synchronising copy, :158-159).
 * Accuracy: ZFP_PRECISION = p (default 14, the reference's variable) gives the absolute
 * bound 2^-p; CCB_SZ_ABS_EB, when set, gives it directly.
 * A chunk is viewed as a field of 64 x 64 x (n / 4096) values when n is a multiple of 4096,
 * of 32 x 8 x (n / 256) when a multiple of 256, else as one row. */
#include <cuda_runtime.h>
#include <math.h>
#include <nccl.h>
#include <stdint.h>
#include <stdlib.h>

#include "ccb/ccb.h"
#include "ccb/ccb_sz.h"

typedef enum {
    AlltoAll = 0, AlltoAll_Inter = 1, AllReduce = 2, AllReduce_Inter = 3, AllGather = 4, AllGather_Inter = 5,
    ReduceScatter = 6, ReduceScatter_Inter = 7, SendRecv = 8, SendRecv_BWD = 9
} ncclCommOp_t;

#define HDR 16

static float bound(void) {
    const char *e = getenv("CCB_SZ_ABS_EB");
    if (e && atof(e) > 0) return (float)atof(e);
    e = getenv("ZFP_PRECISION");
    const int p = e ? atoi(e) : 14;
    return ldexpf(1.0f, -(p < 1 ? 1 : p > 40 ? 40 : p));
}
static void shape(size_t n, int *nx, int *ny, int *nz) {
    if (n % 4096 == 0 && n / 4096 <= 0x7fffffff) { *nx = 64; *ny = 64; *nz = (int)(n / 4096); }
    else if (n % 256 == 0 && n / 256 <= 0x7fffffff) { *nx = 32; *ny = 8; *nz = (int)(n / 256); }
    else { *nx = (int)n; *ny = 1; *nz = 1; }
}

size_t ncclCompressedChunkBytes(size_t chunkCount, ncclDataType_t datatype) {
    if (datatype != ncclFloat32 || chunkCount == 0 || chunkCount > 0x7fffffffu) return 0;
    int nx, ny, nz;
    shape(chunkCount, &nx, &ny, &nz);
    return HDR + (size_t)ccb_sz_capacity(nx, ny, nz);
}

ncclResult_t ncclCompress(const void *orgbuff, void **compbuff, const size_t orgChunkCount, ncclDataType_t orgDatatype,
                          size_t *compChunkCount, ncclDataType_t *compDatatype, const size_t numChunks, const int rank,
                          ncclCommOp_t commOp, cudaStream_t stream) {
    (void)rank;
    (void)commOp;
    const size_t stride = ncclCompressedChunkBytes(orgChunkCount, orgDatatype);
    if (stride == 0 || !compbuff) return ncclInternalError;
    *compDatatype = ncclUint8;
    *compChunkCount = stride;
    if (*compbuff == NULL && cudaMallocAsync(compbuff, stride * numChunks, stream) != cudaSuccess) return ncclInternalError;
    int nx, ny, nz;
    shape(orgChunkCount, &nx, &ny, &nz);
    unsigned long long *used = NULL;
    if (cudaMallocAsync((void **)&used, sizeof(*used) * numChunks, stream) != cudaSuccess) return ncclInternalError;
    int bad = 0;
    for (size_t c = 0; c < numChunks && !bad; ++c) {
        char *chunk = (char *)*compbuff + c * stride;
        bad = cudaMemsetAsync(chunk, 0, HDR, stream) != cudaSuccess ||
              ccb_sz_compress((const float *)orgbuff + c * orgChunkCount, nx, ny, nz, bound(), chunk + HDR, used + c, stream) != CCB_OK ||
              cudaMemcpyAsync(chunk, used + c, 4, cudaMemcpyDeviceToDevice, stream) != cudaSuccess; /* low word, little-endian */
    }
    cudaFreeAsync(used, stream);
    return bad ? ncclInternalError : ncclSuccess;
}

ncclResult_t ncclDecompress(void *decompbuff, const void *compbuff, const size_t decompChunkCount,
                            ncclDataType_t decompDatatype, const size_t compChunkCount, ncclDataType_t compDatatype,
                            const size_t numChunks, ncclCommOp_t commOp, cudaStream_t stream) {
    (void)compDatatype;
    (void)commOp;
    if (decompDatatype != ncclFloat32) return ncclInternalError;
    int nx, ny, nz;
    shape(decompChunkCount, &nx, &ny, &nz);
    for (size_t c = 0; c < numChunks; ++c)
        if (ccb_sz_decompress((const char *)compbuff + c * compChunkCount + HDR, nx, ny, nz, bound(),
                              (float *)decompbuff + c * decompChunkCount, stream))
            return ncclInternalError;
    return ncclSuccess;
}

/* reducebuff[c] += decode(compbuff[c]): decode into a stream-ordered temporary, one add kernel */
ncclResult_t ncclDecompressReduce(void *reducebuff, const void *compbuff, const size_t compChunkCount,
                                  ncclDataType_t compDatatype, const size_t reduceChunkCount, ncclDataType_t reduceDataType,
                                  const size_t numChunks, ncclCommOp_t commOp, cudaStream_t stream) {
    if (reduceDataType != ncclFloat32) return ncclInternalError;
    void *tmp = NULL;
    if (cudaMallocAsync(&tmp, reduceChunkCount * numChunks * sizeof(float), stream) != cudaSuccess) return ncclInternalError;
    ncclResult_t rc = ncclDecompress(tmp, compbuff, reduceChunkCount, reduceDataType, compChunkCount, compDatatype, numChunks, commOp, stream);
    if (rc == ncclSuccess && ccb_accumulate(CCB_F32, tmp, reducebuff, reduceChunkCount * numChunks, stream)) rc = ncclInternalError;
    cudaFreeAsync(tmp, stream);
    return rc;
}

/* *recompbuff = encode(sum over the numChunks compressed chunks) */
ncclResult_t ncclDecompReduceComp(const void *compbuff, void **recompbuff, const size_t orgChunkCount,
                                  ncclDataType_t orgDatatype, const size_t compChunkCount, ncclDataType_t compDatatype,
                                  size_t *reCompChunkCount, ncclDataType_t *reCompDatatype, const size_t numChunks,
                                  ncclCommOp_t commOp, cudaStream_t stream) {
    if (orgDatatype != ncclFloat32 || numChunks == 0 || !recompbuff) return ncclInternalError;
    void *sum = NULL, *tmp = NULL;
    const size_t bytes = orgChunkCount * sizeof(float);
    if (cudaMallocAsync(&sum, bytes, stream) != cudaSuccess || cudaMallocAsync(&tmp, bytes, stream) != cudaSuccess) return ncclInternalError;
    ncclResult_t rc = ncclDecompress(sum, compbuff, orgChunkCount, orgDatatype, compChunkCount, compDatatype, 1, commOp, stream);
    for (size_t c = 1; c < numChunks && rc == ncclSuccess; ++c) {
        rc = ncclDecompress(tmp, (const char *)compbuff + c * compChunkCount, orgChunkCount, orgDatatype, compChunkCount, compDatatype, 1,
                            commOp, stream);
        if (rc == ncclSuccess && ccb_accumulate(CCB_F32, tmp, sum, orgChunkCount, stream)) rc = ncclInternalError;
    }
    if (rc == ncclSuccess)
        rc = ncclCompress(sum, recompbuff, orgChunkCount, orgDatatype, reCompChunkCount, reCompDatatype, 1, 0, commOp, stream);
    cudaFreeAsync(sum, stream);
    cudaFreeAsync(tmp, stream);
    return rc;
}

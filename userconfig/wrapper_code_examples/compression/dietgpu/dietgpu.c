/* Lossless float compression behind the four compression hooks (ncclCompress,
 * ncclDecompress, ncclDecompressReduce, ncclDecompReduceComp), for f32 / f16 / bf16.
 *
 * Role of the reference's DietGPU wrapper (userconfig/wrapper_code_examples/compression/
 * dietgpu/dietgpu.cu:32-103: three callbacks over dietgpu::floatCompress /
 * floatDecompress under coccl_wrapper_template.cu). DietGPU itself is an external
 * library; here the codec is libccb.so's own (csrc/kernels/ccb_lossless.cu: exponents of
 * 512-value blocks in bit planes relative to the block minimum, sign and mantissa raw).
 * Like getMaxFloatCompressedSize the chunk stride is the worst case (raw size plus
 * headers); the bytes actually used are in the container header
 * (ccb_lossless_used_bytes), which is what a ratio measurement reads.
 *
 * All chunks of a call are independent containers at the fixed stride. DecompressReduce
 * adds in the element type (one rounding); DecompReduceComp sums the chunks in a
 * stream-ordered temporary and compresses the sum. */
#include <cuda_runtime.h>
#include <nccl.h>
#include <stdint.h>

#include "dietgpu_common.h"

typedef enum {
    AlltoAll = 0, AlltoAll_Inter = 1, AllReduce = 2, AllReduce_Inter = 3, AllGather = 4, AllGather_Inter = 5,
    ReduceScatter = 6, ReduceScatter_Inter = 7, SendRecv = 8, SendRecv_BWD = 9
} ncclCommOp_t;

static int hook_dtype(ncclDataType_t t) { return lossless_dtype_of(t); }
static size_t esz(int dt) { return lossless_elem_bytes(dt); }

size_t ncclCompressedChunkBytes(size_t chunkCount, ncclDataType_t datatype) {
    const int dt = hook_dtype(datatype);
    return dt < 0 ? 0 : (size_t)ccb_lossless_max_bytes(dt, chunkCount);
}

ncclResult_t ncclCompress(const void *orgbuff, void **compbuff, const size_t orgChunkCount, ncclDataType_t orgDatatype,
                          size_t *compChunkCount, ncclDataType_t *compDatatype, const size_t numChunks, const int rank,
                          ncclCommOp_t commOp, cudaStream_t stream) {
    (void)rank;
    (void)commOp;
    const int dt = hook_dtype(orgDatatype);
    const size_t stride = ncclCompressedChunkBytes(orgChunkCount, orgDatatype);
    if (dt < 0 || stride == 0 || !compbuff) return ncclInternalError;
    *compDatatype = ncclUint8;
    *compChunkCount = stride;
    if (*compbuff == NULL && cudaMallocAsync(compbuff, stride * numChunks, stream) != cudaSuccess) return ncclInternalError;
    for (size_t c = 0; c < numChunks; ++c)
        if (ccb_lossless_encode(dt, (const char *)orgbuff + c * orgChunkCount * esz(dt), orgChunkCount,
                                (char *)*compbuff + c * stride, stream))
            return ncclInternalError;
    return ncclSuccess;
}

ncclResult_t ncclDecompress(void *decompbuff, const void *compbuff, const size_t decompChunkCount,
                            ncclDataType_t decompDatatype, const size_t compChunkCount, ncclDataType_t compDatatype,
                            const size_t numChunks, ncclCommOp_t commOp, cudaStream_t stream) {
    (void)compDatatype;
    (void)commOp;
    const int dt = hook_dtype(decompDatatype);
    if (dt < 0) return ncclInternalError;
    for (size_t c = 0; c < numChunks; ++c)
        if (ccb_lossless_decode(dt, (const char *)compbuff + c * compChunkCount, decompChunkCount,
                                (char *)decompbuff + c * decompChunkCount * esz(dt), 0, stream))
            return ncclInternalError;
    return ncclSuccess;
}

ncclResult_t ncclDecompressReduce(void *reducebuff, const void *compbuff, const size_t compChunkCount,
                                  ncclDataType_t compDatatype, const size_t reduceChunkCount, ncclDataType_t reduceDataType,
                                  const size_t numChunks, ncclCommOp_t commOp, cudaStream_t stream) {
    (void)compDatatype;
    (void)commOp;
    const int dt = hook_dtype(reduceDataType);
    if (dt < 0) return ncclInternalError;
    for (size_t c = 0; c < numChunks; ++c)
        if (ccb_lossless_decode(dt, (const char *)compbuff + c * compChunkCount, reduceChunkCount,
                                (char *)reducebuff + c * reduceChunkCount * esz(dt), 1, stream))
            return ncclInternalError;
    return ncclSuccess;
}

ncclResult_t ncclDecompReduceComp(const void *compbuff, void **recompbuff, const size_t orgChunkCount,
                                  ncclDataType_t orgDatatype, const size_t compChunkCount, ncclDataType_t compDatatype,
                                  size_t *reCompChunkCount, ncclDataType_t *reCompDatatype, const size_t numChunks,
                                  ncclCommOp_t commOp, cudaStream_t stream) {
    (void)compDatatype;
    (void)commOp;
    const int dt = hook_dtype(orgDatatype);
    const size_t stride = ncclCompressedChunkBytes(orgChunkCount, orgDatatype);
    if (dt < 0 || numChunks == 0 || stride == 0 || !recompbuff) return ncclInternalError;
    *reCompDatatype = ncclUint8;
    *reCompChunkCount = stride;
    if (*recompbuff == NULL && cudaMallocAsync(recompbuff, stride, stream) != cudaSuccess) return ncclInternalError;
    void *sum = NULL;
    if (cudaMallocAsync(&sum, orgChunkCount * esz(dt), stream) != cudaSuccess) return ncclInternalError;
    int bad = 0;
    for (size_t c = 0; c < numChunks && !bad; ++c)
        bad = ccb_lossless_decode(dt, (const char *)compbuff + c * compChunkCount, orgChunkCount, sum, c > 0, stream);
    if (!bad) bad = ccb_lossless_encode(dt, sum, orgChunkCount, *recompbuff, stream);
    cudaFreeAsync(sum, stream);
    return bad ? ncclInternalError : ncclSuccess;
}

/* COCCL-style compression hook ABI implemented with the sm_100a codec kernels of
 * libccb.so: ncclCompress, ncclDecompress, ncclDecompressReduce, ncclDecompReduceComp.
 *
 * The ABI is the one the reference's template exports (userconfig/
 * wrapper_code_examples/compression/coccl_wrapper_template.cu:64, 108, 141, 185): a
 * buffer is cut into `numChunks` pieces, each compressed into a fixed stride of
 * `*compChunkBytes` bytes so that the transport needs no size exchange. The
 * reference's template decompresses to temporaries and adds with separate kernels
 * (:161-176, 212-247); here decode+add and decode+add+re-encode are single kernels.
 * Codec: $CCB_HOOK_CODEC = int8 (default) | fp8 | int8_g256 | int4 | none. */
#include <cuda_runtime.h>
#include <nccl.h>
#include <stdint.h>
#include <stdlib.h>
#include <strings.h>

#include "ccb/ccb.h"

/* Operation tags of the ABI (values as in coccl_wrapper_template.cu:33-37); unused here. */
typedef enum {
    AlltoAll = 0, AlltoAll_Inter = 1, AllReduce = 2, AllReduce_Inter = 3, AllGather = 4, AllGather_Inter = 5,
    ReduceScatter = 6, ReduceScatter_Inter = 7, SendRecv = 8, SendRecv_BWD = 9
} ncclCommOp_t;

static int hook_codec(void) {
    const char *e = getenv("CCB_HOOK_CODEC");
    if (!e || !strcasecmp(e, "int8")) return CCB_CODEC_INT8;
    if (!strcasecmp(e, "fp8")) return CCB_CODEC_FP8;
    if (!strcasecmp(e, "int4")) return CCB_CODEC_INT4;
    if (!strcasecmp(e, "int8_g256")) return CCB_CODEC_INT8_G256;
    return CCB_CODEC_NONE;
}
static int hook_dtype(ncclDataType_t t) {
    if (t == ncclFloat32) return CCB_F32;
    if (t == ncclFloat16) return CCB_F16;
    if ((int)t == 9) return CCB_BF16;
    return -1;
}

/* Bytes one compressed chunk occupies (the fixed stride between chunks). */
size_t ncclCompressedChunkBytes(size_t chunkCount, ncclDataType_t datatype) {
    const int dt = hook_dtype(datatype);
    return dt < 0 ? 0 : (size_t)ccb_wire_bytes(hook_codec(), dt, chunkCount);
}

/* orgbuff: numChunks x orgChunkCount elements -> *compbuff: numChunks x *compChunkCount
 * bytes (allocated stream-ordered when *compbuff is NULL). */
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
    /* all chunks in one launch (the reference's template launches per chunk, :74-100) */
    return ccb_encode_chunks(hook_codec(), dt, orgbuff, orgChunkCount, numChunks, *compbuff, stride, stream) ? ncclInternalError
                                                                                                           : ncclSuccess;
}

ncclResult_t ncclDecompress(void *decompbuff, const void *compbuff, const size_t decompChunkCount,
                            ncclDataType_t decompDatatype, const size_t compChunkCount, ncclDataType_t compDatatype,
                            const size_t numChunks, ncclCommOp_t commOp, cudaStream_t stream) {
    (void)compDatatype;
    (void)commOp;
    const int dt = hook_dtype(decompDatatype);
    if (dt < 0) return ncclInternalError;
    return ccb_decode_chunks(hook_codec(), dt, compbuff, compChunkCount, decompChunkCount, numChunks, decompbuff, 0, stream)
               ? ncclInternalError
               : ncclSuccess;
}

/* reducebuff[c] += decode(compbuff[c]) for every chunk, one kernel for all chunks. */
ncclResult_t ncclDecompressReduce(void *reducebuff, const void *compbuff, const size_t compChunkCount,
                                  ncclDataType_t compDatatype, const size_t reduceChunkCount, ncclDataType_t reduceDataType,
                                  const size_t numChunks, ncclCommOp_t commOp, cudaStream_t stream) {
    (void)compDatatype;
    (void)commOp;
    const int dt = hook_dtype(reduceDataType);
    if (dt < 0) return ncclInternalError;
    return ccb_decode_chunks(hook_codec(), dt, compbuff, compChunkCount, reduceChunkCount, numChunks, reducebuff, 1, stream)
               ? ncclInternalError
               : ncclSuccess;
}

/* *recompbuff = encode(sum over the numChunks compressed chunks): one chunk out. */
ncclResult_t ncclDecompReduceComp(const void *compbuff, void **recompbuff, const size_t orgChunkCount,
                                  ncclDataType_t orgDatatype, const size_t compChunkCount, ncclDataType_t compDatatype,
                                  size_t *reCompChunkCount, ncclDataType_t *reCompDatatype, const size_t numChunks,
                                  ncclCommOp_t commOp, cudaStream_t stream) {
    (void)compDatatype;
    (void)commOp;
    const size_t stride = ncclCompressedChunkBytes(orgChunkCount, orgDatatype);
    if (hook_dtype(orgDatatype) < 0 || numChunks == 0 || stride == 0 || !recompbuff) return ncclInternalError;
    *reCompDatatype = ncclUint8;
    *reCompChunkCount = stride;
    if (*recompbuff == NULL && cudaMallocAsync(recompbuff, stride, stream) != cudaSuccess) return ncclInternalError;
    size_t done = 0;
    const void *wires[16];
    int first = 1;
    while (done < numChunks) { /* up to 16 inputs per pass; later passes fold the running total back in */
        int k = 0;
        if (!first) wires[k++] = *recompbuff;
        while (k < 16 && done < numChunks) wires[k++] = (const char *)compbuff + (done++) * compChunkCount;
        if (ccb_reduce_recode(hook_codec(), wires, k, orgChunkCount, *recompbuff, stream)) return ncclInternalError;
        first = 0;
    }
    return ncclSuccess;
}

/* perfnccl: LD_PRELOAD perf wrapper for the NCCL path. Put FIRST in LD_PRELOAD: it
 * sees the outermost call, times it, forwards to the next library (the fused
 * interposer, a compression wrapper, or libnccl) and notes one row per call.
 *
 * Columns follow the reference's NCCL perf wrappers (userconfig/wrapper_code_examples/
 * perf/perfcoccl/perfcoccl.c and perfuccl/perfuccl.c): p2p -> duration, msg_bytes,
 * count, intra; collectives -> duration, data_bytes; compression hooks -> duration,
 * input_size, output_size, compression_ratio (output / input, as perfcoccl.c:151).
 * `duration` is host wall-clock around the call in seconds (enqueue time for
 * asynchronous calls); with PERF_NCCL_DEVICE_TIME=1 a `device_duration` column with
 * the CUDA-event time of the call on its stream is added. Buffers are offered to the
 * gendata capture (perf_gendata_dump_if_target) for device pointers only when
 * PERF_GENDATA_DEVICE=1, through a bounce copy to the host.
 *
 * Build (no nccl.h / CUDA headers needed):
 *   cc -O2 -fPIC -shared perfnccl.c <repo>/csrc/wrappers/perf_helper_nccl.c \
 *      <repo>/csrc/core/perf.c -I run_codes/wrappers/include -I run_codes/wrappers -ldl -lpthread */
#define _GNU_SOURCE
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#include "nccl/perf_helper_nccl.h"
#include "perf_helper.h"

typedef int ncclCommOp_t;

static void capture(const char *func, const void *dev, size_t bytes) {
    static int mode = -1;
    if (mode < 0) {
        const char *e = getenv("PERF_GENDATA_DEVICE");
        mode = e && *e == '1';
    }
    perf_state_t *s = perf_nccl_get_tls();
    if (!getenv("PERF_GENDATA_TARGETS")) return;
    if (!mode || !dev || !bytes) {
        perf_gendata_dump_if_target(s, func, NULL, 0);
        return;
    }
    typedef int (*memcpy_t)(void *, const void *, size_t, int);
    static memcpy_t cpy;
    if (!cpy) cpy = (memcpy_t)dlsym(RTLD_DEFAULT, "cudaMemcpy");
    void *h = cpy ? malloc(bytes) : NULL;
    if (h && cpy(h, dev, bytes, 2 /* cudaMemcpyDeviceToHost */) == 0) perf_gendata_dump_if_target(s, func, h, bytes);
    else perf_gendata_dump_if_target(s, func, NULL, 0);
    free(h);
}

ncclResult_t ncclCommInitRank(ncclComm_t *comm, int nranks, ncclUniqueId commId, int rank) {
    PERF_NCCL_REAL(ncclCommInitRank);
    const double t0 = perf_get_time();
    ncclResult_t r = real_ncclCommInitRank(comm, nranks, commId, rank);
    perf_attr_t a[] = {{"duration", perf_get_time() - t0}, {"nranks", (double)nranks}};
    perf_notedown(perf_nccl_get_tls(), "ncclCommInitRank", t0, 2, a);
    if (r == ncclSuccess && comm) perf_nccl_init_node_map(*comm);
    return r;
}

ncclResult_t ncclSend(const void *sendbuff, size_t count, ncclDataType_t datatype, int peer, ncclComm_t comm,
                      cudaStream_t stream) {
    PERF_NCCL_REAL(ncclSend);
    void *tok = perf_nccl_dev_begin(stream);
    const double t0 = perf_get_time();
    ncclResult_t r = real_ncclSend(sendbuff, count, datatype, peer, comm, stream);
    perf_attr_t a[] = {{"duration", perf_get_time() - t0}, {"msg_bytes", (double)(count * perf_nccl_type_size(datatype))},
                       {"count", (double)count}, {"intra", (double)perf_nccl_is_intra(peer)}};
    perf_nccl_dev_end(tok, stream, "ncclSend", t0, 4, a);
    capture("ncclSend", sendbuff, count * perf_nccl_type_size(datatype));
    return r;
}

ncclResult_t ncclRecv(void *recvbuff, size_t count, ncclDataType_t datatype, int peer, ncclComm_t comm,
                      cudaStream_t stream) {
    PERF_NCCL_REAL(ncclRecv);
    void *tok = perf_nccl_dev_begin(stream);
    const double t0 = perf_get_time();
    ncclResult_t r = real_ncclRecv(recvbuff, count, datatype, peer, comm, stream);
    perf_attr_t a[] = {{"duration", perf_get_time() - t0}, {"msg_bytes", (double)(count * perf_nccl_type_size(datatype))},
                       {"count", (double)count}, {"intra", (double)perf_nccl_is_intra(peer)}};
    perf_nccl_dev_end(tok, stream, "ncclRecv", t0, 4, a);
    return r;
}

#define COLLECTIVE_ROW(NAME, BYTES, BUF)                                                                 \
    perf_attr_t a[] = {{"duration", perf_get_time() - t0}, {"data_bytes", (double)(BYTES)}};             \
    perf_nccl_dev_end(tok, stream, NAME, t0, 2, a);                                                      \
    capture(NAME, BUF, BYTES)

ncclResult_t ncclAllReduce(const void *sendbuff, void *recvbuff, size_t count, ncclDataType_t datatype, ncclRedOp_t op,
                           ncclComm_t comm, cudaStream_t stream) {
    PERF_NCCL_REAL(ncclAllReduce);
    void *tok = perf_nccl_dev_begin(stream);
    const double t0 = perf_get_time();
    ncclResult_t r = real_ncclAllReduce(sendbuff, recvbuff, count, datatype, op, comm, stream);
    COLLECTIVE_ROW("ncclAllReduce", count * perf_nccl_type_size(datatype), sendbuff);
    return r;
}

ncclResult_t ncclBroadcast(const void *sendbuff, void *recvbuff, size_t count, ncclDataType_t datatype, int root,
                           ncclComm_t comm, cudaStream_t stream) {
    PERF_NCCL_REAL(ncclBroadcast);
    void *tok = perf_nccl_dev_begin(stream);
    const double t0 = perf_get_time();
    ncclResult_t r = real_ncclBroadcast(sendbuff, recvbuff, count, datatype, root, comm, stream);
    COLLECTIVE_ROW("ncclBroadcast", count * perf_nccl_type_size(datatype), sendbuff);
    return r;
}

ncclResult_t ncclReduce(const void *sendbuff, void *recvbuff, size_t count, ncclDataType_t datatype, ncclRedOp_t op, int root,
                        ncclComm_t comm, cudaStream_t stream) {
    PERF_NCCL_REAL(ncclReduce);
    void *tok = perf_nccl_dev_begin(stream);
    const double t0 = perf_get_time();
    ncclResult_t r = real_ncclReduce(sendbuff, recvbuff, count, datatype, op, root, comm, stream);
    COLLECTIVE_ROW("ncclReduce", count * perf_nccl_type_size(datatype), sendbuff);
    return r;
}

ncclResult_t ncclAllGather(const void *sendbuff, void *recvbuff, size_t sendcount, ncclDataType_t datatype, ncclComm_t comm,
                           cudaStream_t stream) {
    PERF_NCCL_REAL(ncclAllGather);
    void *tok = perf_nccl_dev_begin(stream);
    const double t0 = perf_get_time();
    ncclResult_t r = real_ncclAllGather(sendbuff, recvbuff, sendcount, datatype, comm, stream);
    COLLECTIVE_ROW("ncclAllGather", sendcount * perf_nccl_type_size(datatype), sendbuff);
    return r;
}

ncclResult_t ncclReduceScatter(const void *sendbuff, void *recvbuff, size_t recvcount, ncclDataType_t datatype,
                               ncclRedOp_t op, ncclComm_t comm, cudaStream_t stream) {
    PERF_NCCL_REAL(ncclReduceScatter);
    void *tok = perf_nccl_dev_begin(stream);
    const double t0 = perf_get_time();
    ncclResult_t r = real_ncclReduceScatter(sendbuff, recvbuff, recvcount, datatype, op, comm, stream);
    COLLECTIVE_ROW("ncclReduceScatter", recvcount * perf_nccl_type_size(datatype), sendbuff);
    return r;
}

/* AllToAll extension (returns int, 0 on success). */
int ncclAllToAll(const void *sendbuf, size_t sendcount, ncclDataType_t sendtype, void *recvbuf, size_t recvcount,
                 ncclDataType_t recvtype, ncclComm_t comm, cudaStream_t stream) {
    static __typeof__(&ncclAllToAll) real = NULL;
    if (!real) real = (__typeof__(&ncclAllToAll))perf_nccl_get_real("ncclAllToAll");
    if (!real) return 1;
    void *tok = perf_nccl_dev_begin(stream);
    const double t0 = perf_get_time();
    int r = real(sendbuf, sendcount, sendtype, recvbuf, recvcount, recvtype, comm, stream);
    COLLECTIVE_ROW("ncclAllToAll", sendcount * perf_nccl_type_size(sendtype), sendbuf);
    return r;
}

/* ---- compression hook ABI (COCCL style) ---------------------------------------- */
ncclResult_t ncclCompress(const void *orgbuff, void **compbuff, const size_t orgChunkCount, ncclDataType_t orgDatatype,
                          size_t *compChunkCount, ncclDataType_t *compDatatype, const size_t numChunks, const int rank,
                          ncclCommOp_t commOp, cudaStream_t stream) {
    PERF_NCCL_REAL(ncclCompress);
    void *tok = perf_nccl_dev_begin(stream);
    const double t0 = perf_get_time();
    ncclResult_t r = real_ncclCompress(orgbuff, compbuff, orgChunkCount, orgDatatype, compChunkCount, compDatatype, numChunks,
                                       rank, commOp, stream);
    const double in = (double)(orgChunkCount * numChunks * perf_nccl_type_size(orgDatatype));
    const double out = compChunkCount ? (double)(*compChunkCount * numChunks) : 0.0;
    perf_attr_t a[] = {{"duration", perf_get_time() - t0}, {"input_size", in}, {"output_size", out},
                       {"compression_ratio", in > 0 ? out / in : 0.0}};
    perf_nccl_dev_end(tok, stream, "ncclCompress", t0, 4, a);
    return r;
}

ncclResult_t ncclDecompress(void *decompbuff, const void *compbuff, const size_t decompChunkCount,
                            ncclDataType_t decompDatatype, const size_t compChunkCount, ncclDataType_t compDatatype,
                            const size_t numChunks, ncclCommOp_t commOp, cudaStream_t stream) {
    PERF_NCCL_REAL(ncclDecompress);
    void *tok = perf_nccl_dev_begin(stream);
    const double t0 = perf_get_time();
    ncclResult_t r = real_ncclDecompress(decompbuff, compbuff, decompChunkCount, decompDatatype, compChunkCount, compDatatype,
                                         numChunks, commOp, stream);
    perf_attr_t a[] = {{"duration", perf_get_time() - t0}, {"input_size", (double)(compChunkCount * numChunks)},
                       {"output_size", (double)(decompChunkCount * numChunks * perf_nccl_type_size(decompDatatype))}};
    perf_nccl_dev_end(tok, stream, "ncclDecompress", t0, 3, a);
    return r;
}

ncclResult_t ncclDecompressReduce(void *reducebuff, const void *compbuff, const size_t compChunkCount,
                                  ncclDataType_t compDatatype, const size_t reduceChunkCount, ncclDataType_t reduceDataType,
                                  const size_t numChunks, ncclCommOp_t commOp, cudaStream_t stream) {
    PERF_NCCL_REAL(ncclDecompressReduce);
    void *tok = perf_nccl_dev_begin(stream);
    const double t0 = perf_get_time();
    ncclResult_t r = real_ncclDecompressReduce(reducebuff, compbuff, compChunkCount, compDatatype, reduceChunkCount,
                                               reduceDataType, numChunks, commOp, stream);
    perf_attr_t a[] = {{"duration", perf_get_time() - t0}, {"input_size", (double)(compChunkCount * numChunks)},
                       {"output_size", (double)(reduceChunkCount * numChunks * perf_nccl_type_size(reduceDataType))}};
    perf_nccl_dev_end(tok, stream, "ncclDecompressReduce", t0, 3, a);
    return r;
}

ncclResult_t ncclDecompReduceComp(const void *compbuff, void **recompbuff, const size_t orgChunkCount,
                                  ncclDataType_t orgDatatype, const size_t compChunkCount, ncclDataType_t compDatatype,
                                  size_t *reCompChunkCount, ncclDataType_t *reCompDatatype, const size_t numChunks,
                                  ncclCommOp_t commOp, cudaStream_t stream) {
    PERF_NCCL_REAL(ncclDecompReduceComp);
    void *tok = perf_nccl_dev_begin(stream);
    const double t0 = perf_get_time();
    ncclResult_t r = real_ncclDecompReduceComp(compbuff, recompbuff, orgChunkCount, orgDatatype, compChunkCount, compDatatype,
                                               reCompChunkCount, reCompDatatype, numChunks, commOp, stream);
    perf_attr_t a[] = {{"duration", perf_get_time() - t0}, {"input_size", (double)(compChunkCount * numChunks)},
                       {"output_size", reCompChunkCount ? (double)*reCompChunkCount : 0.0}};
    perf_nccl_dev_end(tok, stream, "ncclDecompReduceComp", t0, 3, a);
    return r;
}

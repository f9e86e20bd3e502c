/* Starting point for your own NCCL communication wrapper (communication wrapper mode 3:
 * "build from source", see userconfig/config_in_jsonc/communication_lib_selection.jsonc).
 *
 * The library is put in LD_PRELOAD in front of libnccl, so every ncclXxx symbol defined
 * here is called instead of NCCL's; the real one is found with dlsym(RTLD_NEXT). Each
 * hook below forwards unchanged: replace the body between the markers with your
 * algorithm (for instance: compress with ncclCompress from the selected compression
 * wrapper, move the bytes with the real ncclSend/ncclRecv, decompress). Same role as
 * the reference's userconfig/your_wrapper_code/communication/user_wrapper_nccl/
 * user_wrapper_nccl.c:53-190, which hooks the same five collectives.
 *
 * Build:  python3 -m ccbench_b200.cli build-wrappers   (or scripts/build_script.sh)  */
#define _GNU_SOURCE
#include <cuda_runtime.h>
#include <dlfcn.h>
#include <nccl.h>
#include <stdio.h>
#include <stdlib.h>

static int verbose(void) {
    static int v = -1;
    if (v < 0) v = getenv("USER_WRAPPER_VERBOSE") ? atoi(getenv("USER_WRAPPER_VERBOSE")) : 0;
    return v;
}

/* real(name): the next definition of `name` in library search order, resolved once */
#define REAL(name)                                                             \
    static __typeof__(&name) real_fn = NULL;                                   \
    if (!real_fn) real_fn = (__typeof__(&name))dlsym(RTLD_NEXT, #name);        \
    if (!real_fn) {                                                            \
        fprintf(stderr, "[user_wrapper_nccl] %s not found behind this wrapper\n", #name); \
        return ncclSystemError;                                                \
    }                                                                          \
    if (verbose()) fprintf(stderr, "[user_wrapper_nccl] %s count=%zu\n", #name, (size_t)count)

ncclResult_t ncclAllReduce(const void *sendbuff, void *recvbuff, size_t count, ncclDataType_t datatype, ncclRedOp_t op,
                           ncclComm_t comm, cudaStream_t stream) {
    REAL(ncclAllReduce);
    /* ---- your AllReduce starts here ---- */
    return real_fn(sendbuff, recvbuff, count, datatype, op, comm, stream);
    /* ---- and ends here ---- */
}

ncclResult_t ncclReduce(const void *sendbuff, void *recvbuff, size_t count, ncclDataType_t datatype, ncclRedOp_t op, int root,
                        ncclComm_t comm, cudaStream_t stream) {
    REAL(ncclReduce);
    return real_fn(sendbuff, recvbuff, count, datatype, op, root, comm, stream);
}

ncclResult_t ncclBroadcast(const void *sendbuff, void *recvbuff, size_t count, ncclDataType_t datatype, int root, ncclComm_t comm,
                           cudaStream_t stream) {
    REAL(ncclBroadcast);
    return real_fn(sendbuff, recvbuff, count, datatype, root, comm, stream);
}

/* the in-place legacy form some applications still call */
ncclResult_t ncclBcast(void *buff, size_t count, ncclDataType_t datatype, int root, ncclComm_t comm, cudaStream_t stream) {
    REAL(ncclBcast);
    return real_fn(buff, count, datatype, root, comm, stream);
}

ncclResult_t ncclAllGather(const void *sendbuff, void *recvbuff, size_t sendcount, ncclDataType_t datatype, ncclComm_t comm,
                           cudaStream_t stream) {
    const size_t count = sendcount;
    REAL(ncclAllGather);
    return real_fn(sendbuff, recvbuff, sendcount, datatype, comm, stream);
}

ncclResult_t ncclReduceScatter(const void *sendbuff, void *recvbuff, size_t recvcount, ncclDataType_t datatype, ncclRedOp_t op,
                               ncclComm_t comm, cudaStream_t stream) {
    const size_t count = recvcount;
    REAL(ncclReduceScatter);
    return real_fn(sendbuff, recvbuff, recvcount, datatype, op, comm, stream);
}

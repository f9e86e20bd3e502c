/* Starting point for a wrapper that sends one NCCL collective through the fused
 * compressed kernels of libccb.so and leaves the rest to NCCL. No counterpart in the
 * reference: its templates only forward (user_wrapper_nccl.c:53-190).
 *
 * What is shown: the three steps a wrapper needs. (1) the first call on a communicator
 * makes the ranks agree on a rendezvous tag, using the real NCCL once; (2) every rank
 * creates its libccb communicator (symmetric arenas over NVLink); (3) AllReduce on fp32 /
 * fp16 / bf16 with a sum goes to ccb_all_reduce, ONE kernel launch that encodes, moves
 * and reduces. Everything else falls through. bin/libs/libccb_nccl.so is the complete
 * version of this idea (all collectives, size threshold, codec choice by environment).
 *
 * Build:  python3 -m ccbench_b200.cli build-wrappers   with, in
 * communication_lib_selection.jsonc: mode 3, source_files = this file,
 * include_dirs = ["include"], libraries = "-Lccbench_b200/_native -lccb".          */
#define _GNU_SOURCE
#include <cuda_runtime.h>
#include <dlfcn.h>
#include <nccl.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include <unistd.h>

#include "ccb/ccb.h"

#define MAX_COMMS 16
static struct { ncclComm_t nccl; ccb_comm *ccb; } g_comms[MAX_COMMS];

static void *next_symbol(const char *name) {
    void *p = dlsym(RTLD_NEXT, name);
    if (!p) fprintf(stderr, "[user_wrapper_ccb] %s not found behind this wrapper\n", name);
    return p;
}

/* steps (1) and (2) */
static ccb_comm *attach(ncclComm_t comm, cudaStream_t stream) {
    for (int i = 0; i < MAX_COMMS; ++i)
        if (g_comms[i].nccl == comm) return g_comms[i].ccb;
    ncclResult_t (*rank_of)(ncclComm_t, int *) = next_symbol("ncclCommUserRank");
    ncclResult_t (*count_of)(ncclComm_t, int *) = next_symbol("ncclCommCount");
    ncclResult_t (*bcast)(const void *, void *, size_t, ncclDataType_t, int, ncclComm_t, cudaStream_t) = next_symbol("ncclBroadcast");
    if (!rank_of || !count_of || !bcast) return NULL;
    int rank = 0, n = 0;
    rank_of(comm, &rank);
    count_of(comm, &n);
    if (n > CCB_MAX_RANKS) return NULL;
    /* rank 0 picks the tag, the real NCCL carries it to the others */
    unsigned long long *d_tag = NULL, tag = ((unsigned long long)getpid() << 20) ^ (unsigned long long)(size_t)comm;
    if (cudaMalloc((void **)&d_tag, sizeof(tag)) != cudaSuccess) return NULL;
    cudaMemcpyAsync(d_tag, &tag, sizeof(tag), cudaMemcpyHostToDevice, stream);
    bcast(d_tag, d_tag, sizeof(tag), ncclUint8, 0, comm, stream);
    cudaMemcpyAsync(&tag, d_tag, sizeof(tag), cudaMemcpyDeviceToHost, stream);
    cudaStreamSynchronize(stream);
    cudaFree(d_tag);
    char name[64];
    snprintf(name, sizeof(name), "uw%llx", tag);
    ccb_comm *c = NULL;
    if (ccb_comm_create(&c, rank, n, name, 0, 0) != CCB_OK) {
        fprintf(stderr, "[user_wrapper_ccb] %s\n", ccb_last_error());
        return NULL;
    }
    for (int i = 0; i < MAX_COMMS; ++i)
        if (!g_comms[i].nccl) {
            g_comms[i].nccl = comm;
            g_comms[i].ccb = c;
            break;
        }
    return c;
}

/* step (3) */
ncclResult_t ncclAllReduce(const void *sendbuff, void *recvbuff, size_t count, ncclDataType_t datatype, ncclRedOp_t op,
                           ncclComm_t comm, cudaStream_t stream) {
    static ncclResult_t (*real_fn)(const void *, void *, size_t, ncclDataType_t, ncclRedOp_t, ncclComm_t, cudaStream_t) = NULL;
    if (!real_fn) real_fn = next_symbol("ncclAllReduce");
    const int dt = datatype == ncclFloat32 ? CCB_F32 : datatype == ncclFloat16 ? CCB_F16 : (int)datatype == 9 ? CCB_BF16 : -1;
    ccb_comm *c = (dt >= 0 && op == ncclSum) ? attach(comm, stream) : NULL;
    if (c) {
        /* ---- your choice of codec and algorithm goes here ---- */
        const void *send[1] = {sendbuff};
        void *recv[1] = {recvbuff};
        if (ccb_all_reduce(c, send, recv, count, dt, CCB_OP_SUM, CCB_CODEC_INT8, CCB_ALGO_AUTO, NULL, stream) == CCB_OK) return ncclSuccess;
        fprintf(stderr, "[user_wrapper_ccb] %s; falling back to NCCL\n", ccb_last_error());
    }
    return real_fn ? real_fn(sendbuff, recvbuff, count, datatype, op, comm, stream) : ncclSystemError;
}

ncclResult_t ncclCommDestroy(ncclComm_t comm) {
    static ncclResult_t (*real_fn)(ncclComm_t) = NULL;
    if (!real_fn) real_fn = next_symbol("ncclCommDestroy");
    for (int i = 0; i < MAX_COMMS; ++i)
        if (g_comms[i].nccl == comm) {
            ccb_comm_destroy(g_comms[i].ccb);
            memset(&g_comms[i], 0, sizeof(g_comms[i]));
        }
    return real_fn ? real_fn(comm) : ncclSystemError;
}

/* NCCL's API served by libccb.so alone: no libnccl underneath.
 *
 * The reference ships a wrapper that replaces NCCL outright with another transport
 * (userconfig/wrapper_code_examples/communication/nccl_via_uccl/nccl_via_uccl.cu: its own
 * ncclGetUniqueId :377, ncclCommInitRank :390, ncclSend/ncclRecv :751-790 over an RDMA
 * engine, collectives written as rings of sends and receives :802-1215, group calls that
 * only count :1239-1247). This is the same role for one NVSwitch node: preload
 * libccb_nccl_standalone.so and every nccl* call of the program lands here.
 *
 *   rendezvous     ncclGetUniqueId draws 16 random bytes; ncclCommInitRank turns them into the
 *                  rendezvous tag of ccb_comm_create (abstract Unix sockets, peer arenas).
 *   collectives    float / half / bfloat16 go to the fused sm_100a kernels (codec from
 *                  $CCB_CODEC, default none = exact). Other element types: data movement is
 *                  done in bytes; reductions gather the ranks' buffers over the
 *                  point-to-point kernel and fold them locally (ccb_fold).
 *   send / recv    the peer-arena mailbox kernel (ccb_p2p): the operations of one
 *                  ncclGroupStart/End are launched together, so a rank sends and receives
 *                  at the same time. Send and receive to oneself are paired by a copy.
 *
 * Limits, stated rather than hidden: at most 8 ranks, all on one host, one rank per process;
 * ncclCommInitAll, ncclCommSplit, user-defined reduction operators and CUDA-graph capture of
 * the calls are not provided (the entry points that exist return ncclInvalidUsage). */
#include <cuda_runtime.h>
#include <nccl.h>
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include <strings.h>
#include <unistd.h>

#include "ccb/ccb.h"

#define SA_MAGIC 0x63636273u /* "ccbs" */
#define SA_MAX_GROUP 256

struct ncclComm {
    uint32_t magic;
    ccb_comm *c;
    int rank, n, dev;
    ncclResult_t async_err;
};

static __thread char t_err[256];
static void sa_error(const char *what) { snprintf(t_err, sizeof(t_err), "%s: %s", what, ccb_last_error()); }

static ncclResult_t to_nccl(int rc) {
    switch (rc) {
        case CCB_OK: return ncclSuccess;
        case CCB_ERR_ARG: return ncclInvalidArgument;
        case CCB_ERR_CUDA: return ncclUnhandledCudaError;
        case CCB_ERR_TIMEOUT: return ncclRemoteError;
        case CCB_ERR_BOOTSTRAP: return ncclSystemError;
        default: return ncclInternalError;
    }
}
static size_t type_bytes(ncclDataType_t t) {
    switch ((int)t) {
        case ncclInt8: case ncclUint8: return 1;
        case ncclFloat16: case 9 /* ncclBfloat16 */: return 2;
        case ncclInt32: case ncclUint32: case ncclFloat32: return 4;
        case ncclInt64: case ncclUint64: case ncclFloat64: return 8;
        case 10: case 11: /* 8-bit floats: moved, never reduced */ return 1;
        default: return 0;
    }
}
static int fused_dtype(ncclDataType_t t) {
    if (t == ncclFloat32) return CCB_F32;
    if (t == ncclFloat16) return CCB_F16;
    if ((int)t == 9) return CCB_BF16;
    return -1;
}
static int fold_type(ncclDataType_t t) {
    switch ((int)t) {
        case ncclInt8: return CCB_X_I8;
        case ncclUint8: return CCB_X_U8;
        case ncclInt32: return CCB_X_I32;
        case ncclUint32: return CCB_X_U32;
        case ncclInt64: return CCB_X_I64;
        case ncclUint64: return CCB_X_U64;
        case ncclFloat64: return CCB_X_F64;
        default: return -1;
    }
}
static int codec_from_env(const char *name) {
    const char *e = getenv(name);
    if (!e || !*e || !strcasecmp(e, "none")) return CCB_CODEC_NONE;
    if (!strcasecmp(e, "int8")) return CCB_CODEC_INT8;
    if (!strcasecmp(e, "int8_g256")) return CCB_CODEC_INT8_G256;
    if (!strcasecmp(e, "fp8")) return CCB_CODEC_FP8;
    if (!strcasecmp(e, "int4")) return CCB_CODEC_INT4;
    return CCB_CODEC_NONE;
}
static int valid(ncclComm_t c) { return c && c->magic == SA_MAGIC && c->c; }

/* ------------------------------------------------------------ communicators --- */
ncclResult_t ncclGetVersion(int *version) {
    if (!version) return ncclInvalidArgument;
    *version = NCCL_VERSION_CODE;
    return ncclSuccess;
}

ncclResult_t ncclGetUniqueId(ncclUniqueId *id) {
    if (!id) return ncclInvalidArgument;
    memset(id, 0, sizeof(*id));
    uint64_t r[2] = {(uint64_t)getpid() * 0x9E3779B97F4A7C15ull, (uint64_t)(uintptr_t)id};
    FILE *u = fopen("/dev/urandom", "rb");
    if (u) {
        if (fread(r, 1, sizeof(r), u) != sizeof(r)) r[0] ^= 1;
        fclose(u);
    }
    memcpy(id->internal, "ccbs", 4);
    memcpy(id->internal + 8, r, sizeof(r));
    return ncclSuccess;
}

static ncclResult_t init_rank(ncclComm_t *out, int nranks, const ncclUniqueId *id, int rank) {
    if (!out || nranks < 1 || rank < 0 || rank >= nranks) return ncclInvalidArgument;
    if (memcmp(id->internal, "ccbs", 4) != 0) {
        snprintf(t_err, sizeof(t_err), "the unique id was not made by this library's ncclGetUniqueId");
        return ncclInvalidArgument;
    }
    if (nranks > CCB_MAX_RANKS) {
        snprintf(t_err, sizeof(t_err), "%d ranks: this provider serves one NVSwitch node of at most %d GPUs", nranks, CCB_MAX_RANKS);
        return ncclInvalidUsage;
    }
    char tag[40] = "s";
    for (int i = 0; i < 16; ++i) snprintf(tag + 1 + 2 * i, 3, "%02x", (unsigned char)id->internal[8 + i]);
    struct ncclComm *c = (struct ncclComm *)calloc(1, sizeof(*c));
    if (!c) return ncclSystemError;
    c->rank = rank;
    c->n = nranks;
    cudaGetDevice(&c->dev);
    int rc = ccb_comm_create(&c->c, rank, nranks, tag, 0, getenv("CCB_NVLS") ? 1 : 0);
    if (rc != CCB_OK) {
        sa_error("ncclCommInitRank");
        free(c);
        return to_nccl(rc);
    }
    c->magic = SA_MAGIC;
    *out = c;
    if (getenv("CCB_VERBOSE"))
        fprintf(stderr, "[ccb_nccl_standalone] rank %d/%d ready: every nccl call of this process is served without libnccl\n", rank, nranks);
    return ncclSuccess;
}
ncclResult_t ncclCommInitRank(ncclComm_t *comm, int nranks, ncclUniqueId id, int rank) { return init_rank(comm, nranks, &id, rank); }
ncclResult_t ncclCommInitRankConfig(ncclComm_t *comm, int nranks, ncclUniqueId id, int rank, ncclConfig_t *config) {
    (void)config;
    return init_rank(comm, nranks, &id, rank);
}

/* One process driving several GPUs is not served: the kernels of a communicator are
 * launched on the device that is current, one rank per process. */
ncclResult_t ncclCommInitAll(ncclComm_t *comms, int ndev, const int *devlist) {
    (void)comms; (void)devlist;
    snprintf(t_err, sizeof(t_err), "ncclCommInitAll(%d devices): this provider runs one rank per process", ndev);
    return ncclInvalidUsage;
}

ncclResult_t ncclCommFinalize(ncclComm_t comm) { return valid(comm) ? ncclSuccess : ncclInvalidArgument; }
ncclResult_t ncclCommDestroy(ncclComm_t comm) {
    if (!comm) return ncclSuccess;
    if (comm->magic != SA_MAGIC) return ncclInvalidArgument;
    int before = 0;
    cudaGetDevice(&before);
    cudaSetDevice(comm->dev);
    if (comm->c) ccb_comm_destroy(comm->c);
    cudaSetDevice(before);
    comm->magic = 0;
    free(comm);
    return ncclSuccess;
}
ncclResult_t ncclCommAbort(ncclComm_t comm) { return ncclCommDestroy(comm); }
ncclResult_t ncclCommCount(const ncclComm_t comm, int *count) {
    if (!valid(comm) || !count) return ncclInvalidArgument;
    *count = comm->n;
    return ncclSuccess;
}
ncclResult_t ncclCommUserRank(const ncclComm_t comm, int *rank) {
    if (!valid(comm) || !rank) return ncclInvalidArgument;
    *rank = comm->rank;
    return ncclSuccess;
}
ncclResult_t ncclCommCuDevice(const ncclComm_t comm, int *device) {
    if (!valid(comm) || !device) return ncclInvalidArgument;
    *device = comm->dev;
    return ncclSuccess;
}
/* A device-side wait that ran out is reported here: the status words of the communicator
 * are read without synchronising the device. */
ncclResult_t ncclCommGetAsyncError(ncclComm_t comm, ncclResult_t *asyncError) {
    if (!valid(comm) || !asyncError) return ncclInvalidArgument;
    uint32_t w[8] = {0};
    if (comm->async_err == ncclSuccess && ccb_comm_status(comm->c, w) == CCB_OK && w[0] != 0) comm->async_err = ncclRemoteError;
    *asyncError = comm->async_err;
    return ncclSuccess;
}
ncclResult_t ncclCommSplit(ncclComm_t comm, int color, int key, ncclComm_t *newcomm, ncclConfig_t *config) {
    (void)comm; (void)color; (void)key; (void)newcomm; (void)config;
    snprintf(t_err, sizeof(t_err), "ncclCommSplit is not provided: make the sub-communicator with its own ncclGetUniqueId");
    return ncclInvalidUsage;
}
const char *ncclGetErrorString(ncclResult_t r) {
    switch (r) {
        case ncclSuccess: return "no error";
        case ncclUnhandledCudaError: return "unhandled cuda error";
        case ncclSystemError: return "unhandled system error";
        case ncclInternalError: return "internal error";
        case ncclInvalidArgument: return "invalid argument";
        case ncclInvalidUsage: return "invalid usage";
        case ncclRemoteError: return "remote process exited or a device-side wait ran out";
        case ncclInProgress: return "in progress";
        default: return "unknown result code";
    }
}
const char *ncclGetLastError(ncclComm_t comm) {
    (void)comm;
    return t_err[0] ? t_err : ccb_last_error();
}

/* ------------------------------------------------------------ point to point --- */
typedef struct {
    ncclComm_t comm;
    ccb_p2p_op op;
    cudaStream_t stream;
} group_op;
static __thread int t_depth;
static __thread int t_nops;
static __thread group_op t_ops[SA_MAX_GROUP];

/* Launches what the group holds: per communicator, the operations in issue order. */
static ncclResult_t flush_group(void) {
    ncclResult_t result = ncclSuccess;
    const int n = t_nops;
    t_nops = 0;
    char done[SA_MAX_GROUP];
    memset(done, 0, sizeof(done));
    int before = 0;
    cudaGetDevice(&before);
    for (int i = 0; i < n; ++i) {
        if (done[i]) continue;
        ncclComm_t comm = t_ops[i].comm;
        cudaStream_t stream = t_ops[i].stream;
        ccb_p2p_op batch[SA_MAX_GROUP];
        int k = 0;
        /* sends and receives to oneself pair up in order and become copies */
        int self_send[SA_MAX_GROUP], self_recv[SA_MAX_GROUP], ns = 0, nr = 0;
        for (int j = i; j < n; ++j) {
            if (done[j] || t_ops[j].comm != comm) continue;
            done[j] = 1;
            if (t_ops[j].op.peer == comm->rank) {
                if (t_ops[j].op.is_recv) self_recv[nr++] = j; else self_send[ns++] = j;
            } else {
                batch[k++] = t_ops[j].op;
            }
        }
        cudaSetDevice(comm->dev);
        if (ns != nr) {
            snprintf(t_err, sizeof(t_err), "%d sends to oneself but %d receives from oneself in one group", ns, nr);
            result = ncclInvalidUsage;
        }
        for (int s = 0; s < ns && s < nr; ++s) {
            const ccb_p2p_op *a = &t_ops[self_send[s]].op, *b = &t_ops[self_recv[s]].op;
            if (a->bytes != b->bytes) {
                snprintf(t_err, sizeof(t_err), "send to oneself of %llu bytes meets a receive of %llu", (unsigned long long)a->bytes,
                         (unsigned long long)b->bytes);
                result = ncclInvalidArgument;
            } else if (a->buf != b->buf && a->bytes &&
                       cudaMemcpyAsync(b->buf, a->buf, a->bytes, cudaMemcpyDeviceToDevice, stream) != cudaSuccess) {
                result = ncclUnhandledCudaError;
            }
        }
        if (k > 0) {
            int rc = ccb_p2p(comm->c, batch, k, stream);
            if (rc != CCB_OK) {
                sa_error("send/recv");
                result = to_nccl(rc);
            }
        }
    }
    cudaSetDevice(before);
    return result;
}

static ncclResult_t enqueue(ncclComm_t comm, void *buf, size_t count, ncclDataType_t dt, int peer, int is_recv, cudaStream_t stream) {
    const size_t tb = type_bytes(dt);
    if (!valid(comm) || tb == 0 || peer < 0 || peer >= comm->n) return ncclInvalidArgument;
    if (t_nops >= SA_MAX_GROUP) {
        snprintf(t_err, sizeof(t_err), "more than %d sends and receives in one group", SA_MAX_GROUP);
        return ncclInvalidUsage;
    }
    group_op *g = &t_ops[t_nops++];
    g->comm = comm;
    g->op.buf = buf;
    g->op.bytes = count * tb;
    g->op.peer = peer;
    g->op.is_recv = is_recv;
    g->stream = stream;
    return t_depth > 0 ? ncclSuccess : flush_group();
}
ncclResult_t ncclSend(const void *sendbuff, size_t count, ncclDataType_t datatype, int peer, ncclComm_t comm, cudaStream_t stream) {
    return enqueue(comm, (void *)sendbuff, count, datatype, peer, 0, stream);
}
ncclResult_t ncclRecv(void *recvbuff, size_t count, ncclDataType_t datatype, int peer, ncclComm_t comm, cudaStream_t stream) {
    return enqueue(comm, recvbuff, count, datatype, peer, 1, stream);
}
ncclResult_t ncclGroupStart(void) {
    ++t_depth;
    return ncclSuccess;
}
ncclResult_t ncclGroupEnd(void) {
    if (t_depth <= 0) return ncclInvalidUsage;
    if (--t_depth > 0) return ncclSuccess;
    return flush_group();
}

/* Byte exchange over the mailbox kernel: cnt[p] bytes from send + soff[p] to peer p, and
 * rcnt[p] bytes from peer p into recv + roff[p]; the own part is copied. One launch. */
static ncclResult_t byte_exchange(ncclComm_t comm, const char *send, const size_t *scnt, const size_t *soff, char *recv,
                                  const size_t *rcnt, const size_t *roff, cudaStream_t stream) {
    ccb_p2p_op ops[2 * CCB_MAX_RANKS];
    int k = 0;
    const int me = comm->rank;
    for (int d = 1; d < comm->n; ++d) { /* the same pairing order on every rank */
        const int to = (me + d) % comm->n, from = (me - d + comm->n) % comm->n;
        if (scnt[to]) ops[k++] = (ccb_p2p_op){(void *)(send + soff[to]), scnt[to], to, 0};
        if (rcnt[from]) ops[k++] = (ccb_p2p_op){recv + roff[from], rcnt[from], from, 1};
    }
    if (scnt[me] && send + soff[me] != recv + roff[me] &&
        cudaMemcpyAsync(recv + roff[me], send + soff[me], scnt[me], cudaMemcpyDeviceToDevice, stream) != cudaSuccess)
        return ncclUnhandledCudaError;
    if (k == 0) return ncclSuccess;
    int rc = ccb_p2p(comm->c, ops, k, stream);
    if (rc != CCB_OK) sa_error("exchange");
    return to_nccl(rc);
}

/* ------------------------------------------------------------ collectives --- */
/* Movement collectives see their payload as the widest element the byte count allows. */
static int move_dtype(size_t bytes_per_block, size_t *count) {
    if (bytes_per_block % 4 == 0) {
        *count = bytes_per_block / 4;
        return CCB_F32;
    }
    if (bytes_per_block % 2 == 0) {
        *count = bytes_per_block / 2;
        return CCB_F16;
    }
    return -1;
}
static int move_codec(ncclDataType_t t) { return fused_dtype(t) >= 0 ? codec_from_env("CCB_MOVE_CODEC") : CCB_CODEC_NONE; }
static int fused_failed(int rc) { return rc == CCB_ERR_UNSUPPORTED || rc == CCB_ERR_CAPACITY; }

ncclResult_t ncclAllGather(const void *sendbuff, void *recvbuff, size_t sendcount, ncclDataType_t datatype, ncclComm_t comm,
                           cudaStream_t stream) {
    const size_t tb = type_bytes(datatype), bytes = sendcount * tb;
    if (!valid(comm) || tb == 0) return ncclInvalidArgument;
    if (bytes == 0) return ncclSuccess;
    const int codec = move_codec(datatype);
    size_t cnt = sendcount;
    const int dt = codec != CCB_CODEC_NONE ? fused_dtype(datatype) : move_dtype(bytes, &cnt);
    if (dt >= 0 && comm->n > 1) {
        const void *s[1] = {sendbuff};
        void *r[1] = {recvbuff};
        int rc = ccb_all_gather(comm->c, s, r, cnt, dt, codec, stream);
        if (!fused_failed(rc)) {
            if (rc != CCB_OK) sa_error("ncclAllGather");
            return to_nccl(rc);
        }
    }
    size_t scnt[CCB_MAX_RANKS], soff[CCB_MAX_RANKS], roff[CCB_MAX_RANKS];
    for (int p = 0; p < comm->n; ++p) scnt[p] = bytes, soff[p] = 0, roff[p] = (size_t)p * bytes;
    return byte_exchange(comm, (const char *)sendbuff, scnt, soff, (char *)recvbuff, scnt, roff, stream);
}

/* The extension collectives keep the signatures of the reference's extension library
 * (send and receive sides described separately); ncclAlltoAll is NCCL 2.28's own spelling. */
static ncclResult_t all_to_all(const void *sendbuff, void *recvbuff, size_t count, ncclDataType_t datatype, ncclComm_t comm,
                               cudaStream_t stream) {
    const size_t tb = type_bytes(datatype), bytes = count * tb;
    if (!valid(comm) || tb == 0) return ncclInvalidArgument;
    if (bytes == 0) return ncclSuccess;
    const int codec = move_codec(datatype);
    size_t cnt = count;
    const int dt = codec != CCB_CODEC_NONE ? fused_dtype(datatype) : move_dtype(bytes, &cnt);
    if (dt >= 0 && comm->n > 1 && sendbuff != recvbuff) {
        const void *s[1] = {sendbuff};
        void *r[1] = {recvbuff};
        int rc = ccb_all_to_all(comm->c, s, r, cnt, dt, codec, stream);
        if (!fused_failed(rc)) {
            if (rc != CCB_OK) sa_error("ncclAllToAll");
            return to_nccl(rc);
        }
    }
    size_t scnt[CCB_MAX_RANKS], off[CCB_MAX_RANKS];
    for (int p = 0; p < comm->n; ++p) scnt[p] = bytes, off[p] = (size_t)p * bytes;
    return byte_exchange(comm, (const char *)sendbuff, scnt, off, (char *)recvbuff, scnt, off, stream);
}
int ncclAllToAll(const void *sendbuf, size_t sendcount, ncclDataType_t sendtype, void *recvbuf, size_t recvcount,
                 ncclDataType_t recvtype, ncclComm_t comm, cudaStream_t stream) {
    if (sendcount * type_bytes(sendtype) != recvcount * type_bytes(recvtype)) return (int)ncclInvalidArgument;
    return (int)all_to_all(sendbuf, recvbuf, sendcount, sendtype, comm, stream);
}
ncclResult_t ncclAlltoAll(const void *sendbuff, void *recvbuff, size_t count, ncclDataType_t datatype, ncclComm_t comm,
                          cudaStream_t stream) {
    return all_to_all(sendbuff, recvbuff, count, datatype, comm, stream);
}

ncclResult_t ncclBroadcast(const void *sendbuff, void *recvbuff, size_t count, ncclDataType_t datatype, int root, ncclComm_t comm,
                           cudaStream_t stream) {
    const size_t tb = type_bytes(datatype), bytes = count * tb;
    if (!valid(comm) || tb == 0 || root < 0 || root >= comm->n) return ncclInvalidArgument;
    if (bytes == 0) return ncclSuccess;
    const int codec = move_codec(datatype);
    size_t cnt = count;
    const int dt = codec != CCB_CODEC_NONE ? fused_dtype(datatype) : move_dtype(bytes, &cnt);
    if (dt >= 0 && comm->n > 1) {
        const void *s[1] = {sendbuff};
        void *r[1] = {recvbuff};
        int rc = ccb_broadcast(comm->c, s, r, cnt, dt, root, codec, stream);
        if (!fused_failed(rc)) {
            if (rc != CCB_OK) sa_error("ncclBroadcast");
            return to_nccl(rc);
        }
    }
    size_t scnt[CCB_MAX_RANKS] = {0}, rcnt[CCB_MAX_RANKS] = {0}, zero[CCB_MAX_RANKS] = {0};
    if (comm->rank == root)
        for (int p = 0; p < comm->n; ++p) scnt[p] = bytes;
    rcnt[root] = bytes;
    return byte_exchange(comm, (const char *)sendbuff, scnt, zero, (char *)recvbuff, rcnt, zero, stream);
}
ncclResult_t ncclBcast(void *buff, size_t count, ncclDataType_t datatype, int root, ncclComm_t comm, cudaStream_t stream) {
    return ncclBroadcast(buff, buff, count, datatype, root, comm, stream);
}

int ncclScatter(const void *sendbuf, size_t sendcount, ncclDataType_t sendtype, void *recvbuf, size_t recvcount,
                ncclDataType_t recvtype, int root, ncclComm_t comm, cudaStream_t stream) {
    const size_t bytes = recvcount * type_bytes(recvtype);
    if (!valid(comm) || type_bytes(recvtype) == 0 || root < 0 || root >= comm->n) return (int)ncclInvalidArgument;
    if (comm->rank == root && sendcount * type_bytes(sendtype) != bytes) return (int)ncclInvalidArgument;
    if (bytes == 0) return (int)ncclSuccess;
    size_t scnt[CCB_MAX_RANKS] = {0}, soff[CCB_MAX_RANKS] = {0}, rcnt[CCB_MAX_RANKS] = {0}, zero[CCB_MAX_RANKS] = {0};
    if (comm->rank == root)
        for (int p = 0; p < comm->n; ++p) scnt[p] = bytes, soff[p] = (size_t)p * bytes;
    rcnt[root] = bytes;
    return (int)byte_exchange(comm, (const char *)sendbuf, scnt, soff, (char *)recvbuf, rcnt, zero, stream);
}
int ncclGather(const void *sendbuf, size_t sendcount, ncclDataType_t sendtype, void *recvbuf, size_t recvcount,
               ncclDataType_t recvtype, int root, ncclComm_t comm, cudaStream_t stream) {
    const size_t bytes = sendcount * type_bytes(sendtype);
    if (!valid(comm) || type_bytes(sendtype) == 0 || root < 0 || root >= comm->n) return (int)ncclInvalidArgument;
    if (comm->rank == root && recvcount * type_bytes(recvtype) != bytes) return (int)ncclInvalidArgument;
    if (bytes == 0) return (int)ncclSuccess;
    size_t scnt[CCB_MAX_RANKS] = {0}, zero[CCB_MAX_RANKS] = {0}, rcnt[CCB_MAX_RANKS] = {0}, roff[CCB_MAX_RANKS] = {0};
    scnt[root] = bytes;
    if (comm->rank == root)
        for (int p = 0; p < comm->n; ++p) rcnt[p] = bytes, roff[p] = (size_t)p * bytes;
    return (int)byte_exchange(comm, (const char *)sendbuf, scnt, zero, (char *)recvbuf, rcnt, roff, stream);
}

/* Reduction of a type the fused kernels do not carry: bring every rank's piece here, fold.
 * piece_of[p] = byte offset in `send` of what rank p must receive (all-reduce: 0 for all). */
static ncclResult_t gathered_reduce(ncclComm_t comm, const char *send, const size_t *send_off, int everyone_sends_to, void *recv,
                                    size_t count, ncclDataType_t dt, ncclRedOp_t op, cudaStream_t stream) {
    const int xt = fold_type(dt);
    const size_t bytes = count * type_bytes(dt);
    if (xt < 0 || (int)op < 0 || (int)op > 4) {
        snprintf(t_err, sizeof(t_err), "reduction of this element type or with this operator is not provided");
        return ncclInvalidArgument;
    }
    const int receives = everyone_sends_to < 0 || everyone_sends_to == comm->rank;
    char *tmp = NULL;
    if (receives && cudaMallocAsync((void **)&tmp, bytes * comm->n, stream) != cudaSuccess) return ncclUnhandledCudaError;
    size_t scnt[CCB_MAX_RANKS] = {0}, rcnt[CCB_MAX_RANKS] = {0}, roff[CCB_MAX_RANKS] = {0};
    for (int p = 0; p < comm->n; ++p) {
        if (everyone_sends_to < 0 || everyone_sends_to == p) scnt[p] = bytes;
        if (receives) rcnt[p] = bytes, roff[p] = (size_t)p * bytes;
    }
    ncclResult_t r = byte_exchange(comm, send, scnt, send_off, tmp, rcnt, roff, stream);
    if (r == ncclSuccess && receives && ccb_fold(xt, (int)op, tmp, count, comm->n, count, recv, stream) != CCB_OK) {
        sa_error("fold");
        r = ncclInternalError;
    }
    if (tmp) cudaFreeAsync(tmp, stream);
    return r;
}

ncclResult_t ncclAllReduce(const void *sendbuff, void *recvbuff, size_t count, ncclDataType_t datatype, ncclRedOp_t op,
                           ncclComm_t comm, cudaStream_t stream) {
    if (!valid(comm) || type_bytes(datatype) == 0) return ncclInvalidArgument;
    if (count == 0) return ncclSuccess;
    const int dt = fused_dtype(datatype);
    if (dt < 0 || (int)op > 3) {
        size_t zero[CCB_MAX_RANKS] = {0};
        return gathered_reduce(comm, (const char *)sendbuff, zero, -1, recvbuff, count, datatype, op, stream);
    }
    int codec = codec_from_env("CCB_CODEC");
    if (op != ncclSum) codec = CCB_CODEC_NONE;
    /* a message larger than the arena allows is reduced in pieces */
    size_t done = 0, piece = count;
    const size_t tb = type_bytes(datatype);
    while (done < count) {
        const size_t len = count - done < piece ? count - done : piece;
        const void *s[1] = {(const char *)sendbuff + done * tb};
        void *r[1] = {(char *)recvbuff + done * tb};
        int rc = ccb_all_reduce(comm->c, s, r, len, dt, (int)op, codec, CCB_ALGO_AUTO, NULL, stream);
        if (rc == CCB_ERR_CAPACITY && piece > 4096) {
            piece = ((piece / 2) + 4095) & ~(size_t)4095;
            continue;
        }
        if (rc != CCB_OK) {
            sa_error("ncclAllReduce");
            return to_nccl(rc);
        }
        done += len;
    }
    return ncclSuccess;
}

ncclResult_t ncclReduceScatter(const void *sendbuff, void *recvbuff, size_t recvcount, ncclDataType_t datatype, ncclRedOp_t op,
                               ncclComm_t comm, cudaStream_t stream) {
    if (!valid(comm) || type_bytes(datatype) == 0) return ncclInvalidArgument;
    if (recvcount == 0) return ncclSuccess;
    const int dt = fused_dtype(datatype);
    if (dt < 0 || (int)op > 3) {
        size_t soff[CCB_MAX_RANKS];
        for (int p = 0; p < comm->n; ++p) soff[p] = (size_t)p * recvcount * type_bytes(datatype);
        return gathered_reduce(comm, (const char *)sendbuff, soff, -1, recvbuff, recvcount, datatype, op, stream);
    }
    int codec = codec_from_env("CCB_CODEC");
    if (op != ncclSum) codec = CCB_CODEC_NONE;
    const void *s[1] = {sendbuff};
    void *r[1] = {recvbuff};
    int rc = ccb_reduce_scatter(comm->c, s, r, recvcount, dt, (int)op, codec, NULL, stream);
    if (rc != CCB_OK) sa_error("ncclReduceScatter");
    return to_nccl(rc);
}

ncclResult_t ncclReduce(const void *sendbuff, void *recvbuff, size_t count, ncclDataType_t datatype, ncclRedOp_t op, int root,
                        ncclComm_t comm, cudaStream_t stream) {
    if (!valid(comm) || type_bytes(datatype) == 0 || root < 0 || root >= comm->n) return ncclInvalidArgument;
    if (count == 0) return ncclSuccess;
    const int dt = fused_dtype(datatype);
    if (dt < 0 || (int)op > 3) {
        size_t zero[CCB_MAX_RANKS] = {0};
        return gathered_reduce(comm, (const char *)sendbuff, zero, root, recvbuff, count, datatype, op, stream);
    }
    int codec = codec_from_env("CCB_CODEC");
    if (op != ncclSum) codec = CCB_CODEC_NONE;
    const void *s[1] = {sendbuff};
    void *r[1] = {recvbuff};
    int rc = ccb_reduce(comm->c, s, r, count, dt, (int)op, root, codec, stream);
    if (rc != CCB_OK) sa_error("ncclReduce");
    return to_nccl(rc);
}

/* Entry points of NCCL that have no meaning without NCCL's proxy and registration cache. */
ncclResult_t ncclCommRegister(const ncclComm_t comm, void *buff, size_t size, void **handle) {
    (void)comm; (void)buff; (void)size;
    if (handle) *handle = NULL;
    return ncclSuccess; /* every device buffer is reachable by the kernels already */
}
ncclResult_t ncclCommDeregister(const ncclComm_t comm, void *handle) {
    (void)comm; (void)handle;
    return ncclSuccess;
}
ncclResult_t ncclMemAlloc(void **ptr, size_t size) { return cudaMalloc(ptr, size) == cudaSuccess ? ncclSuccess : ncclUnhandledCudaError; }
ncclResult_t ncclMemFree(void *ptr) { return cudaFree(ptr) == cudaSuccess ? ncclSuccess : ncclUnhandledCudaError; }
ncclResult_t ncclRedOpCreatePreMulSum(ncclRedOp_t *op, void *scalar, ncclDataType_t datatype, ncclScalarResidence_t residence,
                                      ncclComm_t comm) {
    (void)op; (void)scalar; (void)datatype; (void)residence; (void)comm;
    snprintf(t_err, sizeof(t_err), "user-defined reduction operators are not provided");
    return ncclInvalidUsage;
}
ncclResult_t ncclRedOpDestroy(ncclRedOp_t op, ncclComm_t comm) {
    (void)op; (void)comm;
    return ncclInvalidUsage;
}

/* Lets a test or a driver tell which library answered. */
const char *ccb_nccl_provider(void) { return "ccb-standalone"; }
unsigned long long ccb_nccl_fused_calls(void) { return (unsigned long long)ccb_launch_count(); }

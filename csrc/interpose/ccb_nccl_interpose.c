/* libccb_nccl.so: LD_PRELOAD interposer that replaces NCCL collectives with the fused
 * codec+collective kernels of libccb.so.
 *
 * The reference's interposer (userconfig/wrapper_code_examples/communication/
 * plain_nccl_compress/plain_nccl_compress.cu) hands the application a fake
 * ncclComm_t that wraps the real one (:368-376, 415-436) and rebuilds each collective
 * from ncclSend/ncclRecv hops. This one keeps the application's real ncclComm_t and
 * holds its own state in a side table keyed by it, so any call it does not handle
 * (other dtypes, ncclAvg, calls inside ncclGroupStart/End, a stream that is being
 * captured, communicators that span hosts) goes to the next library in the preload
 * chain untouched.
 *
 * First use of a communicator: the ranks agree on a rendezvous tag and check that
 * they share a host with one real ncclAllGather, then build the symmetric arenas
 * (ccb_comm_create). Environment:
 *   NCCL_COMPRESS_DISABLE=1      pass everything through (reference variable)
 *   NCCL_COMPRESS_GROUP=128|256  int8 group size (reference variable; default 128)
 *   CCB_CODEC=int8|fp8|none|int8_g256      wire codec of reductions (default int8)
 *   CCB_MOVE_CODEC=...           codec of AllGather/Broadcast/AlltoAll (default = CCB_CODEC)
 *   CCB_ALGO=auto|twoshot|oneshot|ring|tree|nvls
 *   CCB_ERROR_FEEDBACK=1         keep a residual per (communicator, buffer, count)
 *   CCB_P2P_CODEC=int8|fp8|int4  also compress ncclSend / ncclRecv (default: off, plain NCCL).
 *                                The bytes still travel by NCCL point-to-point (pipeline
 *                                traffic stays there); one encode kernel before the send and
 *                                one decode kernel after the receive, stream-ordered, no host
 *                                synchronisation, also inside ncclGroupStart/End.
 *   CCB_NVLS=1                   also map the arenas through an NVLS multicast object (lets the
 *                                large two-shot kernel broadcast its reduced shard in one store)
 *   CCB_MIN_BYTES=N              smaller messages go to NCCL (default 0)
 *   CCB_VERBOSE=1                log decisions to stderr                         */
#define _GNU_SOURCE
#include <cuda_runtime.h>
#include <dlfcn.h>
#include <nccl.h>
#include <pthread.h>
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include <unistd.h>

#include "ccb/ccb.h"

#define MAX_COMMS 64
#define MAX_EF 32

typedef struct {
    ncclComm_t real;
    ccb_comm *c;
    int state; /* 0 = not tried, 1 = ready, -1 = unsupported: always pass through */
    int rank, n;
} comm_slot;

typedef struct {
    ncclComm_t comm;
    const void *buf, *out; /* the call's send and receive buffers: an in-place call and an */
    size_t count;          /* out-of-place call on the same send buffer keep separate residuals */
    int kind;              /* 0 = AllReduce, 1 = ReduceScatter */
    float *resid;
    uint64_t last_use;
} ef_slot;

static comm_slot g_comms[MAX_COMMS];
static ef_slot g_ef[MAX_EF];
static uint64_t g_tick;
static pthread_mutex_t g_lock = PTHREAD_MUTEX_INITIALIZER;
static __thread int g_group_depth;

static struct {
    int inited, disabled, codec, move_codec, algo, ef, verbose, p2p_codec;
    size_t min_bytes;
} cfg;

#define LOGV(...)                                      \
    do {                                               \
        if (cfg.verbose) {                             \
            fprintf(stderr, "[ccb_nccl] " __VA_ARGS__); \
            fputc('\n', stderr);                       \
        }                                              \
    } while (0)

static int codec_by_name(const char *s, int dflt) {
    if (!s || !*s) return dflt;
    if (!strcasecmp(s, "int8")) return CCB_CODEC_INT8;
    if (!strcasecmp(s, "fp8")) return CCB_CODEC_FP8;
    if (!strcasecmp(s, "int4")) return CCB_CODEC_INT4;
    if (!strcasecmp(s, "none")) return CCB_CODEC_NONE;
    if (!strcasecmp(s, "int8_g256")) return CCB_CODEC_INT8_G256;
    return dflt;
}

static void load_cfg(void) {
    if (cfg.inited) return;
    const char *e;
    cfg.verbose = (e = getenv("CCB_VERBOSE")) && *e && *e != '0';
    cfg.disabled = (e = getenv("NCCL_COMPRESS_DISABLE")) && (*e == '1' || *e == 'y' || *e == 'Y');
    int dflt = CCB_CODEC_INT8;
    if ((e = getenv("NCCL_COMPRESS_GROUP")) && atoi(e) == 256) dflt = CCB_CODEC_INT8_G256;
    cfg.codec = codec_by_name(getenv("CCB_CODEC"), dflt);
    cfg.move_codec = codec_by_name(getenv("CCB_MOVE_CODEC"), cfg.codec);
    cfg.algo = CCB_ALGO_AUTO;
    if ((e = getenv("CCB_ALGO"))) {
        if (!strcasecmp(e, "twoshot")) cfg.algo = CCB_ALGO_TWOSHOT;
        else if (!strcasecmp(e, "oneshot")) cfg.algo = CCB_ALGO_ONESHOT;
        else if (!strcasecmp(e, "ring")) cfg.algo = CCB_ALGO_RING;
        else if (!strcasecmp(e, "tree")) cfg.algo = CCB_ALGO_TREE;
        else if (!strcasecmp(e, "nvls")) cfg.algo = CCB_ALGO_NVLS;
    }
    cfg.ef = (e = getenv("CCB_ERROR_FEEDBACK")) && *e == '1';
    cfg.min_bytes = (e = getenv("CCB_MIN_BYTES")) ? (size_t)strtoull(e, NULL, 10) : 0;
    cfg.p2p_codec = codec_by_name(getenv("CCB_P2P_CODEC"), CCB_CODEC_NONE);
    cfg.inited = 1;
    LOGV("config: disabled=%d codec=%d move_codec=%d algo=%d error_feedback=%d min_bytes=%zu", cfg.disabled, cfg.codec,
         cfg.move_codec, cfg.algo, cfg.ef, cfg.min_bytes);
}

/* ------------------------------------------------------- next-in-chain NCCL -- */
#define REAL(name, type)                                                    \
    static type real_##name;                                                \
    static type get_##name(void) {                                          \
        if (!real_##name) real_##name = (type)dlsym(RTLD_NEXT, #name);      \
        return real_##name;                                                 \
    }
typedef ncclResult_t (*fn_allreduce)(const void *, void *, size_t, ncclDataType_t, ncclRedOp_t, ncclComm_t, cudaStream_t);
typedef ncclResult_t (*fn_reducescatter)(const void *, void *, size_t, ncclDataType_t, ncclRedOp_t, ncclComm_t, cudaStream_t);
typedef ncclResult_t (*fn_allgather)(const void *, void *, size_t, ncclDataType_t, ncclComm_t, cudaStream_t);
typedef ncclResult_t (*fn_broadcast)(const void *, void *, size_t, ncclDataType_t, int, ncclComm_t, cudaStream_t);
typedef ncclResult_t (*fn_bcast)(void *, size_t, ncclDataType_t, int, ncclComm_t, cudaStream_t);
typedef ncclResult_t (*fn_reduce)(const void *, void *, size_t, ncclDataType_t, ncclRedOp_t, int, ncclComm_t, cudaStream_t);
typedef ncclResult_t (*fn_commdestroy)(ncclComm_t);
typedef ncclResult_t (*fn_group)(void);
typedef ncclResult_t (*fn_send)(const void *, size_t, ncclDataType_t, int, ncclComm_t, cudaStream_t);
typedef ncclResult_t (*fn_recv)(void *, size_t, ncclDataType_t, int, ncclComm_t, cudaStream_t);
typedef ncclResult_t (*fn_commint)(const ncclComm_t, int *);
typedef int (*fn_ext_a2a)(const void *, size_t, ncclDataType_t, void *, size_t, ncclDataType_t, ncclComm_t, cudaStream_t);
typedef int (*fn_ext_rooted)(const void *, size_t, ncclDataType_t, void *, size_t, ncclDataType_t, int, ncclComm_t, cudaStream_t);
REAL(ncclAllReduce, fn_allreduce)
REAL(ncclReduceScatter, fn_reducescatter)
REAL(ncclAllGather, fn_allgather)
REAL(ncclBroadcast, fn_broadcast)
REAL(ncclBcast, fn_bcast)
REAL(ncclReduce, fn_reduce)
REAL(ncclCommDestroy, fn_commdestroy)
REAL(ncclCommAbort, fn_commdestroy)
REAL(ncclSend, fn_send)
REAL(ncclRecv, fn_recv)
REAL(ncclGroupStart, fn_group)
REAL(ncclGroupEnd, fn_group)
REAL(ncclCommUserRank, fn_commint)
REAL(ncclCommCount, fn_commint)
REAL(ncclCommCuDevice, fn_commint)
REAL(ncclAllToAll, fn_ext_a2a)
REAL(ncclScatter, fn_ext_rooted)
REAL(ncclGather, fn_ext_rooted)

/* ------------------------------------------------------------ comm set-up --- */
static int dtype_of(ncclDataType_t t);
/* bytes of `count` elements, for the CCB_MIN_BYTES test (0 for types the fused path does not take) */
static size_t bytes_of(size_t count, ncclDataType_t t) {
    const int d = dtype_of(t);
    return d < 0 ? 0 : count * (d == CCB_F32 ? 4u : 2u);
}
static int dtype_of(ncclDataType_t t) {
    if (t == ncclFloat32) return CCB_F32;
    if (t == ncclFloat16) return CCB_F16;
    if ((int)t == 9) return CCB_BF16; /* ncclBfloat16 */
    return -1;
}

static int stream_is_capturing(cudaStream_t s) {
    enum cudaStreamCaptureStatus st = cudaStreamCaptureStatusNone;
    if (cudaStreamIsCapturing(s, &st) != cudaSuccess) {
        (void)cudaGetLastError();
        return 0;
    }
    return st != cudaStreamCaptureStatusNone;
}

static comm_slot *slot_of(ncclComm_t comm) {
    for (int i = 0; i < MAX_COMMS; ++i)
        if (g_comms[i].real == comm && g_comms[i].state != 0) return &g_comms[i];
    for (int i = 0; i < MAX_COMMS; ++i)
        if (g_comms[i].real == NULL) {
            g_comms[i].real = comm;
            return &g_comms[i];
        }
    return NULL;
}

/* Agree on a tag and check co-location with one real AllGather of 80 bytes per rank. */
static void setup_comm(comm_slot *s, cudaStream_t stream) {
    s->state = -1;
    if (!get_ncclCommUserRank() || !get_ncclCommCount() || !get_ncclAllGather()) return;
    if (get_ncclCommUserRank()(s->real, &s->rank) != ncclSuccess || get_ncclCommCount()(s->real, &s->n) != ncclSuccess) return;
    if (s->n > CCB_MAX_RANKS) {
        LOGV("communicator of %d ranks exceeds one NVSwitch domain (%d): passing through", s->n, CCB_MAX_RANKS);
        return;
    }
    enum { REC = 80 };
    unsigned char mine[REC], *all = (unsigned char *)malloc((size_t)REC * s->n);
    memset(mine, 0, sizeof(mine));
    if (s->rank == 0) {
        FILE *u = fopen("/dev/urandom", "rb");
        uint64_t r[2] = {(uint64_t)getpid() * 0x9E3779B97F4A7C15ull, (uint64_t)(uintptr_t)s};
        if (u) {
            if (fread(r, 1, sizeof(r), u) != sizeof(r)) r[0] ^= 1;
            fclose(u);
        }
        memcpy(mine, r, 16);
    }
    if (gethostname((char *)mine + 16, 63) != 0) strcpy((char *)mine + 16, "unknown");
    void *d_in = NULL, *d_out = NULL;
    if (cudaMalloc(&d_in, REC) != cudaSuccess || cudaMalloc(&d_out, (size_t)REC * s->n) != cudaSuccess) goto out;
    if (cudaMemcpyAsync(d_in, mine, REC, cudaMemcpyHostToDevice, stream) != cudaSuccess) goto out;
    if (get_ncclAllGather()(d_in, d_out, REC, ncclUint8, s->real, stream) != ncclSuccess) goto out;
    if (cudaMemcpyAsync(all, d_out, (size_t)REC * s->n, cudaMemcpyDeviceToHost, stream) != cudaSuccess) goto out;
    if (cudaStreamSynchronize(stream) != cudaSuccess) goto out;
    for (int r = 0; r < s->n; ++r)
        if (strncmp((char *)all + (size_t)r * REC + 16, (char *)mine + 16, 63) != 0) {
            LOGV("rank %d is on another host: passing through", r);
            goto out;
        }
    {
        char tag[40];
        const unsigned char *t = all; /* rank 0's 16 random bytes */
        for (int i = 0; i < 16; ++i) snprintf(tag + 2 * i, 3, "%02x", t[i]);
        int want_nvls = cfg.algo == CCB_ALGO_NVLS || getenv("CCB_NVLS") != NULL;
        int rc = ccb_comm_create(&s->c, s->rank, s->n, tag, 0, want_nvls ? 1 : 0);
        if (rc != CCB_OK) {
            fprintf(stderr, "[ccb_nccl] rank %d: fused path unavailable (%s); using NCCL\n", s->rank, ccb_last_error());
            s->c = NULL;
            goto out;
        }
        s->state = 1;
        LOGV("rank %d/%d: fused path ready (arena %llu MiB, nvls %d)", s->rank, s->n,
             (unsigned long long)(ccb_comm_arena_bytes(s->c) >> 20), ccb_comm_has_nvls(s->c));
    }
out:
    if (d_in) cudaFree(d_in);
    if (d_out) cudaFree(d_out);
    free(all);
    (void)cudaGetLastError();
}

/* Returns the ccb communicator to use for this call, or NULL to pass through. */
static ccb_comm *fused_comm(ncclComm_t comm, ncclDataType_t dt, size_t bytes, cudaStream_t stream, int *rank, int *n) {
    load_cfg();
    if (cfg.disabled || g_group_depth > 0 || dtype_of(dt) < 0 || bytes < cfg.min_bytes) return NULL;
    if (stream_is_capturing(stream)) return NULL;
    pthread_mutex_lock(&g_lock);
    comm_slot *s = slot_of(comm);
    if (s && s->state == 0) setup_comm(s, stream);
    ccb_comm *c = (s && s->state == 1) ? s->c : NULL;
    if (c && rank) *rank = s->rank;
    if (c && n) *n = s->n;
    pthread_mutex_unlock(&g_lock);
    return c;
}

static float *ef_buffer(ncclComm_t comm, const void *buf, const void *out, size_t count, int kind) {
    if (!cfg.ef) return NULL;
    pthread_mutex_lock(&g_lock);
    ef_slot *hit = NULL, *victim = &g_ef[0];
    for (int i = 0; i < MAX_EF; ++i) {
        if (g_ef[i].resid && g_ef[i].comm == comm && g_ef[i].buf == buf && g_ef[i].out == out && g_ef[i].count == count &&
            g_ef[i].kind == kind)
            hit = &g_ef[i];
        if (g_ef[i].last_use < victim->last_use) victim = &g_ef[i];
    }
    if (!hit) {
        if (victim->resid) cudaFree(victim->resid);
        memset(victim, 0, sizeof(*victim));
        if (cudaMalloc((void **)&victim->resid, count * sizeof(float)) == cudaSuccess &&
            cudaMemset(victim->resid, 0, count * sizeof(float)) == cudaSuccess) {
            victim->comm = comm;
            victim->buf = buf;
            victim->out = out;
            victim->kind = kind;
            victim->count = count;
            hit = victim;
        } else {
            (void)cudaGetLastError();
            victim->resid = NULL;
        }
    }
    if (hit) hit->last_use = ++g_tick;
    pthread_mutex_unlock(&g_lock);
    return hit ? hit->resid : NULL;
}

static ncclResult_t to_nccl(int rc) {
    switch (rc) {
        case CCB_OK: return ncclSuccess;
        case CCB_ERR_ARG: return ncclInvalidArgument;
        case CCB_ERR_CUDA: return ncclUnhandledCudaError;
        case CCB_ERR_TIMEOUT: return ncclRemoteError;
        default: return ncclInternalError;
    }
}
static int lossy_ok(int codec, ncclRedOp_t op) { return codec == CCB_CODEC_NONE ? ((int)op <= 3) : (op == ncclSum); }

/* ---------------------------------------------------------------- exports --- */
ncclResult_t ncclAllReduce(const void *sendbuff, void *recvbuff, size_t count, ncclDataType_t datatype, ncclRedOp_t op,
                           ncclComm_t comm, cudaStream_t stream) {
    load_cfg();
    ccb_comm *c = lossy_ok(cfg.codec, op) ? fused_comm(comm, datatype, bytes_of(count, datatype), stream, NULL, NULL) : NULL;
    if (c) {
        float *ef = cfg.codec != CCB_CODEC_NONE ? ef_buffer(comm, sendbuff, recvbuff, count, 0) : NULL;
        const void *s[1] = {sendbuff};
        void *r[1] = {recvbuff};
        float *e[1] = {ef};
        int algo = cfg.algo;
        if (algo == CCB_ALGO_NVLS && (cfg.codec != CCB_CODEC_NONE || !ccb_comm_has_nvls(c))) algo = CCB_ALGO_AUTO;
        int rc = ccb_all_reduce(c, s, r, count, dtype_of(datatype), (int)op, cfg.codec, algo, ef ? e : NULL, stream);
        if (rc != CCB_ERR_UNSUPPORTED && rc != CCB_ERR_CAPACITY) return to_nccl(rc);
    }
    fn_allreduce f = get_ncclAllReduce();
    return f ? f(sendbuff, recvbuff, count, datatype, op, comm, stream) : ncclInternalError;
}

ncclResult_t ncclReduceScatter(const void *sendbuff, void *recvbuff, size_t recvcount, ncclDataType_t datatype,
                               ncclRedOp_t op, ncclComm_t comm, cudaStream_t stream) {
    load_cfg();
    int n = 0;
    ccb_comm *c = lossy_ok(cfg.codec, op) ? fused_comm(comm, datatype, bytes_of(recvcount, datatype), stream, NULL, &n) : NULL;
    if (c) {
        /* the residual covers the whole send buffer: every rank quantises all n shards */
        float *ef = cfg.codec != CCB_CODEC_NONE ? ef_buffer(comm, sendbuff, recvbuff, recvcount * (size_t)n, 1) : NULL;
        const void *s[1] = {sendbuff};
        void *r[1] = {recvbuff};
        float *e[1] = {ef};
        int rc = ccb_reduce_scatter(c, s, r, recvcount, dtype_of(datatype), (int)op, cfg.codec, ef ? e : NULL, stream);
        if (rc != CCB_ERR_UNSUPPORTED && rc != CCB_ERR_CAPACITY) return to_nccl(rc);
    }
    fn_reducescatter f = get_ncclReduceScatter();
    return f ? f(sendbuff, recvbuff, recvcount, datatype, op, comm, stream) : ncclInternalError;
}

ncclResult_t ncclAllGather(const void *sendbuff, void *recvbuff, size_t sendcount, ncclDataType_t datatype,
                           ncclComm_t comm, cudaStream_t stream) {
    ccb_comm *c = fused_comm(comm, datatype, bytes_of(sendcount, datatype), stream, NULL, NULL);
    if (c) {
        const void *s[1] = {sendbuff};
        void *r[1] = {recvbuff};
        int rc = ccb_all_gather(c, s, r, sendcount, dtype_of(datatype), cfg.move_codec, stream);
        if (rc != CCB_ERR_UNSUPPORTED && rc != CCB_ERR_CAPACITY) return to_nccl(rc);
    }
    fn_allgather f = get_ncclAllGather();
    return f ? f(sendbuff, recvbuff, sendcount, datatype, comm, stream) : ncclInternalError;
}

ncclResult_t ncclBroadcast(const void *sendbuff, void *recvbuff, size_t count, ncclDataType_t datatype, int root,
                           ncclComm_t comm, cudaStream_t stream) {
    ccb_comm *c = fused_comm(comm, datatype, bytes_of(count, datatype), stream, NULL, NULL);
    if (c) {
        const void *s[1] = {sendbuff};
        void *r[1] = {recvbuff};
        int rc = ccb_broadcast(c, s, r, count, dtype_of(datatype), root, cfg.move_codec, stream);
        if (rc != CCB_ERR_UNSUPPORTED && rc != CCB_ERR_CAPACITY) return to_nccl(rc);
    }
    fn_broadcast f = get_ncclBroadcast();
    return f ? f(sendbuff, recvbuff, count, datatype, root, comm, stream) : ncclInternalError;
}

ncclResult_t ncclBcast(void *buff, size_t count, ncclDataType_t datatype, int root, ncclComm_t comm, cudaStream_t stream) {
    return ncclBroadcast(buff, buff, count, datatype, root, comm, stream);
}

ncclResult_t ncclReduce(const void *sendbuff, void *recvbuff, size_t count, ncclDataType_t datatype, ncclRedOp_t op,
                        int root, ncclComm_t comm, cudaStream_t stream) {
    load_cfg();
    int rank = -1;
    ccb_comm *c = lossy_ok(cfg.codec, op) ? fused_comm(comm, datatype, bytes_of(count, datatype), stream, &rank, NULL) : NULL;
    if (c) {
        const void *s[1] = {sendbuff};
        void *r[1] = {recvbuff ? recvbuff : (void *)sendbuff}; /* non-root ranks may pass NULL; it is not written */
        int rc = ccb_reduce(c, s, r, count, dtype_of(datatype), (int)op, root, cfg.codec, stream);
        if (rc != CCB_ERR_UNSUPPORTED && rc != CCB_ERR_CAPACITY) return to_nccl(rc);
    }
    fn_reduce f = get_ncclReduce();
    return f ? f(sendbuff, recvbuff, count, datatype, op, root, comm, stream) : ncclInternalError;
}

/* Extended collectives (signatures of nccl_extensions.h; 0 = success). */
int ncclAllToAll(const void *sendbuf, size_t sendcount, ncclDataType_t sendtype, void *recvbuf, size_t recvcount,
                 ncclDataType_t recvtype, ncclComm_t comm, cudaStream_t stream) {
    ccb_comm *c = (sendtype == recvtype && sendcount == recvcount) ? fused_comm(comm, sendtype, bytes_of(sendcount, sendtype), stream, NULL, NULL) : NULL;
    if (c) {
        const void *s[1] = {sendbuf};
        void *r[1] = {recvbuf};
        int rc = ccb_all_to_all(c, s, r, sendcount, dtype_of(sendtype), cfg.move_codec, stream);
        if (rc != CCB_ERR_UNSUPPORTED && rc != CCB_ERR_CAPACITY) return rc != CCB_OK;
    }
    fn_ext_a2a f = get_ncclAllToAll();
    return f ? f(sendbuf, sendcount, sendtype, recvbuf, recvcount, recvtype, comm, stream) : 1;
}

/* NCCL 2.28 added its own all-to-all under a different spelling and signature (count per
 * peer, one type): same fused path. The prototype is written out because older nccl.h
 * headers, which this file must also compile against, do not have it. */
typedef ncclResult_t (*fn_a2a_228)(const void *, void *, size_t, ncclDataType_t, ncclComm_t, cudaStream_t);
ncclResult_t ncclAlltoAll(const void *sendbuff, void *recvbuff, size_t count, ncclDataType_t datatype, ncclComm_t comm,
                          cudaStream_t stream) {
    ccb_comm *c = fused_comm(comm, datatype, bytes_of(count, datatype), stream, NULL, NULL);
    if (c) {
        const void *s[1] = {sendbuff};
        void *r[1] = {recvbuff};
        int rc = ccb_all_to_all(c, s, r, count, dtype_of(datatype), cfg.move_codec, stream);
        if (rc != CCB_ERR_UNSUPPORTED && rc != CCB_ERR_CAPACITY) return to_nccl(rc);
    }
    static fn_a2a_228 real;
    if (!real) real = (fn_a2a_228)dlsym(RTLD_NEXT, "ncclAlltoAll");
    return real ? real(sendbuff, recvbuff, count, datatype, comm, stream) : ncclInvalidUsage;
}

int ncclScatter(const void *sendbuf, size_t sendcount, ncclDataType_t sendtype, void *recvbuf, size_t recvcount,
                ncclDataType_t recvtype, int root, ncclComm_t comm, cudaStream_t stream) {
    ccb_comm *c = (sendtype == recvtype && sendcount == recvcount) ? fused_comm(comm, sendtype, bytes_of(sendcount, sendtype), stream, NULL, NULL) : NULL;
    if (c) {
        const void *s[1] = {sendbuf ? sendbuf : recvbuf};
        void *r[1] = {recvbuf};
        int rc = ccb_scatter(c, s, r, recvcount, dtype_of(recvtype), root, cfg.move_codec, stream);
        if (rc != CCB_ERR_UNSUPPORTED && rc != CCB_ERR_CAPACITY) return rc != CCB_OK;
    }
    fn_ext_rooted f = get_ncclScatter();
    return f ? f(sendbuf, sendcount, sendtype, recvbuf, recvcount, recvtype, root, comm, stream) : 1;
}

int ncclGather(const void *sendbuf, size_t sendcount, ncclDataType_t sendtype, void *recvbuf, size_t recvcount,
               ncclDataType_t recvtype, int root, ncclComm_t comm, cudaStream_t stream) {
    ccb_comm *c = (sendtype == recvtype && sendcount == recvcount) ? fused_comm(comm, sendtype, bytes_of(sendcount, sendtype), stream, NULL, NULL) : NULL;
    if (c) {
        const void *s[1] = {sendbuf};
        void *r[1] = {recvbuf ? recvbuf : (void *)sendbuf};
        int rc = ccb_gather(c, s, r, sendcount, dtype_of(sendtype), root, cfg.move_codec, stream);
        if (rc != CCB_ERR_UNSUPPORTED && rc != CCB_ERR_CAPACITY) return rc != CCB_OK;
    }
    fn_ext_rooted f = get_ncclGather();
    return f ? f(sendbuf, sendcount, sendtype, recvbuf, recvcount, recvtype, root, comm, stream) : 1;
}

/* ------------------------------------------------------- point-to-point --
 * Compressed ncclSend / ncclRecv (CCB_P2P_CODEC): encode into a stream-ordered temporary,
 * move the wire bytes with the real NCCL call, decode after the receive. Inside a group NCCL
 * only records the call and runs it at the outermost ncclGroupEnd, so the decode and the
 * release of the temporaries are deferred to that point as well. Both ends must run with the
 * same setting; the wire size is a function of (codec, dtype, count) only. */
typedef struct {
    void *wire, *user; /* user != NULL: a receive to decode into user */
    size_t count;
    int dtype;
    cudaStream_t stream;
} p2p_pending;
static __thread p2p_pending *g_pending; /* grows as needed: a full table must never change the wire format */
static __thread int g_npending, g_pending_cap;

static int pending_push(const p2p_pending *p) {
    if (g_npending == g_pending_cap) {
        const int cap = g_pending_cap ? 2 * g_pending_cap : 64;
        p2p_pending *q = (p2p_pending *)realloc(g_pending, (size_t)cap * sizeof(*q));
        if (!q) return -1;
        g_pending = q;
        g_pending_cap = cap;
    }
    g_pending[g_npending++] = *p;
    return 0;
}

static ncclResult_t p2p_finish(const p2p_pending *p) {
    ncclResult_t rc = ncclSuccess;
    if (p->user && ccb_decode(cfg.p2p_codec, p->dtype, p->wire, p->count, p->user, p->stream) != CCB_OK) rc = ncclInternalError;
    cudaFreeAsync(p->wire, p->stream);
    return rc;
}
static int p2p_wanted(size_t count, ncclDataType_t dt, cudaStream_t stream) {
    load_cfg();
    if (cfg.disabled || cfg.p2p_codec == CCB_CODEC_NONE || dtype_of(dt) < 0 || count == 0) return 0;
    /* only values both ends share (codec, type, count) may decide the wire format */
    if (bytes_of(count, dt) < cfg.min_bytes || stream_is_capturing(stream)) return 0;
    return 1;
}

ncclResult_t ncclSend(const void *sendbuff, size_t count, ncclDataType_t datatype, int peer, ncclComm_t comm, cudaStream_t stream) {
    fn_send f = get_ncclSend();
    if (!f) return ncclInternalError;
    if (!p2p_wanted(count, datatype, stream)) return f(sendbuff, count, datatype, peer, comm, stream);
    const int dt = dtype_of(datatype);
    const size_t wb = (size_t)ccb_wire_bytes(cfg.p2p_codec, dt, count);
    p2p_pending p = {NULL, NULL, count, dt, stream};
    if (cudaMallocAsync(&p.wire, wb, stream) != cudaSuccess) return ncclUnhandledCudaError;
    if (ccb_encode(cfg.p2p_codec, dt, sendbuff, count, p.wire, stream) != CCB_OK) {
        cudaFreeAsync(p.wire, stream);
        return ncclInternalError;
    }
    ncclResult_t rc = f(p.wire, wb, ncclUint8, peer, comm, stream);
    if (g_group_depth > 0 && rc == ncclSuccess) {
        if (pending_push(&p) != 0) return ncclSystemError; /* the wire is leaked rather than freed under NCCL */
    } else {
        p2p_finish(&p);
    }
    return rc;
}

ncclResult_t ncclRecv(void *recvbuff, size_t count, ncclDataType_t datatype, int peer, ncclComm_t comm, cudaStream_t stream) {
    fn_recv f = get_ncclRecv();
    if (!f) return ncclInternalError;
    if (!p2p_wanted(count, datatype, stream)) return f(recvbuff, count, datatype, peer, comm, stream);
    const int dt = dtype_of(datatype);
    const size_t wb = (size_t)ccb_wire_bytes(cfg.p2p_codec, dt, count);
    p2p_pending p = {NULL, recvbuff, count, dt, stream};
    if (cudaMallocAsync(&p.wire, wb, stream) != cudaSuccess) return ncclUnhandledCudaError;
    ncclResult_t rc = f(p.wire, wb, ncclUint8, peer, comm, stream);
    if (rc != ncclSuccess) {
        cudaFreeAsync(p.wire, stream);
        return rc;
    }
    if (g_group_depth > 0) return pending_push(&p) == 0 ? ncclSuccess : ncclSystemError;
    return p2p_finish(&p);
}

ncclResult_t ncclGroupStart(void) {
    ++g_group_depth;
    fn_group f = get_ncclGroupStart();
    return f ? f() : ncclInternalError;
}
ncclResult_t ncclGroupEnd(void) {
    if (g_group_depth > 0) --g_group_depth;
    fn_group f = get_ncclGroupEnd();
    ncclResult_t rc = f ? f() : ncclInternalError;
    if (g_group_depth == 0 && g_npending > 0) { /* the grouped transfers are enqueued now */
        for (int i = 0; i < g_npending; ++i) {
            const ncclResult_t r2 = (rc == ncclSuccess) ? p2p_finish(&g_pending[i]) : (cudaFreeAsync(g_pending[i].wire, g_pending[i].stream), ncclSuccess);
            if (rc == ncclSuccess) rc = r2;
        }
        g_npending = 0;
    }
    return rc;
}

static void drop_comm(ncclComm_t comm) {
    pthread_mutex_lock(&g_lock);
    for (int i = 0; i < MAX_COMMS; ++i)
        if (g_comms[i].real == comm) {
            if (g_comms[i].c) ccb_comm_destroy(g_comms[i].c);
            memset(&g_comms[i], 0, sizeof(g_comms[i]));
        }
    for (int i = 0; i < MAX_EF; ++i)
        if (g_ef[i].comm == comm && g_ef[i].resid) {
            cudaFree(g_ef[i].resid);
            memset(&g_ef[i], 0, sizeof(g_ef[i]));
        }
    pthread_mutex_unlock(&g_lock);
}

ncclResult_t ncclCommDestroy(ncclComm_t comm) {
    drop_comm(comm);
    fn_commdestroy f = get_ncclCommDestroy();
    return f ? f(comm) : ncclInternalError;
}
ncclResult_t ncclCommAbort(ncclComm_t comm) {
    drop_comm(comm);
    fn_commdestroy f = get_ncclCommAbort();
    return f ? f(comm) : ncclInternalError;
}

/* How many calls took the fused path so far (for tests and logs). */
unsigned long long ccb_nccl_fused_calls(void) { return (unsigned long long)ccb_launch_count(); }

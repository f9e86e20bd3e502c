/* base_ncclXxx: calls into the NCCL library that findso recorded, past every preloaded
 * wrapper (see include/ccb/compat/nccl/nccl_base.h). One table drives loading and lookup. */
#define _GNU_SOURCE
#include <dlfcn.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include "base_impl.h"
#include "nccl/nccl_base.h"

enum { F_ALLREDUCE, F_BROADCAST, F_REDUCE, F_ALLGATHER, F_REDUCESCATTER, F_SEND, F_RECV, F_COUNT };
static const char *const k_names[F_COUNT] = {"ncclAllReduce", "ncclBroadcast", "ncclReduce", "ncclAllGather",
                                             "ncclReduceScatter", "ncclSend", "ncclRecv"};
static void *g_fn[F_COUNT];
static void *g_lib;
static int g_state; /* 0 not tried, 1 loaded, -1 failed */
static ncclComm_t g_comm_override;

static int read_state(const char *path, char *line, size_t cap) {
    FILE *f = fopen(path, "r");
    if (!f) return -1;
    const int ok = fgets(line, (int)cap, f) != NULL;
    fclose(f);
    if (!ok) return -1;
    line[strcspn(line, "\r\n")] = '\0';
    return line[0] ? 0 : -1;
}

int load_base_impl(const char *state_path) {
    if (g_state == 1) return 0;
    char line[1024] = "", tried[1200] = "";
    int have = -1;
    if (state_path && *state_path) {
        have = read_state(state_path, line, sizeof(line));
        snprintf(tried, sizeof(tried), "%s", state_path);
    } else {
        const char *bench = getenv("BENCH_DIR");
        if (bench && *bench) {
            snprintf(tried, sizeof(tried), "%s/%s", bench, BASE_SO_FILE);
            have = read_state(tried, line, sizeof(line));
        }
        if (have != 0) {
            snprintf(tried, sizeof(tried), "%s", BASE_SO_FILE);
            have = read_state(tried, line, sizeof(line));
        }
    }
    if (have != 0) {
        fprintf(stderr, "[base_impl] no library recorded in %s (run bin/nccl/findso first)\n", tried);
        g_state = -1;
        return -1;
    }
    g_lib = dlopen(line, RTLD_NOW | RTLD_LOCAL);
    if (!g_lib) {
        fprintf(stderr, "[base_impl] cannot open %s: %s\n", line, dlerror());
        g_state = -1;
        return -1;
    }
    for (int i = 0; i < F_COUNT; ++i) {
        g_fn[i] = dlsym(g_lib, k_names[i]);
        if (!g_fn[i]) {
            fprintf(stderr, "[base_impl] %s has no %s\n", line, k_names[i]);
            g_state = -1;
            return -1;
        }
    }
    g_state = 1;
    return 0;
}

void base_nccl_set_comm(ncclComm_t comm) { g_comm_override = comm; }

static void *entry(int which) {
    if (g_state == 0) load_base_impl(NULL);
    return g_state == 1 ? g_fn[which] : NULL;
}
#define COMM(c) (g_comm_override ? g_comm_override : (c))

ncclResult_t base_ncclAllReduce(const void *s, void *r, size_t n, ncclDataType_t dt, ncclRedOp_t op, ncclComm_t c, cudaStream_t st) {
    ncclResult_t (*f)(const void *, void *, size_t, ncclDataType_t, ncclRedOp_t, ncclComm_t, cudaStream_t) = entry(F_ALLREDUCE);
    return f ? f(s, r, n, dt, op, COMM(c), st) : ncclSystemError;
}
ncclResult_t base_ncclBroadcast(const void *s, void *r, size_t n, ncclDataType_t dt, int root, ncclComm_t c, cudaStream_t st) {
    ncclResult_t (*f)(const void *, void *, size_t, ncclDataType_t, int, ncclComm_t, cudaStream_t) = entry(F_BROADCAST);
    return f ? f(s, r, n, dt, root, COMM(c), st) : ncclSystemError;
}
ncclResult_t base_ncclReduce(const void *s, void *r, size_t n, ncclDataType_t dt, ncclRedOp_t op, int root, ncclComm_t c,
                             cudaStream_t st) {
    ncclResult_t (*f)(const void *, void *, size_t, ncclDataType_t, ncclRedOp_t, int, ncclComm_t, cudaStream_t) = entry(F_REDUCE);
    return f ? f(s, r, n, dt, op, root, COMM(c), st) : ncclSystemError;
}
ncclResult_t base_ncclAllGather(const void *s, void *r, size_t n, ncclDataType_t dt, ncclComm_t c, cudaStream_t st) {
    ncclResult_t (*f)(const void *, void *, size_t, ncclDataType_t, ncclComm_t, cudaStream_t) = entry(F_ALLGATHER);
    return f ? f(s, r, n, dt, COMM(c), st) : ncclSystemError;
}
ncclResult_t base_ncclReduceScatter(const void *s, void *r, size_t n, ncclDataType_t dt, ncclRedOp_t op, ncclComm_t c,
                                    cudaStream_t st) {
    ncclResult_t (*f)(const void *, void *, size_t, ncclDataType_t, ncclRedOp_t, ncclComm_t, cudaStream_t) = entry(F_REDUCESCATTER);
    return f ? f(s, r, n, dt, op, COMM(c), st) : ncclSystemError;
}
ncclResult_t base_ncclSend(const void *s, size_t n, ncclDataType_t dt, int peer, ncclComm_t c, cudaStream_t st) {
    ncclResult_t (*f)(const void *, size_t, ncclDataType_t, int, ncclComm_t, cudaStream_t) = entry(F_SEND);
    return f ? f(s, n, dt, peer, COMM(c), st) : ncclSystemError;
}
ncclResult_t base_ncclRecv(void *r, size_t n, ncclDataType_t dt, int peer, ncclComm_t c, cudaStream_t st) {
    ncclResult_t (*f)(void *, size_t, ncclDataType_t, int, ncclComm_t, cudaStream_t) = entry(F_RECV);
    return f ? f(r, n, dt, peer, COMM(c), st) : ncclSystemError;
}

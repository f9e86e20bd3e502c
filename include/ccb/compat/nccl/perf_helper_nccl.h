/* Helper for LD_PRELOAD perf wrappers around NCCL. Declares just enough of the NCCL
 * and CUDA types for a wrapper to compile with plain `cc`, without nccl.h or the
 * CUDA toolkit, and the per-process timing table shared by all hooks.
 * Source-compatible with the reference's run_codes/wrappers/include/nccl/
 * perf_helper_nccl.h (same macro PERF_NCCL_REAL and entry points). */
#ifndef PERF_HELPER_NCCL_H
#define PERF_HELPER_NCCL_H

#include <dlfcn.h>
#include <stddef.h>
#include <stdio.h>

#include "perf_helper.h"

#ifdef __cplusplus
extern "C" {
#endif

#ifndef NCCL_H_ /* real nccl.h not included: provide stand-ins with the same values */
struct CUstream_st;
typedef struct CUstream_st *cudaStream_t;
typedef struct ncclComm *ncclComm_t;
#ifndef NCCL_UNIQUE_ID_BYTES
#define NCCL_UNIQUE_ID_BYTES 128
typedef struct { char internal[NCCL_UNIQUE_ID_BYTES]; } ncclUniqueId;
#endif
typedef enum {
    ncclSuccess = 0, ncclUnhandledCudaError = 1, ncclSystemError = 2, ncclInternalError = 3,
    ncclInvalidArgument = 4, ncclInvalidUsage = 5, ncclRemoteError = 6, ncclInProgress = 7
} ncclResult_t;
typedef enum {
    ncclInt8 = 0, ncclUint8 = 1, ncclInt32 = 2, ncclUint32 = 3, ncclInt64 = 4, ncclUint64 = 5,
    ncclFloat16 = 6, ncclFloat32 = 7, ncclFloat64 = 8, ncclBfloat16 = 9
} ncclDataType_t;
typedef enum { ncclSum = 0, ncclProd = 1, ncclMax = 2, ncclMin = 3, ncclAvg = 4 } ncclRedOp_t;
#endif

static inline size_t perf_nccl_type_size(ncclDataType_t t) {
    switch ((int)t) {
        case 0: case 1: return 1;
        case 6: case 9: return 2;
        case 2: case 3: case 7: return 4;
        case 4: case 5: case 8: return 8;
        default: return 4;
    }
}
#ifndef NCCL_COMPRESS_TOOLS_H
#define nccl_type_size perf_nccl_type_size
#endif

static inline void *perf_nccl_get_real(const char *name) {
    void *p = dlsym(RTLD_NEXT, name);
    if (!p) fprintf(stderr, "[perf_nccl] dlsym(RTLD_NEXT, %s) failed: %s\n", name, dlerror());
    return p;
}
/* Inside a hook called `name`: resolves the next `name` in the preload chain into
 * real_<name>, returning ncclInternalError from the hook when there is none. */
#define PERF_NCCL_REAL(name)                                                        \
    static __typeof__(&name) real_##name = NULL;                                    \
    if (!real_##name) real_##name = (__typeof__(&name))perf_nccl_get_real(#name);   \
    if (!real_##name) return ncclInternalError

perf_state_t *perf_nccl_get_tls(void); /* process-wide table (the name is historical) */
void perf_nccl_flush(void);            /* -> <PERF_OUTPUT_DIR>/perf_nccl_<rank>.csv     */
void perf_nccl_set_node_map_comm(ncclComm_t comm);
void perf_nccl_init_node_map(ncclComm_t comm);
int perf_nccl_is_intra(int rank);      /* 1 when `rank` runs on this host               */
int perf_nccl_local_size(void);
int perf_nccl_rank(void);

/* Addition: device-side duration of an asynchronous call. Bracket the call with
 * perf_nccl_dev_begin / perf_nccl_dev_end on its stream; the row is written once the
 * events have completed (at a later hook or at flush) with an extra column
 * "device_duration" (seconds). Active when PERF_NCCL_DEVICE_TIME=1 and libcudart is
 * loaded in the process; otherwise perf_nccl_dev_end notes the row down at once. */
void *perf_nccl_dev_begin(cudaStream_t stream);
void perf_nccl_dev_end(void *token, cudaStream_t stream, const char *func_name, double start, int num_attrs,
                       const perf_attr_t *attrs);

#ifdef __cplusplus
}
#endif
#endif /* PERF_HELPER_NCCL_H */

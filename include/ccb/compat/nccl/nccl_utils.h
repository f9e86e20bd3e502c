/* NCCL benchmark bridge without MPI: rank discovery from the launcher's
 * environment, ncclUniqueId bootstrap through a shared file, a TCP barrier,
 * file-based aggregation of per-rank results, CSV output. Source-compatible with the
 * reference's run_codes/benchmark-core/include/nccl/nccl_utils.h. */
#ifndef NCCL_UTILS_H
#define NCCL_UTILS_H

#include <cuda_runtime.h>
#include <nccl.h>
#include <stddef.h>
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>

#include "utils.h"
#include "validation.h"

#ifdef __cplusplus
extern "C" {
#endif

#ifndef NCCLCHECK
#define NCCLCHECK(call)                                                                              \
    do {                                                                                             \
        ncclResult_t r_ = (call);                                                                    \
        if (r_ != ncclSuccess) {                                                                     \
            fprintf(stderr, "[NCCLCHECK error at %s:%d] %s\n", __FILE__, __LINE__, ncclGetErrorString(r_)); \
            exit(1);                                                                                 \
        }                                                                                            \
    } while (0)
#endif

typedef struct {
    int rank;
    int size;
    test_config_t config;
    ncclComm_t comm;
    cudaStream_t stream;
    int *d_barrier;         /* kept for layout compatibility; unused        */
    int barrier_peers[256]; /* rank 0: one socket per peer; peers: [0] only */
    int barrier_listen_fd;
} nccl_test_context_t;

nccl_test_context_t nccl_test_init(int argc, char **argv, const char *test_name);
void nccl_test_fini(nccl_test_context_t *ctx);
void nccl_load_input(const nccl_test_context_t *ctx, void *buf, size_t msg_size, ncclDataType_t datatype);
void nccl_report_results(const nccl_test_context_t *ctx, size_t msg_size, int count, float total_time_ms,
                         int local_errors, const validation_result_t *metrics, double bw);
data_type_t nccl_to_data_type(ncclDataType_t nccl_type);
ncclDataType_t data_type_to_nccl(data_type_t type);
size_t nccl_dtype_size(ncclDataType_t dtype);
int nccl_get_my_rank(void);
void nccl_barrier(nccl_test_context_t *ctx);
int *nccl_parse_env_int_array(const char *env_name, int expected_len, int *out_len);
void nccl_csv_write(const char *path, const char *header, const char *fmt, ...);

/* Additions of this implementation: the name of the running test (for CSV rows and
 * the oracle cache) and a bus-bandwidth factor for the result CSV. */
void nccl_set_busbw_factor(double factor);
const char *nccl_test_name(void);

#ifdef __cplusplus
}
#endif
#endif /* NCCL_UTILS_H */

/* MPI benchmark bridge: lifecycle, input loading, result reporting, type maps.
 * Source-compatible with the reference's
 * run_codes/benchmark-core/include/mpi/mpi_utils.h. */
#ifndef MPI_UTILS_H
#define MPI_UTILS_H

#include <mpi.h>

#include "utils.h"
#include "validation.h"

#ifdef __cplusplus
extern "C" {
#endif

data_type_t mpi_to_data_type(MPI_Datatype mpi_type);
MPI_Datatype data_type_to_mpi(data_type_t type);
MPI_Op parse_mpi_op(const char *name);

typedef struct {
    int rank;
    int size;
    test_config_t config;
} mpi_test_context_t;

/* PMPI_Init, the job->device map (bin/libs/libjob_device_mapper.so when present),
 * argv, banner. */
mpi_test_context_t mpi_test_init(int argc, char **argv, const char *test_name);
void mpi_test_fini(const mpi_test_context_t *ctx);
void mpi_load_input(const mpi_test_context_t *ctx, void *buf, size_t msg_size, MPI_Datatype datatype);
/* total_time_user in seconds over all iterations; prints avg / min / max over ranks. */
void mpi_report_results(const mpi_test_context_t *ctx, size_t msg_size, int count, double total_time_user,
                        int local_errors, const validation_result_t *metrics);
int *parse_env_int_array(const char *env_name, int expected_len, int *out_len);
void mpi_csv_write(const char *path, const char *header, const char *fmt, ...);

/* Additions: bandwidth definitions for the result CSV (set before mpi_report_results). */
void mpi_set_bandwidth(double ref_bw_gbs, double busbw_factor);

#ifdef __cplusplus
}
#endif
#endif /* MPI_UTILS_H */

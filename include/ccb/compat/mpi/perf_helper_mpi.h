/* Helper for LD_PRELOAD perf wrappers around MPI: one process-wide timing table, the
 * node map, message sizes. Source-compatible with the reference's
 * run_codes/wrappers/include/mpi/perf_helper_mpi.h. */
#ifndef PERF_HELPER_MPI_H
#define PERF_HELPER_MPI_H

#include <mpi.h>

#include "perf_helper.h"

#ifdef __cplusplus
extern "C" {
#endif

perf_state_t *perf_mpi_get_tls(void); /* process-wide (the name is historical) */
void perf_mpi_flush(void);            /* -> <PERF_OUTPUT_DIR>/perf_function_<rank>.csv */
void perf_mpi_init_node_map(void);    /* one PMPI_Allgather of processor names */
int perf_mpi_world_rank(void);
int perf_mpi_is_intra(int rank);
double perf_mpi_msg_size(int count, MPI_Datatype datatype);

#ifdef __cplusplus
}
#endif
#endif /* PERF_HELPER_MPI_H */

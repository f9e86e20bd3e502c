/* CPU oracle of every collective: each rank recomputes the expected result from the
 * deterministic data source of all ranks, so no communication call is needed while
 * an interposer is loaded. Source-compatible with the reference's
 * run_codes/benchmark-core/include/dummy_collectives.h. The reference accumulates
 * sums in the element type; that behaviour is kept for these entry points and a
 * float64-accumulating AllReduce is offered beside it. */
#ifndef DUMMY_COLLECTIVES_H
#define DUMMY_COLLECTIVES_H

#include <stddef.h>

#include "utils.h"

#ifdef __cplusplus
extern "C" {
#endif

void dummy_load_rank_data(const char *input_file, data_type_t datatype, pattern_type_t pattern_type, void *buf,
                          size_t bytes, int sim_rank, int nranks);
void dummy_allreduce(void *ref, const char *input_file, data_type_t datatype, pattern_type_t pattern_type, int count,
                     int nranks);
void dummy_alltoall(void *ref, const char *input_file, data_type_t datatype, pattern_type_t pattern_type,
                    int count_per, int nranks, int rank);
void dummy_allgather(void *ref, const char *input_file, data_type_t datatype, pattern_type_t pattern_type, int count,
                     int nranks);
void dummy_reduce(void *ref, const char *input_file, data_type_t datatype, pattern_type_t pattern_type, int count,
                  int nranks, int root);
void dummy_scatter(void *ref, const char *input_file, data_type_t datatype, pattern_type_t pattern_type, int count,
                   int nranks, int root, int rank);
void dummy_gather(void *ref, const char *input_file, data_type_t datatype, pattern_type_t pattern_type, int count,
                  int nranks, int root);
void dummy_reduce_scatter(void *ref, const char *input_file, data_type_t datatype, pattern_type_t pattern_type,
                          int count, int nranks, int rank);
void dummy_bcast(void *ref, const char *input_file, data_type_t datatype, pattern_type_t pattern_type, int count,
                 int nranks, int root);
/* Same as dummy_allreduce but sums in float64 and rounds once at the end. */
void dummy_allreduce_f64(void *ref, const char *input_file, data_type_t datatype, pattern_type_t pattern_type,
                         int count, int nranks);

#ifdef __cplusplus
}
#endif
#endif /* DUMMY_COLLECTIVES_H */

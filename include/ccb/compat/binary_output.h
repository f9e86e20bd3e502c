/* Raw dumps of reference and user results: "<base>_<suffix>.bin", written by one
 * rank or by every rank at offset rank * chunk. Source-compatible with the
 * reference's run_codes/benchmark-core/include/binary_output.h. */
#ifndef BINARY_OUTPUT_H
#define BINARY_OUTPUT_H

#include <stddef.h>

#include "utils.h"

#ifdef __cplusplus
extern "C" {
#endif

void write_binary_single(const char *base_path, const char *suffix, const void *buf, size_t bytes, int rank,
                         int writer_rank);
void write_binary_multi(const char *base_path, const char *suffix, const void *buf, size_t chunk_size, int rank,
                        int nranks);
void binary_accumulate(void *accum, const void *buf, int count, data_type_t dtype);
void binary_average(void *accum, int count, data_type_t dtype, int divisor);

#ifdef __cplusplus
}
#endif
#endif /* BINARY_OUTPUT_H */

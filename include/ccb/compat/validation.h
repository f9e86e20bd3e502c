/* Result validation and the deviation-metric registry. Source-compatible with the
 * reference's run_codes/benchmark-core/include/validation.h. Metrics come from
 * bin/libs/validation.so when that file exists (same g_metric_registry contract as
 * the reference's scripts/register_metrics.sh output) and otherwise from the
 * registry compiled into the core library. */
#ifndef VALIDATION_H
#define VALIDATION_H

#include <stddef.h>
#include <stdint.h>

#include "utils.h"

#ifdef __cplusplus
extern "C" {
#endif

#define MAX_METRICS 30

typedef double (*metric_func_t)(const void *buf1, const void *buf2, int count, data_type_t dtype);
typedef struct {
    const char *name;
    metric_func_t func;
} metric_entry_t;

int init_validation_so(void);
int validation_registry_count(void);
const char *validation_metric_name(int idx);
size_t get_element_size(data_type_t dtype);
double to_double(const void *ptr, data_type_t dtype, int index);

typedef struct {
    int correct;
    size_t num_elements;
    double values[MAX_METRICS];
} validation_result_t;

uint32_t parse_metric_mask(const char *str);
validation_result_t validate_result(const void *user_buf, const void *reference_buf, int count, data_type_t dtype,
                                    double tolerance, uint32_t metrics_mask);
int buffers_equal(const void *buf1, const void *buf2, int count, data_type_t datatype, double tolerance);

#ifdef __cplusplus
}
#endif
#endif /* VALIDATION_H */

/* Largest absolute element error. */
#include "metric_iter.h"
double compute_max_abs_err(const void *buf1, const void *buf2, int count, data_type_t dtype) {
    double m = 0.0;
    METRIC_FOR_EACH(buf1, buf2, count, dtype, a, b, { const double d = fabs(a - b); if (d > m || d != d) m = d; });
    return m;
}

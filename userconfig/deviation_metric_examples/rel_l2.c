/* Relative L2 error: ||user - reference|| / ||reference|| (0 when both are zero). */
#include "metric_iter.h"
double compute_rel_l2(const void *buf1, const void *buf2, int count, data_type_t dtype) {
    double num = 0.0, den = 0.0;
    METRIC_FOR_EACH(buf1, buf2, count, dtype, a, b, { num += (a - b) * (a - b); den += b * b; });
    if (den == 0.0) return num == 0.0 ? 0.0 : INFINITY;
    return sqrt(num / den);
}

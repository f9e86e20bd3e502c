/* Root mean squared error (sqrt of mse). */
#include "metric_iter.h"
double compute_rmse(const void *buf1, const void *buf2, int count, data_type_t dtype) {
    if (count <= 0) return 0.0;
    double s = 0.0;
    METRIC_FOR_EACH(buf1, buf2, count, dtype, a, b, s += (a - b) * (a - b));
    return sqrt(s / count);
}

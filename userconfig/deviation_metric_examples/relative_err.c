/* Mean of |user - ref| / max(|ref|, eps); eps from $METRIC_RELATIVE_ERR_EPS (1e-8). */
#include "metric_iter.h"
double compute_relative_err(const void *buf1, const void *buf2, int count, data_type_t dtype) {
    if (count <= 0) return 0.0;
    const char *env = getenv("METRIC_RELATIVE_ERR_EPS");
    const double eps = env ? atof(env) : 1e-8;
    double s = 0.0;
    METRIC_FOR_EACH(buf1, buf2, count, dtype, a, b, { double d = fabs(b); if (d < eps) d = eps; s += fabs(a - b) / d; });
    return s / count;
}

/* Peak signal-to-noise ratio: 20 log10(peak) - 10 log10(mse). The peak comes from
 * $METRIC_PSNR_MAX_VAL, else 1.0 for float/double, 65535 for int, 255 for char. */
#include "metric_iter.h"
double compute_psnr(const void *buf1, const void *buf2, int count, data_type_t dtype) {
    if (count <= 0) return INFINITY;
    double s = 0.0;
    METRIC_FOR_EACH(buf1, buf2, count, dtype, a, b, s += (a - b) * (a - b));
    const double mse = s / count;
    if (mse <= 0.0) return INFINITY;
    const char *env = getenv("METRIC_PSNR_MAX_VAL");
    double peak = env ? atof(env) : (dtype == TYPE_INT ? 65535.0 : dtype == TYPE_CHAR ? 255.0 : 1.0);
    return 20.0 * log10(peak) - 10.0 * log10(mse);
}

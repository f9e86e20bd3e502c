/* Global one-dimensional structural similarity with stabilisers (K1, K2) from
 * $METRIC_SSIM_K1 / $METRIC_SSIM_K2 (0.01 / 0.03). Two passes: means, then moments. */
#include "metric_iter.h"
double compute_ssim(const void *buf1, const void *buf2, int count, data_type_t dtype) {
    if (count <= 0) return 0.0;
    const char *e1 = getenv("METRIC_SSIM_K1"), *e2 = getenv("METRIC_SSIM_K2");
    const double k1 = e1 ? atof(e1) : 0.01, k2 = e2 ? atof(e2) : 0.03;
    double ma = 0.0, mb = 0.0;
    METRIC_FOR_EACH(buf1, buf2, count, dtype, a, b, { ma += a; mb += b; });
    ma /= count;
    mb /= count;
    double va = 0.0, vb = 0.0, cab = 0.0;
    METRIC_FOR_EACH(buf1, buf2, count, dtype, a, b,
                    { va += (a - ma) * (a - ma); vb += (b - mb) * (b - mb); cab += (a - ma) * (b - mb); });
    va /= count;
    vb /= count;
    cab /= count;
    const double c1 = k1 * k1, c2 = k2 * k2;
    const double den = (ma * ma + mb * mb + c1) * (va + vb + c2);
    return den == 0.0 ? 1.0 : (2.0 * ma * mb + c1) * (2.0 * cab + c2) / den;
}

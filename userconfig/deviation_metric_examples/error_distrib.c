/* Error percentiles. Appends "P50= P95= P99= P99.9= Max= msg_bytes=" to
 * $METRIC_ERROR_DISTRIB_OUTPUT (default error_distrib.txt) and returns P50.
 * Percentiles are taken by selection on a float copy of the absolute errors. */
#include <string.h>

#include "metric_iter.h"

static float kth(float *v, int n, int k) { /* quickselect, in place */
    int lo = 0, hi = n - 1;
    while (lo < hi) {
        const float pivot = v[lo + (hi - lo) / 2];
        int i = lo, j = hi;
        while (i <= j) {
            while (v[i] < pivot) ++i;
            while (v[j] > pivot) --j;
            if (i <= j) { const float t = v[i]; v[i] = v[j]; v[j] = t; ++i; --j; }
        }
        if (k <= j) hi = j;
        else if (k >= i) lo = i;
        else break;
    }
    return v[k];
}

double compute_error_distrib(const void *buf1, const void *buf2, int count, data_type_t dtype) {
    if (count <= 0) return 0.0;
    const char *out = getenv("METRIC_ERROR_DISTRIB_OUTPUT");
    if (!out) out = "error_distrib.txt";
    const size_t bytes = (size_t)count * get_element_size(dtype);
    float *err = (float *)malloc((size_t)count * sizeof(float));
    double mx = 0.0;
    if (!err) {
        METRIC_FOR_EACH(buf1, buf2, count, dtype, a, b, { const double d = fabs(a - b); if (d > mx) mx = d; });
        FILE *f = fopen(out, "a");
        if (f) { fprintf(f, "Max=%.6e  msg_bytes=%zu\n", mx, bytes); fclose(f); }
        return -1.0;
    }
    int n = 0;
    METRIC_FOR_EACH(buf1, buf2, count, dtype, a, b, { const double d = fabs(a - b); if (d > mx) mx = d; err[n++] = (float)d; });
    const int c = count - 1;
    const double p50 = kth(err, count, (int)(0.50 * c)), p95 = kth(err, count, (int)(0.95 * c));
    const double p99 = kth(err, count, (int)(0.99 * c)), p999 = kth(err, count, (int)(0.999 * c));
    FILE *f = fopen(out, "a");
    if (f) {
        fprintf(f, "P50=%.6e  P95=%.6e  P99=%.6e  P99.9=%.6e  Max=%.6e  msg_bytes=%zu\n", p50, p95, p99, p999, mx, bytes);
        fclose(f);
    }
    free(err);
    return p50;
}

/* Mean absolute error: (1/n) * sum |user_i - expected_i|, accumulated with Neumaier's
 * compensated sum so that a gigabyte of small differences does not lose its low bits. */
#include "metric_iter.h"

static inline void neumaier_add(double *total, double *lost, double term) {
    const double next = *total + term;
    *lost += fabs(*total) >= term ? (*total - next) + term : (term - next) + *total;
    *total = next;
}

double compute_mae(const void *user, const void *expected, int n, data_type_t kind) {
    double total = 0.0, lost = 0.0;
    if (n <= 0) return total;
    METRIC_FOR_EACH(user, expected, n, kind, got, want, neumaier_add(&total, &lost, fabs(got - want)));
    return (total + lost) / (double)n;
}

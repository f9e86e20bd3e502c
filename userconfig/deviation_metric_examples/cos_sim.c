/* Cosine similarity; 1 when both vectors are zero, 0 when exactly one is. */
#include "metric_iter.h"
double compute_cos_sim(const void *buf1, const void *buf2, int count, data_type_t dtype) {
    if (count <= 0) return 0.0;
    double ab = 0.0, aa = 0.0, bb = 0.0;
    METRIC_FOR_EACH(buf1, buf2, count, dtype, a, b, { ab += a * b; aa += a * a; bb += b * b; });
    if (aa == 0.0 && bb == 0.0) return 1.0;
    if (aa == 0.0 || bb == 0.0) return 0.0;
    return ab / (sqrt(aa) * sqrt(bb));
}

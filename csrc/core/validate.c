/* Correctness check and metric dispatch.
 *
 * The reference loads its registry only from bin/libs/validation.so
 * (run_codes/benchmark-core/src/validation.c:21-51). Here that file, when present
 * ($BENCH_DIR/bin/libs/validation.so, then ./bin/libs/validation.so), overrides a
 * registry that is compiled in, so the benchmarks also work before
 * scripts/register_metrics.sh has been run. Bit positions are the alphabetical order
 * of the metric names in both cases (scripts/register_metrics.sh:58). */
#define _GNU_SOURCE
#include <dlfcn.h>
#include <math.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include "validation.h"

#define DECL(n) double compute_##n(const void *, const void *, int, data_type_t)
DECL(cos_sim); DECL(error_distrib); DECL(mae); DECL(max_abs_err); DECL(mse); DECL(psnr); DECL(rel_l2);
DECL(relative_err); DECL(rmse); DECL(ssim);

static metric_entry_t builtin_registry[] = {
    {"cos_sim", compute_cos_sim},         {"error_distrib", compute_error_distrib},
    {"mae", compute_mae},                 {"max_abs_err", compute_max_abs_err},
    {"mse", compute_mse},                 {"psnr", compute_psnr},
    {"rel_l2", compute_rel_l2},           {"relative_err", compute_relative_err},
    {"rmse", compute_rmse},               {"ssim", compute_ssim},
};

static metric_entry_t *g_reg = NULL;
static int g_reg_n = 0;
static void *g_so = NULL;

int init_validation_so(void) {
    if (g_reg) return 0;
    char path[4096];
    const char *bd = getenv("BENCH_DIR");
    if (!getenv("CCB_BUILTIN_METRICS")) {
        if (bd) {
            snprintf(path, sizeof(path), "%s/bin/libs/validation.so", bd);
            g_so = dlopen(path, RTLD_NOW | RTLD_LOCAL);
        }
        if (!g_so) g_so = dlopen("bin/libs/validation.so", RTLD_NOW | RTLD_LOCAL);
    }
    if (g_so) {
        metric_entry_t *r = (metric_entry_t *)dlsym(g_so, "g_metric_registry");
        int *n = (int *)dlsym(g_so, "g_metric_registry_count");
        if (r && n && *n > 0) {
            g_reg = r;
            g_reg_n = *n > MAX_METRICS ? MAX_METRICS : *n;
            return 0;
        }
        dlclose(g_so);
        g_so = NULL;
    }
    g_reg = builtin_registry;
    g_reg_n = (int)(sizeof(builtin_registry) / sizeof(builtin_registry[0]));
    return 0;
}

int validation_registry_count(void) {
    init_validation_so();
    return g_reg_n;
}
const char *validation_metric_name(int idx) {
    init_validation_so();
    return (idx >= 0 && idx < g_reg_n) ? g_reg[idx].name : "";
}

size_t get_element_size(data_type_t dtype) {
    switch (dtype) {
        case TYPE_INT: return sizeof(int);
        case TYPE_FLOAT: return sizeof(float);
        case TYPE_DOUBLE: return sizeof(double);
        case TYPE_BFLOAT16: case TYPE_HALF: return 2;
        default: return 1;
    }
}

double to_double(const void *ptr, data_type_t dtype, int index) {
    switch (dtype) {
        case TYPE_INT: return (double)((const int *)ptr)[index];
        case TYPE_FLOAT: return (double)((const float *)ptr)[index];
        case TYPE_DOUBLE: return ((const double *)ptr)[index];
        case TYPE_BFLOAT16: return (double)ccb_bf16_to_float(((const uint16_t *)ptr)[index]);
        case TYPE_HALF: return (double)ccb_half_to_float(((const uint16_t *)ptr)[index]);
        default: return (double)((const char *)ptr)[index];
    }
}

int buffers_equal(const void *buf1, const void *buf2, int count, data_type_t datatype, double tolerance) {
    if (count <= 0) return 1;
    if (datatype == TYPE_FLOAT) {
        const float *a = (const float *)buf1, *b = (const float *)buf2;
        for (int i = 0; i < count; ++i)
            if (!(fabs((double)a[i] - (double)b[i]) <= tolerance)) return 0;
        return 1;
    }
    if (datatype == TYPE_DOUBLE) {
        const double *a = (const double *)buf1, *b = (const double *)buf2;
        for (int i = 0; i < count; ++i)
            if (!(fabs(a[i] - b[i]) <= tolerance)) return 0;
        return 1;
    }
    if (datatype == TYPE_BFLOAT16 || datatype == TYPE_HALF) {
        for (int i = 0; i < count; ++i)
            if (!(fabs(to_double(buf1, datatype, i) - to_double(buf2, datatype, i)) <= tolerance)) return 0;
        return 1;
    }
    return memcmp(buf1, buf2, (size_t)count * get_element_size(datatype)) == 0;
}

uint32_t parse_metric_mask(const char *str) {
    init_validation_so();
    if (!str || !*str) return 0;
    uint32_t mask = 0;
    char *copy = strdup(str), *save = NULL;
    for (char *tok = strtok_r(copy, ",", &save); tok; tok = strtok_r(NULL, ",", &save)) {
        while (*tok == ' ') ++tok;
        if (strcmp(tok, "all") == 0) {
            mask |= g_reg_n >= 32 ? 0xffffffffu : ((1u << g_reg_n) - 1u);
            continue;
        }
        int hit = 0;
        for (int i = 0; i < g_reg_n; ++i)
            if (strcmp(tok, g_reg[i].name) == 0) {
                mask |= 1u << i;
                hit = 1;
            }
        if (!hit) fprintf(stderr, "[validation] unknown metric '%s' ignored\n", tok);
    }
    free(copy);
    return mask;
}

validation_result_t validate_result(const void *user_buf, const void *reference_buf, int count, data_type_t dtype,
                                    double tolerance, uint32_t metrics_mask) {
    init_validation_so();
    validation_result_t r;
    memset(&r, 0, sizeof(r));
    r.num_elements = (size_t)(count > 0 ? count : 0);
    r.correct = buffers_equal(user_buf, reference_buf, count, dtype, tolerance);
    for (int i = 0; i < g_reg_n && i < MAX_METRICS; ++i)
        if (metrics_mask & (1u << i)) r.values[i] = g_reg[i].func(user_buf, reference_buf, count, dtype);
    return r;
}

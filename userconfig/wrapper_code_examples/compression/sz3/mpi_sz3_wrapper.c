/* SZ3 compression wrapper for the MPI path: strong mpi_compress / mpi_decompress, 1-D.
 *
 * As the reference's wrapper (userconfig/wrapper_code_examples/compression/sz3/
 * mpi_sz3_wrapper.c): the SZ3 C library is looked up at first use with dlopen under the
 * names libSZ3c.so, libSZ3.so, libsz3c.so, libsz3.so (:57-101) and driven through its
 * SZ_compress_args / SZ_decompress entry points with the data as one dimension (:138-218).
 * Environment (:106-133): MPI_SZ3_TYPE 0 = float (default), 1 = double ("float" / "double"
 * are accepted too); MPI_SZ3_EB_MODE 0 = absolute (default), 1 = relative to the value
 * range; MPI_SZ3_ABS_EB (1e-6); MPI_SZ3_REL_EB (0.01).
 *
 * Where no SZ3 library can be loaded the reference fails every call; this wrapper then
 * uses the in-tree error-bounded CPU codec (../sz_cpu/mpi_szcpu_wrapper.c: quantise under
 * the bound, previous-value prediction, bit planes), which honours the same four
 * variables. MPI_SZ3_FORCE_BUILTIN=1 skips the library. Both ends of a transfer must make
 * the same choice: the library's stream is its own raw blob, as in the reference. */
#define _GNU_SOURCE
#include <dlfcn.h>
#include <stdio.h>

#define SZCPU_NO_HOOKS
#include "../sz_cpu/mpi_szcpu_wrapper.c"

typedef unsigned char *(*sz3_compress_fn)(int, void *, size_t *, int, double, double, double, size_t, size_t, size_t, size_t, size_t);
typedef void *(*sz3_decompress_fn)(int, unsigned char *, size_t, size_t, size_t, size_t, size_t, size_t);
static sz3_compress_fn lib_compress;
static sz3_decompress_fn lib_decompress;

/* 1 when the library is usable; looked up once. */
static int have_library(void) {
    static int state; /* 0 = not tried, 1 = loaded, -1 = absent */
    if (state) return state > 0;
    state = -1;
    const char *force = getenv("MPI_SZ3_FORCE_BUILTIN");
    if (force && *force == '1') return 0;
    static const char *const names[] = {"libSZ3c.so", "libSZ3.so", "libsz3c.so", "libsz3.so"};
    for (unsigned i = 0; i < sizeof(names) / sizeof(names[0]); ++i) {
        void *h = dlopen(names[i], RTLD_NOW | RTLD_GLOBAL);
        if (!h) continue;
        lib_compress = (sz3_compress_fn)dlsym(h, "SZ_compress_args");
        lib_decompress = (sz3_decompress_fn)dlsym(h, "SZ_decompress");
        if (lib_compress && lib_decompress) {
            fprintf(stderr, "[SZ3 wrapper] loaded %s\n", names[i]);
            state = 1;
            return 1;
        }
        dlclose(h);
    }
    fprintf(stderr, "[SZ3 wrapper] no SZ3 library found: using the built-in error-bounded codec\n");
    return 0;
}

typedef struct { int dbl, rel; double abs_eb, rel_eb; } sz3_cfg;
static sz3_cfg config(void) {
    sz3_cfg c = {0, 0, 1e-6, 0.01};
    const char *e;
    if ((e = getenv("MPI_SZ3_TYPE"))) c.dbl = !strcasecmp(e, "double") || atoi(e) == 1;
    if ((e = getenv("MPI_SZ3_EB_MODE"))) c.rel = atoi(e) == 1 || !strcasecmp(e, "rel");
    if ((e = getenv("MPI_SZ3_ABS_EB")) && atof(e) > 0) c.abs_eb = atof(e);
    if ((e = getenv("MPI_SZ3_REL_EB")) && atof(e) > 0) c.rel_eb = atof(e);
    return c;
}

/* The codec with explicit parameters: the hooks below call it with the environment's
 * configuration, the ZCCL codec variant (../sz3_for_zccl) with the bound ZCCL passes. */
static int sz3_encode(sz3_cfg c, void *input, size_t input_size, void *output, size_t *output_size) {
    const size_t es = c.dbl ? 8 : 4, n = input_size / es;
    if (n == 0) return -1;
    if (have_library()) {
        size_t got = n;
        unsigned char *blob = lib_compress(c.dbl ? 1 : 0, input, &got, c.rel ? 1 : 0, c.abs_eb, c.rel_eb, 0.0, 0, 0, 0, 0, n);
        if (!blob) return -1;
        const int fits = got <= *output_size;
        if (fits) {
            memcpy(output, blob, got);
            *output_size = got;
        }
        free(blob);
        return fits ? 0 : -1;
    }
    double eb = c.abs_eb;
    if (c.rel) { /* relative to the value range of this buffer, as SZ3's REL mode */
        double lo = INFINITY, hi = -INFINITY;
        for (size_t i = 0; i < n; ++i) {
            const double x = c.dbl ? ((double *)input)[i] : (double)((float *)input)[i];
            if (x < lo) lo = x;
            if (x > hi) hi = x;
        }
        eb = (hi > lo) ? c.rel_eb * (hi - lo) : c.abs_eb;
    }
    return szcpu_compress(input, input_size, output, output_size, eb, c.dbl);
}

static int sz3_decode(sz3_cfg c, void *input, size_t input_size, void *output, size_t output_size) {
    if (have_library()) {
        const size_t n = output_size / (c.dbl ? 8 : 4);
        void *vals = lib_decompress(c.dbl ? 1 : 0, (unsigned char *)input, input_size, 0, 0, 0, 0, n);
        if (!vals) return -1;
        memcpy(output, vals, output_size);
        free(vals);
        return 0;
    }
    return szcpu_decompress(input, input_size, output, output_size, c.dbl);
}

#ifndef SZ3_NO_HOOKS
int mpi_compress(void *input, size_t input_size, void *output, size_t *output_size) {
    if (!input || !output || !output_size) return -1;
    if (input_size == 0) {
        *output_size = 0;
        return 0;
    }
    return sz3_encode(config(), input, input_size, output, output_size);
}
int mpi_decompress(void *input, size_t input_size, void *output, size_t output_size) {
    if (!input || !output) return -1;
    if (input_size == 0 || output_size == 0) return 0;
    return sz3_decode(config(), input, input_size, output, output_size);
}
#endif

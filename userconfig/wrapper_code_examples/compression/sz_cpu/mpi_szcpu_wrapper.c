/* Compression wrapper for the MPI path: error-bounded 1-D codec on the CPU, the
 * scalar restatement of the GPU codec in csrc/kernels/ccb_sz.cu (pre-quantise under
 * an absolute bound, first-order Lorenzo = previous-value prediction on the integers,
 * zig-zag, per-group-of-32 bit width and bit planes). Strong mpi_compress /
 * mpi_decompress; environment as the reference's SZ3 hook
 * (userconfig/wrapper_code_examples/compression/sz3/mpi_sz3_wrapper.c:106-133):
 * MPI_SZ3_ABS_EB (default 1e-6), MPI_SZ3_TYPE = float | double.
 * Layout: [u32 count][f64 step][per group: u8 width, width x u32 planes]. */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#include <strings.h>

static double abs_eb(void) {
    const char *e = getenv("MPI_SZ3_ABS_EB");
    double v = e ? atof(e) : 1e-6;
    return v > 0 ? v : 1e-6;
}
static int is_double(void) {
    const char *e = getenv("MPI_SZ3_TYPE");
    return e && !strcasecmp(e, "double");
}

/* The codec with explicit parameters (absolute bound, element type); the hooks below and
 * the SZ3 wrapper's fall-back path call it. */
static int szcpu_compress(void *input, size_t input_size, void *output, size_t *output_size, double eb, int dbl) {
    const size_t es = dbl ? 8 : 4, n = input_size / es;
    const double step = 2.0 * eb * (1.0 - 1.0 / 1024.0);
    unsigned char *out = (unsigned char *)output, *p = out + 12;
    const unsigned char *end = out + *output_size;
    if (*output_size < 12) return 1;
    uint32_t cnt = (uint32_t)n;
    memcpy(out, &cnt, 4);
    memcpy(out + 4, &step, 8);
    int64_t prev = 0;
    for (size_t g = 0; g < n; g += 32) {
        const size_t m = n - g < 32 ? n - g : 32;
        uint64_t u[32];
        uint64_t mx = 0;
        for (size_t i = 0; i < m; ++i) {
            const double x = dbl ? ((double *)input)[g + i] : (double)((float *)input)[g + i];
            if (!isfinite(x) || fabs(x / step) > 9.0e15) return 1; /* the caller falls back to raw bytes */
            const int64_t q = llrint(x / step);
            const int64_t d = q - prev;
            prev = q;
            u[i] = ((uint64_t)d << 1) ^ (uint64_t)(d >> 63);
            if (u[i] > mx) mx = u[i];
        }
        int w = 0;
        while (w < 64 && (mx >> w)) ++w;
        if (p + 1 + (size_t)w * 4 > end) return 1;
        *p++ = (unsigned char)w;
        for (int j = 0; j < w; ++j) { /* bit plane j of the group */
            uint32_t plane = 0;
            for (size_t i = 0; i < m; ++i) plane |= (uint32_t)((u[i] >> j) & 1u) << i;
            memcpy(p, &plane, 4);
            p += 4;
        }
    }
    const size_t tail = input_size - n * es;
    if (p + tail > end) return 1;
    memcpy(p, (char *)input + n * es, tail);
    *output_size = (size_t)(p - out) + tail;
    return 0;
}

static int szcpu_decompress(void *input, size_t input_size, void *output, size_t output_size, int dbl) {
    const size_t es = dbl ? 8 : 4;
    if (input_size < 12) return 1;
    const unsigned char *in = (const unsigned char *)input, *p = in + 12, *end = in + input_size;
    uint32_t cnt;
    double step;
    memcpy(&cnt, in, 4);
    memcpy(&step, in + 4, 8);
    const size_t n = cnt;
    if (n * es > output_size) return 1;
    int64_t prev = 0;
    for (size_t g = 0; g < n; g += 32) {
        const size_t m = n - g < 32 ? n - g : 32;
        if (p >= end) return 1;
        const int w = *p++;
        if (w > 64 || p + (size_t)w * 4 > end) return 1;
        uint64_t u[32] = {0};
        for (int j = 0; j < w; ++j) {
            uint32_t plane;
            memcpy(&plane, p, 4);
            p += 4;
            for (size_t i = 0; i < m; ++i) u[i] |= (uint64_t)((plane >> i) & 1u) << j;
        }
        for (size_t i = 0; i < m; ++i) {
            const int64_t d = (int64_t)(u[i] >> 1) ^ -(int64_t)(u[i] & 1u);
            prev += d;
            const double x = (double)prev * step;
            if (dbl) ((double *)output)[g + i] = x;
            else ((float *)output)[g + i] = (float)x;
        }
    }
    const size_t tail = output_size - n * es;
    if (tail && p + tail <= end) memcpy((char *)output + n * es, p, tail);
    return 0;
}

#ifndef SZCPU_NO_HOOKS
int mpi_compress(void *input, size_t input_size, void *output, size_t *output_size) {
    return szcpu_compress(input, input_size, output, output_size, abs_eb(), is_double());
}
int mpi_decompress(void *input, size_t input_size, void *output, size_t output_size) {
    return szcpu_decompress(input, input_size, output, output_size, is_double());
}
#endif

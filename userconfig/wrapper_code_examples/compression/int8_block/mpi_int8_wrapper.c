/* Compression wrapper for the MPI path: block-wise int8 with one fp32 absmax/127 scale
 * per block (MPI_INT8_BLOCK elements, default 128). Strong mpi_compress /
 * mpi_decompress: preload before the communication wrapper. The payload is treated
 * as fp32 (MPI_INT8_TYPE=double switches to fp64 input). Same arithmetic as the GPU
 * codec in csrc/kernels/ccb_codec.cuh; layout [u32 count][f32 scale x nblocks][i8 x count].
 * Takes the place of the reference's library-backed hooks
 * (userconfig/wrapper_code_examples/compression/sz3/mpi_sz3_wrapper.c,
 * zfp/mpi_zfp_wrapper.c), whose libraries are not available here. */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#include <strings.h>

static int block_size(void) {
    const char *e = getenv("MPI_INT8_BLOCK");
    int b = e ? atoi(e) : 128;
    return b > 0 ? b : 128;
}
static int is_double(void) {
    const char *e = getenv("MPI_INT8_TYPE");
    return e && !strcasecmp(e, "double");
}

int mpi_compress(void *input, size_t input_size, void *output, size_t *output_size) {
    const int dbl = is_double(), B = block_size();
    const size_t es = dbl ? 8 : 4, n = input_size / es, nb = (n + (size_t)B - 1) / (size_t)B;
    const size_t need = 4 + nb * 4 + n + (input_size - n * es);
    if (*output_size < need) return 1;
    unsigned char *out = (unsigned char *)output;
    uint32_t cnt = (uint32_t)n;
    memcpy(out, &cnt, 4);
    float *scales = (float *)(out + 4);
    int8_t *q = (int8_t *)(out + 4 + nb * 4);
    for (size_t b = 0; b < nb; ++b) {
        const size_t lo = b * (size_t)B, hi = lo + (size_t)B < n ? lo + (size_t)B : n;
        float m = 0.f;
        for (size_t i = lo; i < hi; ++i) {
            const float v = fabsf(dbl ? (float)((double *)input)[i] : ((float *)input)[i]);
            if (v > m) m = v;
        }
        const float inv = m > 0.f ? 127.f / m : 0.f;
        float s = m / 127.f;
        memcpy(&scales[b], &s, 4);
        for (size_t i = lo; i < hi; ++i) {
            const float v = dbl ? (float)((double *)input)[i] : ((float *)input)[i];
            q[i] = (int8_t)lrintf(v * inv);
        }
    }
    memcpy(q + n, (char *)input + n * es, input_size - n * es); /* bytes that do not make a whole element */
    *output_size = need;
    return 0;
}

int mpi_decompress(void *input, size_t input_size, void *output, size_t output_size) {
    const int dbl = is_double(), B = block_size();
    const size_t es = dbl ? 8 : 4;
    if (input_size < 4) return 1;
    uint32_t cnt;
    memcpy(&cnt, input, 4);
    const size_t n = cnt, nb = (n + (size_t)B - 1) / (size_t)B;
    if (n * es > output_size || 4 + nb * 4 + n > input_size) return 1;
    const unsigned char *in = (const unsigned char *)input;
    const int8_t *q = (const int8_t *)(in + 4 + nb * 4);
    for (size_t i = 0; i < n; ++i) {
        float s;
        memcpy(&s, in + 4 + (i / (size_t)B) * 4, 4);
        const float v = (float)q[i] * s;
        if (dbl) ((double *)output)[i] = v;
        else ((float *)output)[i] = v;
    }
    const size_t tail = output_size - n * es;
    if (tail && 4 + nb * 4 + n + tail <= input_size) memcpy((char *)output + n * es, q + n, tail);
    return 0;
}

/* Fixed-rate compression wrapper for the MPI path, at the path and with the environment
 * of the reference's ZFP wrapper (userconfig/wrapper_code_examples/compression/zfp/
 * mpi_zfp_wrapper.c:59-111: MPI_ZFP_TYPE float|double, MPI_ZFP_MODE, MPI_ZFP_RATE bits per
 * value, default 16). libzfp is not available here, so the codec is in this file: block
 * floating point. Every block of 64 values shares one exponent (the largest in the
 * block); each value keeps `rate` bits, sign included, of its mantissa aligned to that
 * exponent. Like ZFP's fixed-rate mode the output size depends only on the element count
 * and the rate, never on the data, and the error of a value is bounded by
 * 2^(block exponent - rate + 2). MPI_ZFP_MODE other than "rate" is accepted and treated
 * as fixed rate (precision / accuracy modes need the transform coder of the library).
 *
 * Layout: [u32 count][u8 rate][u8 type][u16 0] then per block [i16 exponent][packed codes],
 * codes little-endian bit-packed; trailing bytes that do not make a whole element follow
 * verbatim. Strong mpi_compress / mpi_decompress: preload before the communication wrapper. */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#include <strings.h>

#define ZBLOCK 64

static int cfg_rate(void) {
    const char *e = getenv("MPI_ZFP_RATE");
    int r = e ? atoi(e) : 16;
    if (r < 2) r = 2;
    if (r > 30) r = 30;
    return r;
}
static int cfg_double(void) {
    const char *e = getenv("MPI_ZFP_TYPE");
    return e && !strcasecmp(e, "double");
}
static size_t block_bytes(int rate) { return 2 + ((size_t)ZBLOCK * (size_t)rate + 7) / 8; }

static void put_bits(unsigned char *dst, size_t bitpos, uint32_t v, int nbits) {
    for (int b = 0; b < nbits; ++b, ++bitpos)
        if ((v >> b) & 1u) dst[bitpos >> 3] |= (unsigned char)(1u << (bitpos & 7));
}
static uint32_t get_bits(const unsigned char *src, size_t bitpos, int nbits) {
    uint32_t v = 0;
    for (int b = 0; b < nbits; ++b, ++bitpos) v |= (uint32_t)((src[bitpos >> 3] >> (bitpos & 7)) & 1u) << b;
    return v;
}

int mpi_compress(void *input, size_t input_size, void *output, size_t *output_size) {
    const int dbl = cfg_double(), rate = cfg_rate();
    const size_t es = dbl ? 8 : 4, n = input_size / es, nb = (n + ZBLOCK - 1) / ZBLOCK;
    const size_t tail = input_size - n * es, need = 8 + nb * block_bytes(rate) + tail;
    if (*output_size < need) return 1;
    unsigned char *out = (unsigned char *)output;
    memset(out, 0, need);
    const uint32_t cnt = (uint32_t)n;
    memcpy(out, &cnt, 4);
    out[4] = (unsigned char)rate;
    out[5] = (unsigned char)dbl;
    const int32_t qmax = (1 << (rate - 1)) - 1;
    for (size_t b = 0; b < nb; ++b) {
        const size_t lo = b * ZBLOCK, hi = lo + ZBLOCK < n ? lo + ZBLOCK : n;
        double m = 0.0;
        for (size_t i = lo; i < hi; ++i) {
            const double v = fabs(dbl ? ((double *)input)[i] : (double)((float *)input)[i]);
            if (v > m && isfinite(v)) m = v;
        }
        int e = 0;
        if (m > 0.0) (void)frexp(m, &e);             /* m = f * 2^e with f in [0.5, 1) */
        if (e > 32000) e = 32000;
        if (e < -32000) e = -32000;
        unsigned char *blk = out + 8 + b * block_bytes(rate);
        const int16_t e16 = (int16_t)e;
        memcpy(blk, &e16, 2);
        const double scale = ldexp(1.0, rate - 1 - e);   /* |v| < 2^e  ->  |v * scale| < 2^(rate-1) */
        for (size_t i = lo; i < hi; ++i) {
            double v = dbl ? ((double *)input)[i] : (double)((float *)input)[i];
            if (!isfinite(v)) v = 0.0;
            long q = lrint(v * scale);
            if (q > qmax) q = qmax;
            if (q < -qmax) q = -qmax;
            put_bits(blk + 2, (i - lo) * (size_t)rate, (uint32_t)q & ((1u << rate) - 1u), rate);
        }
    }
    memcpy(out + 8 + nb * block_bytes(rate), (char *)input + n * es, tail);
    *output_size = need;
    return 0;
}

int mpi_decompress(void *input, size_t input_size, void *output, size_t output_size) {
    if (input_size < 8) return 1;
    const unsigned char *in = (const unsigned char *)input;
    uint32_t cnt;
    memcpy(&cnt, in, 4);
    const int rate = in[4], dbl = in[5];
    if (rate < 2 || rate > 30) return 1;
    const size_t es = dbl ? 8 : 4, n = cnt, nb = (n + ZBLOCK - 1) / ZBLOCK;
    if (n * es > output_size || 8 + nb * block_bytes(rate) > input_size) return 1;
    for (size_t b = 0; b < nb; ++b) {
        const size_t lo = b * ZBLOCK, hi = lo + ZBLOCK < n ? lo + ZBLOCK : n;
        const unsigned char *blk = in + 8 + b * block_bytes(rate);
        int16_t e16;
        memcpy(&e16, blk, 2);
        const double inv = ldexp(1.0, (int)e16 - (rate - 1));
        for (size_t i = lo; i < hi; ++i) {
            uint32_t u = get_bits(blk + 2, (i - lo) * (size_t)rate, rate);
            int32_t q = (int32_t)(u << (32 - rate)) >> (32 - rate);   /* sign-extend */
            const double v = (double)q * inv;
            if (dbl) ((double *)output)[i] = v;
            else ((float *)output)[i] = (float)v;
        }
    }
    const size_t tail = output_size - n * es;
    if (tail && 8 + nb * block_bytes(rate) + tail <= input_size) memcpy((char *)output + n * es, in + 8 + nb * block_bytes(rate), tail);
    return 0;
}

/* ZFP compression wrapper for the MPI path: strong mpi_compress / mpi_decompress, 1-D.
 *
 * As the reference's wrapper (userconfig/wrapper_code_examples/compression/zfp/
 * mpi_zfp_wrapper.c): MPI_ZFP_TYPE selects the element type (zfp_type numbers: 3 = float,
 * the default, 4 = double; "float" / "double" are accepted too) and MPI_ZFP_MODE one of
 * the library's five modes (:59-111):
 *   1 expert       MPI_ZFP_MINBITS, MPI_ZFP_MAXBITS, MPI_ZFP_MAXPREC, MPI_ZFP_MINEXP
 *   2 fixed rate   MPI_ZFP_RATE bits per value (default 16)          [the default mode]
 *   3 precision    MPI_ZFP_PREC bit planes kept (default 10)
 *   4 accuracy     MPI_ZFP_TOL absolute tolerance (default 1e-3)
 *   5 reversible   lossless
 * The reference links libzfp; this wrapper looks it up at first use (dlopen of
 * libzfp.so / libzfp.so.1) and drives it the same way: a 1-D field over the caller's
 * buffer, the stream configured from the environment on both ends, the raw ZFP stream as
 * the payload. MPI_ZFP_FORCE_BUILTIN=1 skips the library.
 *
 * Without the library the codec below is used: block floating point. Every block of 64
 * values shares the exponent of its largest magnitude and each value keeps `bits` bits
 * (sign included) aligned to it, so a value's error is at most 2^(exponent - bits). The
 * five modes map onto how `bits` is chosen per block: rate = the same for all blocks
 * (output size independent of the data, like ZFP's fixed rate); precision = PREC + 1;
 * accuracy = just enough for 2^(exponent - bits) <= TOL (0 bits for blocks below the
 * tolerance); expert = accuracy with tolerance 2^MINEXP, capped by MAXPREC + 1 and by
 * MAXBITS / 64 per value; reversible = the raw bytes.
 * Layout: [u32 count][u8 mode][u8 type][u16 0], then per block [i16 exponent][u8 bits]
 * [packed codes, little-endian]; reversible: the raw values. Trailing bytes that do not
 * make a whole element follow verbatim. */
#define _GNU_SOURCE
#include <dlfcn.h>
#include <math.h>
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include <strings.h>

#define ZBLOCK 64

typedef struct {
    int mode, dbl;
    double rate, tol;
    unsigned prec, minbits, maxbits, maxprec;
    int minexp;
} zcfg;

static zcfg config(void) {
    zcfg c = {2, 0, 16.0, 1e-3, 10, 0, 0, 0, 0};
    const char *e;
    if ((e = getenv("MPI_ZFP_TYPE"))) c.dbl = !strcasecmp(e, "double") || atoi(e) == 4;
    if ((e = getenv("MPI_ZFP_MODE"))) {
        c.mode = atoi(e);
        if (!strcasecmp(e, "expert")) c.mode = 1;
        else if (!strcasecmp(e, "rate")) c.mode = 2;
        else if (!strcasecmp(e, "precision")) c.mode = 3;
        else if (!strcasecmp(e, "accuracy")) c.mode = 4;
        else if (!strcasecmp(e, "reversible")) c.mode = 5;
    }
    if ((e = getenv("MPI_ZFP_RATE"))) c.rate = atof(e);
    if ((e = getenv("MPI_ZFP_PREC"))) c.prec = (unsigned)atoi(e);
    if ((e = getenv("MPI_ZFP_TOL"))) c.tol = atof(e);
    if ((e = getenv("MPI_ZFP_MINBITS"))) c.minbits = (unsigned)atoi(e);
    if ((e = getenv("MPI_ZFP_MAXBITS"))) c.maxbits = (unsigned)atoi(e);
    if ((e = getenv("MPI_ZFP_MAXPREC"))) c.maxprec = (unsigned)atoi(e);
    if ((e = getenv("MPI_ZFP_MINEXP"))) c.minexp = atoi(e);
    return c;
}

/* ------------------------------------------------------------ libzfp, when present -- */
static struct {
    int state; /* 0 = not tried, 1 = loaded, -1 = absent */
    void *(*stream_open)(void *, size_t);
    void (*stream_close)(void *);
    void *(*zfp_stream_open)(void *);
    void (*zfp_stream_close)(void *);
    int (*set_params)(void *, unsigned, unsigned, unsigned, int);
    double (*set_rate)(void *, double, int, unsigned, int);
    unsigned (*set_precision)(void *, unsigned);
    double (*set_accuracy)(void *, double);
    void (*set_reversible)(void *);
    void *(*field_1d)(void *, int, size_t);
    void (*field_free)(void *);
    size_t (*compress)(void *, const void *);
    size_t (*decompress)(void *, void *);
} Z;

static int have_library(void) {
    if (Z.state) return Z.state > 0;
    Z.state = -1;
    const char *force = getenv("MPI_ZFP_FORCE_BUILTIN");
    if (force && *force == '1') return 0;
    static const char *const names[] = {"libzfp.so", "libzfp.so.1"};
    for (unsigned i = 0; i < 2; ++i) {
        void *h = dlopen(names[i], RTLD_NOW | RTLD_GLOBAL);
        if (!h) continue;
#define ZSYM(field, name) (*(void **)&Z.field = dlsym(h, name))
        ZSYM(stream_open, "stream_open");
        ZSYM(stream_close, "stream_close");
        ZSYM(zfp_stream_open, "zfp_stream_open");
        ZSYM(zfp_stream_close, "zfp_stream_close");
        ZSYM(set_params, "zfp_stream_set_params");
        ZSYM(set_rate, "zfp_stream_set_rate");
        ZSYM(set_precision, "zfp_stream_set_precision");
        ZSYM(set_accuracy, "zfp_stream_set_accuracy");
        ZSYM(set_reversible, "zfp_stream_set_reversible");
        ZSYM(field_1d, "zfp_field_1d");
        ZSYM(field_free, "zfp_field_free");
        ZSYM(compress, "zfp_compress");
        ZSYM(decompress, "zfp_decompress");
#undef ZSYM
        if (Z.stream_open && Z.stream_close && Z.zfp_stream_open && Z.zfp_stream_close && Z.set_params && Z.set_rate &&
            Z.set_precision && Z.set_accuracy && Z.set_reversible && Z.field_1d && Z.field_free && Z.compress && Z.decompress) {
            fprintf(stderr, "[ZFP wrapper] loaded %s\n", names[i]);
            Z.state = 1;
            return 1;
        }
        dlclose(h);
    }
    fprintf(stderr, "[ZFP wrapper] no ZFP library found: using the built-in block-floating-point codec\n");
    return 0;
}

static int lib_configure(void *zfp, const zcfg *c) {
    const int type = c->dbl ? 4 : 3; /* zfp_type_double, zfp_type_float */
    switch (c->mode) {
        case 1: return Z.set_params(zfp, c->minbits, c->maxbits, c->maxprec, c->minexp) ? 0 : -1;
        case 2: Z.set_rate(zfp, c->rate, type, 1, 0); return 0;
        case 3: Z.set_precision(zfp, c->prec); return 0;
        case 4: Z.set_accuracy(zfp, c->tol); return 0;
        case 5: Z.set_reversible(zfp); return 0;
        default: return -1;
    }
}

/* direction 0 = compress `data` (n values) into buf, 1 = decompress buf into `data` */
static long lib_run(int direction, void *buf, size_t buf_bytes, void *data, size_t n, const zcfg *c) {
    void *bs = Z.stream_open(buf, buf_bytes);
    void *zfp = bs ? Z.zfp_stream_open(bs) : NULL;
    void *field = (zfp && lib_configure(zfp, c) == 0) ? Z.field_1d(data, c->dbl ? 4 : 3, n) : NULL;
    size_t got = 0;
    if (field) got = direction ? Z.decompress(zfp, field) : Z.compress(zfp, field);
    if (field) Z.field_free(field);
    if (zfp) Z.zfp_stream_close(zfp);
    if (bs) Z.stream_close(bs);
    return got ? (long)got : -1;
}

/* --------------------------------------------------------------- the built-in codec -- */
static void put_bits(unsigned char *dst, size_t bitpos, uint32_t v, int nbits) {
    for (int b = 0; b < nbits; ++b, ++bitpos)
        if ((v >> b) & 1u) dst[bitpos >> 3] |= (unsigned char)(1u << (bitpos & 7));
}
static uint32_t get_bits(const unsigned char *src, size_t bitpos, int nbits) {
    uint32_t v = 0;
    for (int b = 0; b < nbits; ++b, ++bitpos) v |= (uint32_t)((src[bitpos >> 3] >> (bitpos & 7)) & 1u) << b;
    return v;
}
static int clampi(int v, int lo, int hi) { return v < lo ? lo : v > hi ? hi : v; }

/* Bits per value for a block whose largest magnitude is below 2^e. */
static int block_bits(const zcfg *c, int e) {
    switch (c->mode) {
        case 3: return clampi((int)c->prec + 1, 2, 30);
        case 4: {
            if (!(c->tol > 0)) return 30;
            int te;
            (void)frexp(c->tol, &te);          /* tol = f * 2^te, f in [0.5, 1): 2^(te-1) <= tol */
            /* rounding errs by at most 2^(e - bits), the clamp of a value that rounds up to
             * 2^e by at most 2^(e + 1 - bits): one extra bit keeps both within 2^(te-1) <= tol */
            const int need = e - (te - 1) + 1;
            return need <= 1 ? 0 : clampi(need, 2, 30);
        }
        case 1: {
            int bits = e - c->minexp + 1;      /* error at most 2^minexp, as in the accuracy mode */
            if (c->maxprec && bits > (int)c->maxprec + 1) bits = (int)c->maxprec + 1;
            if (c->maxbits && bits > (int)(c->maxbits / ZBLOCK)) bits = (int)(c->maxbits / ZBLOCK);
            if (c->minbits && bits < (int)((c->minbits + ZBLOCK - 1) / ZBLOCK)) bits = (int)((c->minbits + ZBLOCK - 1) / ZBLOCK);
            return bits <= 0 ? 0 : clampi(bits, 2, 30);
        }
        default: return clampi((int)lrint(c->rate), 2, 30);
    }
}
static size_t codes_bytes(int bits) { return ((size_t)ZBLOCK * (size_t)bits + 7) / 8; }

static int builtin_compress(const zcfg *c, void *input, size_t input_size, void *output, size_t *output_size) {
    const size_t es = c->dbl ? 8 : 4, n = input_size / es, nb = (n + ZBLOCK - 1) / ZBLOCK, tail = input_size - n * es;
    unsigned char *out = (unsigned char *)output, *p = out + 8;
    const unsigned char *end = out + *output_size;
    if (*output_size < 8) return 1;
    const uint32_t cnt = (uint32_t)n;
    memset(out, 0, 8);
    memcpy(out, &cnt, 4);
    out[4] = (unsigned char)c->mode;
    out[5] = (unsigned char)c->dbl;
    if (c->mode == 5) {
        if (p + input_size > end) return 1;
        memcpy(p, input, input_size);
        *output_size = 8 + input_size;
        return 0;
    }
    for (size_t b = 0; b < nb; ++b) {
        const size_t lo = b * ZBLOCK, hi = lo + ZBLOCK < n ? lo + ZBLOCK : n;
        double m = 0.0;
        for (size_t i = lo; i < hi; ++i) {
            const double v = fabs(c->dbl ? ((double *)input)[i] : (double)((float *)input)[i]);
            if (v > m && isfinite(v)) m = v;
        }
        int e = 0;
        if (m > 0.0) (void)frexp(m, &e); /* m = f * 2^e with f in [0.5, 1) */
        e = clampi(e, -32000, 32000);
        const int bits = m > 0.0 ? block_bits(c, e) : (c->mode == 2 ? block_bits(c, e) : 0);
        if (p + 3 + codes_bytes(bits) > end) return 1;
        const int16_t e16 = (int16_t)e;
        memcpy(p, &e16, 2);
        p[2] = (unsigned char)bits;
        p += 3;
        memset(p, 0, codes_bytes(bits));
        if (bits) {
            const int32_t qmax = (1 << (bits - 1)) - 1;
            const double scale = ldexp(1.0, bits - 1 - e); /* |v| < 2^e -> |v * scale| < 2^(bits-1) */
            for (size_t i = lo; i < hi; ++i) {
                double v = c->dbl ? ((double *)input)[i] : (double)((float *)input)[i];
                if (!isfinite(v)) v = 0.0;
                long q = lrint(v * scale);
                if (q > qmax) q = qmax;
                if (q < -qmax) q = -qmax;
                put_bits(p, (i - lo) * (size_t)bits, (uint32_t)q & ((1u << bits) - 1u), bits);
            }
        }
        p += codes_bytes(bits);
    }
    if (p + tail > end) return 1;
    memcpy(p, (char *)input + n * es, tail);
    *output_size = (size_t)(p - out) + tail;
    return 0;
}

static int builtin_decompress(void *input, size_t input_size, void *output, size_t output_size) {
    if (input_size < 8) return 1;
    const unsigned char *in = (const unsigned char *)input, *p = in + 8, *end = in + input_size;
    uint32_t cnt;
    memcpy(&cnt, in, 4);
    const int mode = in[4], dbl = in[5];
    const size_t es = dbl ? 8 : 4, n = cnt, nb = (n + ZBLOCK - 1) / ZBLOCK;
    if (n * es > output_size) return 1;
    if (mode == 5) {
        const size_t bytes = input_size - 8 < output_size ? input_size - 8 : output_size;
        memcpy(output, p, bytes);
        return 0;
    }
    for (size_t b = 0; b < nb; ++b) {
        const size_t lo = b * ZBLOCK, hi = lo + ZBLOCK < n ? lo + ZBLOCK : n;
        if (p + 3 > end) return 1;
        int16_t e16;
        memcpy(&e16, p, 2);
        const int bits = p[2];
        p += 3;
        if (bits > 30 || p + codes_bytes(bits) > end) return 1;
        const double inv = bits ? ldexp(1.0, (int)e16 - (bits - 1)) : 0.0;
        for (size_t i = lo; i < hi; ++i) {
            double v = 0.0;
            if (bits) {
                const uint32_t u = get_bits(p, (i - lo) * (size_t)bits, bits);
                v = (double)((int32_t)(u << (32 - bits)) >> (32 - bits)) * inv; /* sign-extend */
            }
            if (dbl) ((double *)output)[i] = v;
            else ((float *)output)[i] = (float)v;
        }
        p += codes_bytes(bits);
    }
    const size_t tail = output_size - n * es;
    if (tail && p + tail <= end) memcpy((char *)output + n * es, p, tail);
    return 0;
}

/* The codec with an explicit configuration (the hooks pass the environment's, the ZCCL
 * codec variant ../zfp_for_zccl the tolerance ZCCL asks for). */
static int zfp_encode(zcfg c, void *input, size_t input_size, void *output, size_t *output_size) {
    if (c.mode < 1 || c.mode > 5) return -1;
    if (have_library()) {
        const size_t n = input_size / (c.dbl ? 8 : 4);
        if (n == 0) return -1;
        const size_t cap = input_size + 1024; /* the library writes into a scratch stream first */
        void *buf = malloc(cap);
        if (!buf) return -1;
        const long got = lib_run(0, buf, cap, input, n, &c);
        const int ok = got > 0 && (size_t)got <= *output_size;
        if (ok) {
            memcpy(output, buf, (size_t)got);
            *output_size = (size_t)got;
        }
        free(buf);
        return ok ? 0 : -1;
    }
    return builtin_compress(&c, input, input_size, output, output_size);
}
static int zfp_decode(zcfg c, void *input, size_t input_size, void *output, size_t output_size) {
    if (have_library()) {
        const size_t n = output_size / (c.dbl ? 8 : 4);
        return (n && lib_run(1, input, input_size, output, n, &c) > 0) ? 0 : -1;
    }
    return builtin_decompress(input, input_size, output, output_size);
}

#ifndef ZFP_NO_HOOKS
int mpi_compress(void *input, size_t input_size, void *output, size_t *output_size) {
    if (!input || !output || !output_size) return -1;
    if (input_size == 0) {
        *output_size = 0;
        return 0;
    }
    return zfp_encode(config(), input, input_size, output, output_size);
}
int mpi_decompress(void *input, size_t input_size, void *output, size_t output_size) {
    if (!input || !output) return -1;
    if (input_size == 0 || output_size == 0) return 0;
    return zfp_decode(config(), input, input_size, output, output_size);
}
#endif

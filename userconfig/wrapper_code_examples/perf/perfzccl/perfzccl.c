/* perfzccl: perf wrapper for ZCCL runs (first in LD_PRELOAD). The MPI half is the MPI perf
 * wrapper (../perfmpi/perfmpi.c: point-to-point, the collectives, mpi_compress /
 * mpi_decompress); on top of it this file times the codec entry points ZCCL calls inside
 * its collectives, whoever defines them next in the chain (libZCCL itself, or a preloaded
 * sz3_for_zccl / zfp_for_zccl). Rows and columns as the reference's
 * userconfig/wrapper_code_examples/perf/perfzccl/perfzccl.c:65-262:
 *   ZCCL_compress, ZCCL_compress_mt, ZCCL_compress_chunk
 *       duration, input_bytes, output_bytes, compression_ratio (output / input), nbEle
 *   ZCCL_decompress_st, ZCCL_decompress_mt          duration, output_bytes, nbEle
 *   ZCCL_homoadd_st, ZCCL_homoadd_mt                duration, output_bytes, nbEle */
#include "../perfmpi/perfmpi.c"

#define ZNEXT(var, name) \
    if (!var) *(void **)&var = dlsym(RTLD_NEXT, name)

static void note_compress(const char *row, double t0, size_t n, const size_t *out_size) {
    const double in_bytes = (double)n * sizeof(float), out_bytes = out_size ? (double)*out_size : 0.0;
    ROW(row, t0, {"duration", perf_get_time() - t0}, {"input_bytes", in_bytes}, {"output_bytes", out_bytes},
        {"compression_ratio", in_bytes > 0 ? out_bytes / in_bytes : 1.0}, {"nbEle", (double)n});
}

void ZCCL_float_single_thread_arg(unsigned char *out, float *data, size_t *out_size, float eb, size_t n, int block) {
    static void (*next)(unsigned char *, float *, size_t *, float, size_t, int);
    ZNEXT(next, "ZCCL_float_single_thread_arg");
    if (!next) return;
    const double t0 = perf_get_time();
    next(out, data, out_size, eb, n, block);
    note_compress("ZCCL_compress", t0, n, out_size);
}
void ZCCL_float_openmp_threadblock_arg(unsigned char *out, float *data, size_t *out_size, float eb, size_t n, int block) {
    static void (*next)(unsigned char *, float *, size_t *, float, size_t, int);
    ZNEXT(next, "ZCCL_float_openmp_threadblock_arg");
    if (!next) return;
    const double t0 = perf_get_time();
    next(out, data, out_size, eb, n, block);
    note_compress("ZCCL_compress_mt", t0, n, out_size);
}
void ZCCL_float_single_thread_arg_split_record(unsigned char *out, float *data, size_t *out_size, float eb, size_t n, int block,
                                               unsigned char *chunk_arr, size_t chunk_iter) {
    static void (*next)(unsigned char *, float *, size_t *, float, size_t, int, unsigned char *, size_t);
    ZNEXT(next, "ZCCL_float_single_thread_arg_split_record");
    if (!next) return;
    const double t0 = perf_get_time();
    next(out, data, out_size, eb, n, block, chunk_arr, chunk_iter);
    note_compress("ZCCL_compress_chunk", t0, n, out_size);
}
unsigned char *ZCCL_float_openmp_threadblock(float *data, size_t *out_size, float eb, size_t n, int block) {
    static unsigned char *(*next)(float *, size_t *, float, size_t, int);
    ZNEXT(next, "ZCCL_float_openmp_threadblock");
    if (!next) return NULL;
    const double t0 = perf_get_time();
    unsigned char *r = next(data, out_size, eb, n, block);
    note_compress("ZCCL_compress_mt", t0, n, out_size);
    return r;
}
void ZCCL_float_decompress_single_thread_arg(float *out, size_t n, float eb, int block, unsigned char *in) {
    static void (*next)(float *, size_t, float, int, unsigned char *);
    ZNEXT(next, "ZCCL_float_decompress_single_thread_arg");
    if (!next) return;
    const double t0 = perf_get_time();
    next(out, n, eb, block, in);
    ROW("ZCCL_decompress_st", t0, {"duration", perf_get_time() - t0}, {"output_bytes", (double)n * sizeof(float)}, {"nbEle", (double)n});
}
void ZCCL_float_decompress_openmp_threadblock_arg(float *out, size_t n, float eb, int block, unsigned char *in) {
    static void (*next)(float *, size_t, float, int, unsigned char *);
    ZNEXT(next, "ZCCL_float_decompress_openmp_threadblock_arg");
    if (!next) return;
    const double t0 = perf_get_time();
    next(out, n, eb, block, in);
    ROW("ZCCL_decompress_mt", t0, {"duration", perf_get_time() - t0}, {"output_bytes", (double)n * sizeof(float)}, {"nbEle", (double)n});
}
void ZCCL_float_homomophic_add_single_thread(unsigned char *out, size_t *out_size, size_t n, float eb, int block, unsigned char *a,
                                             unsigned char *b) {
    static void (*next)(unsigned char *, size_t *, size_t, float, int, unsigned char *, unsigned char *);
    ZNEXT(next, "ZCCL_float_homomophic_add_single_thread");
    if (!next) return;
    const double t0 = perf_get_time();
    next(out, out_size, n, eb, block, a, b);
    ROW("ZCCL_homoadd_st", t0, {"duration", perf_get_time() - t0}, {"output_bytes", out_size ? (double)*out_size : 0.0}, {"nbEle", (double)n});
}
void ZCCL_float_homomophic_add_openmp_threadblock(unsigned char *out, size_t *out_size, size_t n, float eb, int block,
                                                  unsigned char *a, unsigned char *b) {
    static void (*next)(unsigned char *, size_t *, size_t, float, int, unsigned char *, unsigned char *);
    ZNEXT(next, "ZCCL_float_homomophic_add_openmp_threadblock");
    if (!next) return;
    const double t0 = perf_get_time();
    next(out, out_size, n, eb, block, a, b);
    ROW("ZCCL_homoadd_mt", t0, {"duration", perf_get_time() - t0}, {"output_bytes", out_size ? (double)*out_size : 0.0}, {"nbEle", (double)n});
}

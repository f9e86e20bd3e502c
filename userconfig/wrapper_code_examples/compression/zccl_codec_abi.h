/* The ten codec entry points ZCCL's collectives call internally, defined over any
 * error-bounded float codec, so that a preloaded library swaps ZCCL's own compressor for
 * another one. The symbol set and signatures are those the reference interposes
 * (userconfig/wrapper_code_examples/compression/sz3_for_zccl/sz3_for_zccl.c:172-307 and
 * zfp_for_zccl/zfp_for_zccl.c); every stream is framed as [size_t payload bytes][payload]
 * (:116-141) because ZCCL passes no size to its decompressors.
 *
 * The includer defines, before including this header,
 *   static size_t zabi_encode(const float *data, size_t n, float abs_eb, unsigned char *out, size_t cap);
 *       payload bytes written, 0 on failure
 *   static int    zabi_decode(float *out, size_t n, const unsigned char *in, size_t bytes);
 *       0 on success
 *   #define ZABI_TAG "name"      for messages
 * The reference aborts in the two "homomorphic add" entry points (adding two compressed
 * streams without decoding them is a property of ZCCL's own format); here they decode
 * both operands, add and re-encode under the same bound, so collectives that use them
 * still run, at the cost of one more quantisation. */
#ifndef CCB_ZCCL_CODEC_ABI_H
#define CCB_ZCCL_CODEC_ABI_H

#include <stdio.h>
#include <stdlib.h>
#include <string.h>

static size_t zabi_capacity(size_t n) { return n * sizeof(float) + n / 8 + 256; }

/* frame into `out` (which the caller sized); total bytes, 0 on failure */
static size_t zabi_frame(unsigned char *out, const float *data, size_t n, float eb) {
    const size_t got = zabi_encode(data, n, eb, out + sizeof(size_t), zabi_capacity(n));
    if (!got) {
        fprintf(stderr, "[" ZABI_TAG "] compression of %zu values failed\n", n);
        return 0;
    }
    memcpy(out, &got, sizeof(size_t));
    return got + sizeof(size_t);
}
static int zabi_unframe(float *out, size_t n, const unsigned char *in) {
    size_t bytes;
    memcpy(&bytes, in, sizeof(size_t));
    return zabi_decode(out, n, in + sizeof(size_t), bytes);
}

void ZCCL_float_openmp_threadblock_arg(unsigned char *outputBytes, float *oriData, size_t *outSize, float absErrBound,
                                       size_t nbEle, int blockSize) {
    (void)blockSize;
    *outSize = nbEle ? zabi_frame(outputBytes, oriData, nbEle, absErrBound) : 0;
}
void ZCCL_float_single_thread_arg(unsigned char *outputBytes, float *oriData, size_t *outSize, float absErrBound, size_t nbEle,
                                  int blockSize) {
    ZCCL_float_openmp_threadblock_arg(outputBytes, oriData, outSize, absErrBound, nbEle, blockSize);
}
void ZCCL_float_single_thread_arg_split_record(unsigned char *outputBytes, float *oriData, size_t *outSize, float absErrBound,
                                               size_t nbEle, int blockSize, unsigned char *chunk_arr, size_t chunk_iter) {
    (void)chunk_arr;
    (void)chunk_iter;
    ZCCL_float_openmp_threadblock_arg(outputBytes, oriData, outSize, absErrBound, nbEle, blockSize);
}
unsigned char *ZCCL_float_openmp_threadblock(float *oriData, size_t *outSize, float absErrBound, size_t nbEle, int blockSize) {
    (void)blockSize;
    *outSize = 0;
    if (!nbEle) return NULL;
    unsigned char *buf = (unsigned char *)malloc(zabi_capacity(nbEle) + sizeof(size_t));
    if (!buf) return NULL;
    *outSize = zabi_frame(buf, oriData, nbEle, absErrBound);
    if (!*outSize) {
        free(buf);
        return NULL;
    }
    return buf;
}
unsigned char *ZCCL_float_openmp_threadblock_randomaccess(float *oriData, size_t *outSize, float absErrBound, size_t nbEle,
                                                          int blockSize) {
    return ZCCL_float_openmp_threadblock(oriData, outSize, absErrBound, nbEle, blockSize);
}
void ZCCL_float_decompress_openmp_threadblock_arg(float *newData, size_t nbEle, float absErrBound, int blockSize,
                                                  unsigned char *cmpBytes) {
    (void)absErrBound;
    (void)blockSize;
    if (nbEle && zabi_unframe(newData, nbEle, cmpBytes)) fprintf(stderr, "[" ZABI_TAG "] decompression failed\n");
}
void ZCCL_float_decompress_single_thread_arg(float *newData, size_t nbEle, float absErrBound, int blockSize,
                                             unsigned char *cmpBytes) {
    ZCCL_float_decompress_openmp_threadblock_arg(newData, nbEle, absErrBound, blockSize, cmpBytes);
}
void ZCCL_float_decompress_openmp_threadblock(float **newData, size_t nbEle, float absErrBound, int blockSize,
                                              unsigned char *cmpBytes) {
    (void)absErrBound;
    (void)blockSize;
    if (!nbEle) {
        *newData = NULL;
        return;
    }
    if (!*newData) *newData = (float *)malloc(nbEle * sizeof(float)); /* ZCCL's own version allocates too */
    if (*newData && zabi_unframe(*newData, nbEle, cmpBytes)) fprintf(stderr, "[" ZABI_TAG "] decompression failed\n");
}
void ZCCL_float_homomophic_add_openmp_threadblock(unsigned char *final_cmpBytes, size_t *final_cmpSize, size_t nbEle,
                                                  float absErrBound, int blockSize, unsigned char *cmpBytes,
                                                  unsigned char *cmpBytes2) {
    (void)blockSize;
    *final_cmpSize = 0;
    if (!nbEle) return;
    float *a = (float *)malloc(nbEle * sizeof(float)), *b = (float *)malloc(nbEle * sizeof(float));
    if (a && b && !zabi_unframe(a, nbEle, cmpBytes) && !zabi_unframe(b, nbEle, cmpBytes2)) {
        for (size_t i = 0; i < nbEle; ++i) a[i] += b[i];
        *final_cmpSize = zabi_frame(final_cmpBytes, a, nbEle, absErrBound);
    }
    free(a);
    free(b);
}
void ZCCL_float_homomophic_add_single_thread(unsigned char *final_cmpBytes, size_t *final_cmpSize, size_t nbEle, float absErrBound,
                                             int blockSize, unsigned char *cmpBytes, unsigned char *cmpBytes2) {
    ZCCL_float_homomophic_add_openmp_threadblock(final_cmpBytes, final_cmpSize, nbEle, absErrBound, blockSize, cmpBytes, cmpBytes2);
}
#endif

/* SZ3 in place of ZCCL's own compressor: a preloaded library that defines the codec entry
 * points ZCCL's collectives call (../zccl_codec_abi.h), backed by the SZ3 wrapper's codec
 * (../sz3/mpi_sz3_wrapper.c: libSZ3 when it can be loaded, else the built-in error-bounded
 * codec). Role and environment of the reference's file of the same name
 * (userconfig/wrapper_code_examples/compression/sz3_for_zccl/sz3_for_zccl.c:98-104):
 * SZ3_EB_MODE (0 absolute, 1 relative), SZ3_ABS_EB (overrides the bound ZCCL passes when
 * positive), SZ3_REL_EB, SZ3_VERBOSE. */
#define SZ3_NO_HOOKS
#include "../sz3/mpi_sz3_wrapper.c"

static size_t zabi_encode(const float *data, size_t n, float abs_eb, unsigned char *out, size_t cap) {
    sz3_cfg c = {0, 0, (double)abs_eb, 0.01};
    const char *e;
    if ((e = getenv("SZ3_EB_MODE"))) c.rel = atoi(e) == 1;
    if ((e = getenv("SZ3_ABS_EB")) && atof(e) > 0) c.abs_eb = atof(e);
    if ((e = getenv("SZ3_REL_EB")) && atof(e) > 0) c.rel_eb = atof(e);
    if (!(c.abs_eb > 0)) c.abs_eb = 1e-6;
    size_t got = cap;
    if (sz3_encode(c, (void *)data, n * sizeof(float), out, &got) != 0) return 0;
    if (getenv("SZ3_VERBOSE")) fprintf(stderr, "[sz3_for_zccl] %zu values -> %zu bytes (bound %g)\n", n, got, c.abs_eb);
    return got;
}
static int zabi_decode(float *out, size_t n, const unsigned char *in, size_t bytes) {
    const sz3_cfg c = {0, 0, 1e-6, 0.01};
    return sz3_decode(c, (void *)in, bytes, out, n * sizeof(float));
}
#define ZABI_TAG "sz3_for_zccl"
#include "../zccl_codec_abi.h"

/* ZFP in place of ZCCL's own compressor: a preloaded library that defines the codec entry
 * points ZCCL's collectives call (../zccl_codec_abi.h), backed by the ZFP wrapper's codec
 * (../zfp/mpi_zfp_wrapper.c: libzfp when it can be loaded, else the built-in block
 * floating point). Role and environment of the reference's file of the same name
 * (userconfig/wrapper_code_examples/compression/zfp_for_zccl/zfp_for_zccl.c:66-74):
 * ZFP_MODE (2 rate, 3 precision, 4 accuracy = default here, 5 reversible), ZFP_RATE,
 * ZFP_PREC, ZFP_TOL (overrides the bound ZCCL passes when positive), ZFP_VERBOSE. In the
 * accuracy mode the tolerance is the absolute bound of the ZCCL call. The stream is
 * self-describing with the built-in codec; with libzfp the decoder is configured from the
 * same variables, as in the MPI wrapper. */
#define ZFP_NO_HOOKS
#include "../zfp/mpi_zfp_wrapper.c"

static zcfg zccl_cfg(float abs_eb) {
    zcfg c = {4, 0, 16.0, (double)abs_eb, 10, 0, 0, 0, 0};
    const char *e;
    if ((e = getenv("ZFP_MODE")) && atoi(e) >= 1 && atoi(e) <= 5) c.mode = atoi(e);
    if ((e = getenv("ZFP_RATE"))) c.rate = atof(e);
    if ((e = getenv("ZFP_PREC"))) c.prec = (unsigned)atoi(e);
    if ((e = getenv("ZFP_TOL")) && atof(e) > 0) c.tol = atof(e);
    if (!(c.tol > 0)) c.tol = 1e-3;
    return c;
}
static size_t zabi_encode(const float *data, size_t n, float abs_eb, unsigned char *out, size_t cap) {
    const zcfg c = zccl_cfg(abs_eb);
    size_t got = cap;
    if (zfp_encode(c, (void *)data, n * sizeof(float), out, &got) != 0) return 0;
    if (getenv("ZFP_VERBOSE")) fprintf(stderr, "[zfp_for_zccl] %zu values -> %zu bytes (mode %d)\n", n, got, c.mode);
    return got;
}
static int zabi_decode(float *out, size_t n, const unsigned char *in, size_t bytes) {
    return zfp_decode(zccl_cfg(0.f), (void *)in, bytes, out, n * sizeof(float));
}
#define ZABI_TAG "zfp_for_zccl"
#include "../zccl_codec_abi.h"

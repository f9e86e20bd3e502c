"""Numeric constants shared with include/ccb/ccb_types.h."""
F32, BF16, F16 = 0, 1, 2
CODEC_NONE, CODEC_INT8, CODEC_FP8, CODEC_INT8_G256, CODEC_INT4 = 0, 1, 2, 3, 4
OP_SUM, OP_PROD, OP_MAX, OP_MIN = 0, 1, 2, 3
ALGO_AUTO, ALGO_TWOSHOT, ALGO_ONESHOT, ALGO_RING, ALGO_TREE, ALGO_NVLS = 0, 1, 2, 3, 4, 5
OK, ERR_ARG, ERR_CUDA, ERR_BOOTSTRAP, ERR_TIMEOUT, ERR_UNSUPPORTED, ERR_CAPACITY = range(7)

CODECS = {"none": CODEC_NONE, "int8": CODEC_INT8, "fp8": CODEC_FP8, "int8_g256": CODEC_INT8_G256, "int4": CODEC_INT4}
ALGOS = {"auto": ALGO_AUTO, "twoshot": ALGO_TWOSHOT, "oneshot": ALGO_ONESHOT, "ring": ALGO_RING,
         "tree": ALGO_TREE, "nvls": ALGO_NVLS}
OPS = {"sum": OP_SUM, "prod": OP_PROD, "max": OP_MAX, "min": OP_MIN}

__all__ = [n for n in dir() if n.isupper()]

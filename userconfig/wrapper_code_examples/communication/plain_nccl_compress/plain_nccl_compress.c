/* Compressed NCCL collectives as a wrapper built from source (selection mode 2 or 3).
 *
 * The reference keeps its int8 NCCL wrapper at this path
 * (userconfig/wrapper_code_examples/communication/plain_nccl_compress/plain_nccl_compress.cu:
 * quantise kernel, ncclSend / ncclRecv ring, dequantise, reduce, a host synchronisation per
 * hop). A configuration that names this directory in `source_dirs` gets the same role here:
 * the interposer over the fused sm_100a kernels of libccb.so, which the wrapper builder links
 * in because this source uses the ccb API. The code is csrc/interpose/ccb_nccl_interpose.c
 * (also shipped prebuilt as bin/libs/libccb_nccl.so); the environment is the reference's
 * (NCCL_COMPRESS_DISABLE, NCCL_COMPRESS_GROUP = 128 or 256) plus CCB_CODEC, CCB_ALGO,
 * CCB_MOVE_CODEC, CCB_P2P_CODEC, CCB_MIN_BYTES, CCB_ERROR_FEEDBACK. */
#include "ccb/ccb.h"
#include "../../../../csrc/interpose/ccb_nccl_interpose.c"

/* Shared by the lossless hook library (dietgpu.c) and anything else that drives the lossless
 * float codec of libccb through NCCL element types: the map from ncclDataType_t to the
 * codec's element types and their sizes. (The reference's header of this name maps the same
 * NCCL types to the external DietGPU library's enum.) */
#ifndef DIETGPU_COMMON_H
#define DIETGPU_COMMON_H

#include <cuda_runtime.h>
#include <nccl.h>
#include <stddef.h>

#include "ccb/ccb.h"
#include "ccb/ccb_lossless.h"

/* CCB_F32 / CCB_F16 / CCB_BF16, or -1 for a type the codec does not take. */
static inline int lossless_dtype_of(ncclDataType_t t) {
    if (t == ncclFloat32) return CCB_F32;
    if (t == ncclFloat16) return CCB_F16;
    if ((int)t == 9) return CCB_BF16; /* ncclBfloat16, spelled differently across NCCL versions */
    return -1;
}
static inline size_t lossless_elem_bytes(int dtype) { return dtype == CCB_F32 ? 4 : 2; }

#endif

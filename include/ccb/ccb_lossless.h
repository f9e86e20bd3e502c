/* Lossless float codec of libccb.so (csrc/kernels/ccb_lossless.cu): f32, bf16 and f16
 * buffers on the current device, bit-exact round trip. The container is
 *   [32-byte header: u32 magic "CCBL", u32 dtype, u64 count, u64 used bytes, u64 0]
 *   [one slot per 4096 values, at a fixed stride of 32 + 4096 * sizeof(element) bytes]
 * and a slot is [u32 used][u8 width x 8][u8 minimum exponent x 8][12 x 0]
 * [sign and mantissa, raw planes][exponent - minimum of each 512-value block, width planes].
 * Role in the reference: the external DietGPU float codec behind the compression hooks
 * (userconfig/wrapper_code_examples/compression/dietgpu/dietgpu.cu:32-103). */
#ifndef CCB_LOSSLESS_H
#define CCB_LOSSLESS_H

#include <stdint.h>

#include "ccb.h"

#ifdef __cplusplus
extern "C" {
#endif

/* Capacity a container of `count` elements needs (raw size + 32 bytes per 4096 values + 32). */
uint64_t ccb_lossless_max_bytes(int dtype, uint64_t count);
/* `out` must be 16-byte aligned and hold ccb_lossless_max_bytes() bytes. One kernel. */
int ccb_lossless_encode(int dtype, const void* in, uint64_t count, void* out, ccb_stream_t stream);
/* out = decoded values, or out += decoded values (in the element type) when accumulate != 0. */
int ccb_lossless_decode(int dtype, const void* in, uint64_t count, void* out, int accumulate, ccb_stream_t stream);
/* Bytes that carry information: the header plus the used prefix of every slot. Synchronises `stream`. */
int ccb_lossless_used_bytes(const void* comp, uint64_t* bytes, ccb_stream_t stream);

#ifdef __cplusplus
}
#endif
#endif

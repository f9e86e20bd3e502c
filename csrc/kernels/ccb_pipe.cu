// Instantiations of the pipelined two-shot kernel (ccb_pipe.cuh), in a translation unit
// of their own so that they compile beside the rest of the runtime: one kernel per
// element type and codec.
#include "../rt/ccb_rt_internal.h"
#include "ccb_pipe.cuh"

namespace ccb {

static_assert(kPipeChunkElems == kPipeChunkUnits * kWarpElems, "the host sizes grids in chunks of this many elements");

template <class T>
static const void* by_codec(int codec) {
  switch (codec) {
    case CCB_CODEC_NONE: return reinterpret_cast<const void*>(&pipe_kernel<T, CodecNone<T>>);
    case CCB_CODEC_INT8: return reinterpret_cast<const void*>(&pipe_kernel<T, CodecInt8<128>>);
    case CCB_CODEC_FP8: return reinterpret_cast<const void*>(&pipe_kernel<T, CodecFp8>);
    case CCB_CODEC_INT8_G256: return reinterpret_cast<const void*>(&pipe_kernel<T, CodecInt8<256>>);
    case CCB_CODEC_INT4: return reinterpret_cast<const void*>(&pipe_kernel<T, CodecInt4>);
    default: return nullptr;
  }
}

const void* pipe_kernel_fn(int dtype, int codec) {
  switch (dtype) {
    case CCB_F32: return by_codec<float>(codec);
    case CCB_BF16: return by_codec<__nv_bfloat16>(codec);
    case CCB_F16: return by_codec<__half>(codec);
    default: return nullptr;
  }
}

int pipe_kernel_threads() { return kPipeThreads; }

}  // namespace ccb

// Declarations shared between the translation units of libccb.so.
#pragma once
#include <cuda_runtime.h>

#include "ccb/ccb.h"

struct ccb_comm;

namespace ccb {
void set_error(const char* fmt, ...);
void count_launch();
CommDev comm_dev(ccb_comm* c, uint32_t epoch);
uint32_t next_epoch(ccb_comm* c);
int grid_cap(ccb_comm* c, const void* kernel, int threads = 512);
int launch(ccb_comm* c, const void* kernel, int ctas, void* args, cudaStream_t stream, int threads = 512, bool may_overlap = false);
int check_alive(ccb_comm* c);
size_t elem_size(int dtype);
size_t codec_slot_bytes(int codec, int dtype, size_t pad);
// The pipelined two-shot kernel for this element type and codec (csrc/kernels/ccb_pipe.cu),
// or null; its CTAs have pipe_kernel_threads() threads and own runs of kPipeChunkElems elements.
constexpr int kPipeChunkElems = 4096;
const void* pipe_kernel_fn(int dtype, int codec);
int pipe_kernel_threads();
int nvls_all_reduce(ccb_comm* c, const void* const* send, void* const* recv, uint64_t count, int dtype, int op,
                    cudaStream_t stream);
}  // namespace ccb

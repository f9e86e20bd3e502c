// Finite HBM read-modify-write burn kernel for the GPU stress daemon, built for
// sm_100a. Every thread walks the buffer with a large stride so that each step is a
// DRAM round trip (the buffer is four times the 126 MB L2), for a bounded number of
// steps: a launch always ends by itself. The grid is (SMs x occupancy - SMs) CTAs of
// 256 threads: one CTA slot per SM stays free for whatever the daemon is interfering
// with. Counterpart of the reference's run_codes/daemons/src/
// daemon_gpu_burn_kernel.cu:31-48 (which is compiled for sm_80 and sized for a 40 MB L2).
#include <cuda_runtime.h>
#include <stdlib.h>

#include "daemon_gpu_burn_kernel.h"

__global__ void __launch_bounds__(256) gpu_burn_finite_kernel(float* __restrict__ buf, size_t n, int iters) {
  const size_t tid = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  const size_t nthreads = (size_t)gridDim.x * blockDim.x;
  size_t i = (tid * 32) % n;                 // lanes of a warp touch different sectors
  const size_t step = (nthreads * 32 + 4099) % n;
  for (int k = 0; k < iters; ++k) {
    float v = buf[i];
    buf[i] = v * 1.0000001f + 1e-7f;
    i += step;
    if (i >= n) i -= n;
  }
}

struct burn_ctx {
  int device;
  float* buf;
  size_t n;
  int grid;
  cudaStream_t stream;
};

extern "C" int daemon_gpu_burn_device_count(void) {
  int n = 0;
  if (cudaGetDeviceCount(&n) != cudaSuccess) return 0;
  return n;
}

extern "C" void* daemon_gpu_burn_create(int device, unsigned long long buffer_bytes) {
  if (cudaSetDevice(device) != cudaSuccess) return nullptr;
  int sms = 0, l2 = 0, occ = 0;
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
  cudaDeviceGetAttribute(&l2, cudaDevAttrL2CacheSize, device);
  cudaOccupancyMaxActiveBlocksPerMultiprocessor(&occ, gpu_burn_finite_kernel, 256, 0);
  if (occ < 2) occ = 2;
  size_t bytes = buffer_bytes ? (size_t)buffer_bytes : (size_t)l2 * 4;
  if (bytes < (256u << 20)) bytes = 256u << 20;
  burn_ctx* c = (burn_ctx*)calloc(1, sizeof(burn_ctx));
  if (!c) return nullptr;
  c->device = device;
  c->n = bytes / sizeof(float);
  c->grid = sms * occ - sms;
  if (cudaMalloc((void**)&c->buf, bytes) != cudaSuccess || cudaMemset(c->buf, 0, bytes) != cudaSuccess ||
      cudaStreamCreateWithFlags(&c->stream, cudaStreamNonBlocking) != cudaSuccess) {
    if (c->buf) cudaFree(c->buf);
    free(c);
    return nullptr;
  }
  return c;
}

extern "C" int daemon_gpu_burn_launch(void* ctx, int iters) {
  burn_ctx* c = (burn_ctx*)ctx;
  if (!c || iters <= 0) return -1;
  if (iters > 50000000) iters = 50000000;  // a launch must stay short
  cudaSetDevice(c->device);
  gpu_burn_finite_kernel<<<c->grid, 256, 0, c->stream>>>(c->buf, c->n, iters);
  if (cudaGetLastError() != cudaSuccess) return -1;
  return cudaStreamSynchronize(c->stream) == cudaSuccess ? 0 : -1;
}

extern "C" void daemon_gpu_burn_destroy(void* ctx) {
  burn_ctx* c = (burn_ctx*)ctx;
  if (!c) return;
  cudaSetDevice(c->device);
  cudaStreamDestroy(c->stream);
  cudaFree(c->buf);
  free(c);
}

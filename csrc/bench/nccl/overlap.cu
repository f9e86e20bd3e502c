// Compute / communication overlap benchmark: time a memory-bound kernel alone, a
// pairwise ncclSend/ncclRecv exchange (even rank <-> odd rank) alone, then both at
// once on two streams, and print the slow-down each suffers.
//
// Reference: run_codes/benchmarks/nccl/overlap/overlap.cu (columns Comp, Comm, PComp,
// PComm, CSlow%, SSlow%, :274-290). Its work kernel is a scalar read-modify-write
// chain over 512 MB sized against a 50 MB L2; here the kernel is a vectorised stream
// over a buffer four times the device's actual L2 (126 MB on B200 -> 512 MB), run on
// every SM, so "compute" means HBM-bound work as in a training step's elementwise
// phases.
#include <cuda_runtime.h>
#include <nccl.h>
#include <stdio.h>
#include <stdlib.h>

extern "C" {
#include "nccl/nccl_utils.h"
#include "utils.h"
}

__global__ void __launch_bounds__(256) overlap_work_kernel(float4* __restrict__ buf, size_t nvec, int passes) {
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  for (int p = 0; p < passes; ++p)
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < nvec; i += stride) {
      float4 v = buf[i];
      v.x = v.x * 1.0000001f + 1e-7f; v.y = v.y * 1.0000001f + 1e-7f;
      v.z = v.z * 1.0000001f + 1e-7f; v.w = v.w * 1.0000001f + 1e-7f;
      buf[i] = v;
    }
}

static float ms_between(cudaEvent_t a, cudaEvent_t b) {
  float ms = 0.f;
  cudaEventElapsedTime(&ms, a, b);
  return ms;
}

int main(int argc, char** argv) {
  nccl_test_context_t ctx = nccl_test_init(argc, argv, "NCCL_Overlap");
  if (ctx.size < 2 || (ctx.size & 1)) {
    if (ctx.rank == 0) fprintf(stderr, "Error: Need an even number (>= 2) of processes\n");
    nccl_test_fini(&ctx);
    return 1;
  }
  int dev = 0, sms = 0, l2 = 0;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  cudaDeviceGetAttribute(&l2, cudaDevAttrL2CacheSize, dev);
  size_t work_bytes = (size_t)l2 * 4;
  if (work_bytes < (512u << 20)) work_bytes = 512u << 20;
  const char* pe = getenv("OVERLAP_WORK_PASSES");
  const int passes = pe ? atoi(pe) : 4;
  float4* d_work = nullptr;
  cudaMalloc(&d_work, work_bytes);
  cudaMemset(d_work, 0, work_bytes);
  void *d_send = nullptr, *d_recv = nullptr;
  cudaMalloc(&d_send, ctx.config.max_message_size ? ctx.config.max_message_size : 4);
  cudaMalloc(&d_recv, ctx.config.max_message_size ? ctx.config.max_message_size : 4);
  cudaMemset(d_send, 1, ctx.config.max_message_size ? ctx.config.max_message_size : 4);
  cudaStream_t comp, comm;
  cudaStreamCreateWithFlags(&comp, cudaStreamNonBlocking);
  cudaStreamCreateWithFlags(&comm, cudaStreamNonBlocking);
  cudaEvent_t c0, c1, m0, m1;
  cudaEventCreate(&c0); cudaEventCreate(&c1); cudaEventCreate(&m0); cudaEventCreate(&m1);
  const int peer = ctx.rank ^ 1;
  const int grid = sms * 4;
  const size_t nvec = work_bytes / sizeof(float4);
  auto exchange = [&](size_t bytes) {
    ncclGroupStart();
    ncclSend(d_send, bytes, ncclUint8, peer, ctx.comm, comm);
    ncclRecv(d_recv, bytes, ncclUint8, peer, ctx.comm, comm);
    ncclGroupEnd();
  };
  if (ctx.rank == 0)
    printf("%12s %10s %10s %10s %10s %8s %8s\n", "Size(B)", "Comp(ms)", "Comm(ms)", "PComp(ms)", "PComm(ms)", "CSlow%", "SSlow%");
  size_iter_t it;
  size_iter_init(&it, &ctx.config);
  size_t msg;
  while (size_iter_next(&it, &msg)) {
    const int iters = ctx.config.iterations > 0 ? ctx.config.iterations : 1;
    double comp_ms = 0, comm_ms = 0, pcomp_ms = 0, pcomm_ms = 0;
    for (int i = 0; i < ctx.config.warmup_iterations + iters; ++i) {
      const bool measured = i >= ctx.config.warmup_iterations;
      nccl_barrier(&ctx);
      cudaEventRecord(c0, comp);
      overlap_work_kernel<<<grid, 256, 0, comp>>>(d_work, nvec, passes);
      cudaEventRecord(c1, comp);
      cudaEventSynchronize(c1);
      nccl_barrier(&ctx);
      cudaEventRecord(m0, comm);
      exchange(msg);
      cudaEventRecord(m1, comm);
      cudaEventSynchronize(m1);
      if (measured) { comp_ms += ms_between(c0, c1); comm_ms += ms_between(m0, m1); }
      nccl_barrier(&ctx);
      cudaEventRecord(c0, comp);
      cudaEventRecord(m0, comm);
      overlap_work_kernel<<<grid, 256, 0, comp>>>(d_work, nvec, passes);
      exchange(msg);
      cudaEventRecord(c1, comp);
      cudaEventRecord(m1, comm);
      cudaEventSynchronize(c1);
      cudaEventSynchronize(m1);
      if (measured) { pcomp_ms += ms_between(c0, c1); pcomm_ms += ms_between(m0, m1); }
    }
    comp_ms /= iters; comm_ms /= iters; pcomp_ms /= iters; pcomm_ms /= iters;
    if (ctx.rank == 0)
      printf("%12zu %10.3f %10.3f %10.3f %10.3f %8.1f %8.1f\n", msg, comp_ms, comm_ms, pcomp_ms, pcomm_ms,
             comp_ms > 0 ? (pcomp_ms / comp_ms - 1.0) * 100.0 : 0.0, comm_ms > 0 ? (pcomm_ms / comm_ms - 1.0) * 100.0 : 0.0);
    if (ctx.config.save_csv) {
      char csv[600];
      if (ctx.config.csv_path[0]) snprintf(csv, sizeof(csv), "%s", ctx.config.csv_path);
      else snprintf(csv, sizeof(csv), "results/overlap.csv");
      nccl_csv_write(csv, "msg_size,comp_ms,comm_ms,pcomp_ms,pcomm_ms", "%zu,%.4f,%.4f,%.4f,%.4f", msg, comp_ms, comm_ms, pcomp_ms, pcomm_ms);
    }
  }
  cudaFree(d_work);
  cudaFree(d_send);
  cudaFree(d_recv);
  nccl_test_fini(&ctx);
  return 0;
}

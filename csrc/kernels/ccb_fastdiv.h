/* Division of a small unsigned number by a run-time divisor as a multiplication.
 *
 * magic = floor(2^40 / d) + 1, q = (n * magic) >> 40. Exact for n < 2^22 and 1 <= d < 2^18:
 * then n * d < 2^40, which bounds the error of the rounded-up reciprocal below one quotient
 * step, and n * magic < 2^63 fits the 64-bit product. An integer division by a run-time value
 * costs a GPU about 25 instructions; kernels that need one per thread and tile take the magic
 * number from the host instead. Plain C, shared by host code, kernels and the CPU test. */
#ifndef CCB_FASTDIV_H
#define CCB_FASTDIV_H

#include <stdint.h>

#if defined(__CUDACC__)
#define CCB_FASTDIV_FN __host__ __device__ static inline
#else
#define CCB_FASTDIV_FN static inline
#endif

#define CCB_FASTDIV_MAX_N (1ull << 22)
#define CCB_FASTDIV_MAX_D (1ull << 18)

/* 0 when the pair (largest numerator, divisor) is outside the exact range. */
CCB_FASTDIV_FN uint64_t ccb_fastdiv_magic(uint64_t max_n, uint64_t d) {
  if (d == 0 || d >= CCB_FASTDIV_MAX_D || max_n >= CCB_FASTDIV_MAX_N) return 0;
  return (1ull << 40) / d + 1;
}
CCB_FASTDIV_FN uint32_t ccb_fastdiv(uint32_t n, uint64_t magic) { return (uint32_t)(((uint64_t)n * magic) >> 40); }

#endif

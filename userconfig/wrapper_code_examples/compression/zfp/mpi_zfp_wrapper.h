/* The two strong symbols that mpi_zfp_wrapper.c gives to the MPI compression hooks: they
 * replace the weak pass-through pair of mpi_compress_tools. Buffers are host memory; on entry
 * *output_size is the capacity of `output`, on return the bytes written. Both return 0 on
 * success. The codec is configured by the MPI_ZFP_* environment variables listed at the top of
 * the source file. */
#ifndef MPI_ZFP_WRAPPER_H
#define MPI_ZFP_WRAPPER_H

#include <stddef.h>

#ifdef __cplusplus
extern "C" {
#endif

int mpi_compress(void *input, size_t input_size, void *output, size_t *output_size);
int mpi_decompress(void *input, size_t input_size, void *output, size_t output_size);

#ifdef __cplusplus
}
#endif
#endif

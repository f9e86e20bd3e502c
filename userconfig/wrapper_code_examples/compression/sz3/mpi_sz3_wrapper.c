/* Same path and environment (MPI_SZ3_TYPE, MPI_SZ3_ABS_EB) as the reference's SZ3
 * compression wrapper (userconfig/wrapper_code_examples/compression/sz3/mpi_sz3_wrapper.c),
 * which dlopen()s libSZ3c. That library is not available here; the strong mpi_compress /
 * mpi_decompress of this build come from the in-tree error-bounded CPU codec (quantise
 * under an absolute bound, Lorenzo prediction, byte-wise packing), same contract: the
 * decompressed values are within the bound of the input. This file only forwards. */
#include "../sz_cpu/mpi_szcpu_wrapper.c"

/* One library that is both the compressed MPI collectives and their error-bounded codec:
 * the role of the reference's ZCCL wrapper (userconfig/wrapper_code_examples/communication/
 * zccl/mpi_zccl_wrapper.c:96-204), which hands MPI_Bcast / Scatter / Allreduce / Allgather
 * on MPI_FLOAT to libZCCL and everything else to PMPI. libZCCL is not available here; the
 * collectives are the ring / tree algorithms of the in-tree MPI wrapper and the codec is the
 * in-tree error-bounded CPU codec, linked into ONE library (the strong mpi_compress /
 * mpi_decompress of this file replace the weak identity ones of the wrapper):
 *
 *   source_files: this file, ../plain_mpi_compress/plain_mpi_compress.c,
 *                 csrc/wrappers/mpi_compress_tools.c
 *
 * Environment: ZCCL_TOL (absolute error bound, the reference's name, :70-90) is mapped to the
 * codec's bound unless MPI_SZ3_ABS_EB is set; ZCCL_CR, ZCCL_BLOCK and ZCCL_MODE tune
 * libZCCL's own codec and have no meaning for this one. */
#include <stdlib.h>

__attribute__((constructor)) static void zccl_env_alias(void) {
    const char *tol = getenv("ZCCL_TOL");
    if (tol && *tol && !getenv("MPI_SZ3_ABS_EB")) setenv("MPI_SZ3_ABS_EB", tol, 1);
}

#include "../../compression/sz_cpu/mpi_szcpu_wrapper.c"

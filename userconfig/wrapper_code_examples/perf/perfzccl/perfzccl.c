/* Same path as the reference's perf wrapper for ZCCL runs
 * (userconfig/wrapper_code_examples/perf/perfzccl/perfzccl.c). Its MPI half (MPI_Allreduce,
 * Bcast, Scatter, Allgather and point-to-point, with mpi_compress / mpi_decompress) is what
 * the MPI perf wrapper of this repository records; the ZCCL-internal codec symbols have
 * nothing to attach to here, that library being absent. This file only forwards. */
#include "../perfmpi/perfmpi.c"

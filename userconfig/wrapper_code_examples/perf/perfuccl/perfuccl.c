/* Same path as the reference's perf wrapper for the UCCL transport
 * (userconfig/wrapper_code_examples/perf/perfuccl/perfuccl.c: ncclCommInitRank for the
 * node map, ncclSend/Recv/AllReduce/Broadcast). The NCCL perf wrapper of this repository
 * records a superset of those calls with the same columns; this file only forwards to it. */
#include "../perfnccl/perfnccl.c"

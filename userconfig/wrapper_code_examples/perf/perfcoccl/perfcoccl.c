/* Same path as the reference's perf wrapper for COCCL builds
 * (userconfig/wrapper_code_examples/perf/perfcoccl/perfcoccl.c: ncclSend/Recv, the four
 * compression hooks, four collectives), so configurations that name it as `source_files`
 * keep building. The columns and hooks are those of the NCCL perf wrapper of this
 * repository, which times every one of them (and more); this file only forwards to it. */
#include "../perfnccl/perfnccl.c"

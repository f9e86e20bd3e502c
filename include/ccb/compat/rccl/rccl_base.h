/* Source compatibility for wrappers written against the reference's RCCL loader
 * (run_codes/benchmark-core/include/rccl/rccl_base.h): the same base_nccl* functions, here
 * over the NCCL library recorded by findso. There is no RCCL on this hardware. */
#ifndef RCCL_BASE_H
#define RCCL_BASE_H
#include "../nccl/nccl_base.h"
#endif

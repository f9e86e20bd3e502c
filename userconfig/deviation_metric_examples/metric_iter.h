/* Typed iteration over two buffers as doubles, shared by the metric sources. A
 * metric file defines compute_<name>(user, reference, count, dtype) and is picked up
 * by scripts/register_metrics.sh by file name. */
#ifndef CCB_METRIC_ITER_H
#define CCB_METRIC_ITER_H
#include <math.h>
#include <stdio.h>
#include <stdlib.h>

#include "validation.h"

#define METRIC_FOR_EACH(buf1, buf2, count, dtype, A, B, BODY)                          \
    do {                                                                                \
        switch (dtype) {                                                                \
            case TYPE_FLOAT:                                                            \
                for (int i_ = 0; i_ < (count); ++i_) {                                  \
                    const double A = ((const float *)(buf1))[i_], B = ((const float *)(buf2))[i_]; \
                    BODY;                                                               \
                }                                                                       \
                break;                                                                  \
            case TYPE_DOUBLE:                                                           \
                for (int i_ = 0; i_ < (count); ++i_) {                                  \
                    const double A = ((const double *)(buf1))[i_], B = ((const double *)(buf2))[i_]; \
                    BODY;                                                               \
                }                                                                       \
                break;                                                                  \
            case TYPE_INT:                                                              \
                for (int i_ = 0; i_ < (count); ++i_) {                                  \
                    const double A = ((const int *)(buf1))[i_], B = ((const int *)(buf2))[i_]; \
                    BODY;                                                               \
                }                                                                       \
                break;                                                                  \
            case TYPE_BFLOAT16:                                                         \
            case TYPE_HALF:                                                             \
                for (int i_ = 0; i_ < (count); ++i_) {                                  \
                    const double A = to_double((buf1), (dtype), i_), B = to_double((buf2), (dtype), i_); \
                    BODY;                                                               \
                }                                                                       \
                break;                                                                  \
            default:                                                                    \
                for (int i_ = 0; i_ < (count); ++i_) {                                  \
                    const double A = ((const char *)(buf1))[i_], B = ((const char *)(buf2))[i_]; \
                    BODY;                                                               \
                }                                                                       \
                break;                                                                  \
        }                                                                               \
    } while (0)
#endif

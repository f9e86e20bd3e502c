/* Raw result dumps, "<base>_<suffix>.bin". One writer, or all ranks writing their
 * chunk at rank * chunk of a file that rank 0 sized first (POSIX pwrite, no MPI).
 * Same files and layout as the reference's run_codes/benchmark-core/src/
 * binary_output.c:18-87; accumulate / average as :91-149. */
#define _GNU_SOURCE
#include <errno.h>
#include <fcntl.h>
#include <stdio.h>
#include <string.h>
#include <sys/stat.h>
#include <unistd.h>

#include "binary_output.h"

static void full_path(char *dst, size_t cap, const char *base, const char *suffix) {
    snprintf(dst, cap, "%s_%s.bin", base, suffix);
}

static int write_all_at(int fd, const void *buf, size_t n, off_t off) {
    const char *p = (const char *)buf;
    while (n) {
        ssize_t w = pwrite(fd, p, n, off);
        if (w < 0) {
            if (errno == EINTR) continue;
            return -1;
        }
        p += w;
        off += w;
        n -= (size_t)w;
    }
    return 0;
}

void write_binary_single(const char *base_path, const char *suffix, const void *buf, size_t bytes, int rank,
                         int writer_rank) {
    if (!base_path || !suffix || !buf || !bytes || rank != writer_rank) return;
    char path[1024];
    full_path(path, sizeof(path), base_path, suffix);
    int fd = open(path, O_CREAT | O_WRONLY | O_TRUNC, 0644);
    if (fd < 0) {
        fprintf(stderr, "[binary_output] open %s: %s\n", path, strerror(errno));
        return;
    }
    if (write_all_at(fd, buf, bytes, 0) != 0) fprintf(stderr, "[binary_output] write %s: %s\n", path, strerror(errno));
    close(fd);
}

void write_binary_multi(const char *base_path, const char *suffix, const void *buf, size_t chunk_size, int rank,
                        int nranks) {
    if (!base_path || !suffix || !buf || !chunk_size || nranks <= 0) return;
    char path[1024];
    full_path(path, sizeof(path), base_path, suffix);
    const off_t total = (off_t)nranks * (off_t)chunk_size;
    int fd = -1;
    if (rank == 0) {
        fd = open(path, O_CREAT | O_WRONLY | O_TRUNC, 0644);
        if (fd >= 0 && ftruncate(fd, total) != 0) fprintf(stderr, "[binary_output] ftruncate: %s\n", strerror(errno));
    } else {
        /* wait (briefly) for rank 0 to have created and sized the file */
        for (int tries = 0; tries < 3000; ++tries) {
            struct stat st;
            fd = open(path, O_WRONLY);
            if (fd >= 0 && fstat(fd, &st) == 0 && st.st_size >= total) break;
            if (fd >= 0) close(fd);
            fd = -1;
            usleep(1000);
        }
    }
    if (fd < 0) {
        fprintf(stderr, "[binary_output] rank %d cannot open %s\n", rank, path);
        return;
    }
    if (write_all_at(fd, buf, chunk_size, (off_t)rank * (off_t)chunk_size) != 0)
        fprintf(stderr, "[binary_output] rank %d pwrite: %s\n", rank, strerror(errno));
    close(fd);
}

void binary_accumulate(void *accum, const void *buf, int count, data_type_t dtype) {
    switch (dtype) {
        case TYPE_INT: for (int i = 0; i < count; ++i) ((int *)accum)[i] += ((const int *)buf)[i]; break;
        case TYPE_FLOAT: for (int i = 0; i < count; ++i) ((float *)accum)[i] += ((const float *)buf)[i]; break;
        case TYPE_DOUBLE: for (int i = 0; i < count; ++i) ((double *)accum)[i] += ((const double *)buf)[i]; break;
        case TYPE_BFLOAT16:
            for (int i = 0; i < count; ++i)
                ((uint16_t *)accum)[i] = ccb_float_to_bf16(ccb_bf16_to_float(((uint16_t *)accum)[i]) + ccb_bf16_to_float(((const uint16_t *)buf)[i]));
            break;
        case TYPE_HALF:
            for (int i = 0; i < count; ++i)
                ((uint16_t *)accum)[i] = ccb_float_to_half(ccb_half_to_float(((uint16_t *)accum)[i]) + ccb_half_to_float(((const uint16_t *)buf)[i]));
            break;
        default: for (int i = 0; i < count; ++i) ((char *)accum)[i] = (char)(((char *)accum)[i] + ((const char *)buf)[i]); break;
    }
}

void binary_average(void *accum, int count, data_type_t dtype, int divisor) {
    if (divisor <= 1) return;
    switch (dtype) {
        case TYPE_INT: for (int i = 0; i < count; ++i) ((int *)accum)[i] /= divisor; break;
        case TYPE_FLOAT: for (int i = 0; i < count; ++i) ((float *)accum)[i] /= (float)divisor; break;
        case TYPE_DOUBLE: for (int i = 0; i < count; ++i) ((double *)accum)[i] /= (double)divisor; break;
        case TYPE_BFLOAT16:
            for (int i = 0; i < count; ++i) ((uint16_t *)accum)[i] = ccb_float_to_bf16(ccb_bf16_to_float(((uint16_t *)accum)[i]) / (float)divisor);
            break;
        case TYPE_HALF:
            for (int i = 0; i < count; ++i) ((uint16_t *)accum)[i] = ccb_float_to_half(ccb_half_to_float(((uint16_t *)accum)[i]) / (float)divisor);
            break;
        default: for (int i = 0; i < count; ++i) ((char *)accum)[i] = (char)(((char *)accum)[i] / divisor); break;
    }
}

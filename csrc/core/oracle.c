/* CPU oracle ("dummy collectives"): recompute the expected result of a collective
 * from the data source of every simulated rank, without any communication call.
 *
 * Data source rules follow the reference (run_codes/benchmark-core/src/
 * dummy_collectives.c:15-157): pattern fill when no input file is given; with
 * DS_TYPE=folder each rank reads <folder>/rank_<r><suffix>; otherwise one file is
 * read at DS_CUSTOM_OFFSETS[r], or DS_BASE_OFFSET (+ r * bytes unless
 * DS_PER_RANK_OFFSET is set to something other than "true"), wrapped modulo the file
 * size and zero padded. Sums accumulate in the element type as the reference does
 * (dummy_collectives.c:161-189); dummy_allreduce_f64 accumulates in float64. */
#define _GNU_SOURCE
#include <dirent.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include <strings.h>

#include "dummy_collectives.h"
#include "validation.h"

static void load_from_folder(const char *folder, void *buf, size_t bytes, int r) {
    const char *suffix = getenv("DS_SUFFIX");
    const char *fmt = getenv("DS_FORMAT");
    if (!suffix || !*suffix) suffix = (fmt && !strcasecmp(fmt, "text")) ? ".txt" : ".bin";
    char path[1024];
    snprintf(path, sizeof(path), "%s/rank_%d%s", folder, r, suffix);
    FILE *fp = fopen(path, "rb");
    if (!fp) { /* any file called rank_<r> or rank_<r>.<something> */
        DIR *d = opendir(folder);
        if (!d) {
            fprintf(stderr, "[oracle] cannot open folder '%s'\n", folder);
            exit(1);
        }
        char prefix[64];
        const int plen = snprintf(prefix, sizeof(prefix), "rank_%d", r);
        struct dirent *e;
        while ((e = readdir(d))) {
            if (strncmp(e->d_name, prefix, (size_t)plen)) continue;
            if (e->d_name[plen] != '.' && e->d_name[plen] != '\0') continue;
            snprintf(path, sizeof(path), "%s/%s", folder, e->d_name);
            fp = fopen(path, "rb");
            break;
        }
        closedir(d);
    }
    if (!fp) {
        fprintf(stderr, "[oracle] no file matching 'rank_%d*' in '%s'\n", r, folder);
        exit(1);
    }
    size_t got = fread(buf, 1, bytes, fp);
    fclose(fp);
    if (got < bytes) memset((char *)buf + got, 0, bytes - got);
}

void dummy_load_rank_data(const char *input_file, data_type_t datatype, pattern_type_t pattern_type, void *buf,
                          size_t bytes, int sim_rank, int nranks) {
    (void)nranks;
    if (!input_file) {
        const size_t es = get_element_size(datatype);
        int count = (int)(bytes / es);
        if (count < 1) count = 1;
        init_buffer_pattern(buf, count, datatype, pattern_type, sim_rank);
        return;
    }
    const char *ds = getenv("DS_TYPE");
    if (ds && !strcmp(ds, "folder")) {
        load_from_folder(input_file, buf, bytes, sim_rank);
        return;
    }
    FILE *fp = fopen(input_file, "rb");
    if (!fp) {
        fprintf(stderr, "[oracle] cannot open '%s'\n", input_file);
        exit(1);
    }
    fseek(fp, 0, SEEK_END);
    const size_t fsize = (size_t)ftell(fp);
    size_t chunk = bytes, off = (size_t)sim_rank * bytes;
    const char *custom = getenv("DS_CUSTOM_OFFSETS");
    if (custom && *custom) {
        char *copy = strdup(custom), *save = NULL;
        int r = 0;
        for (char *tok = strtok_r(copy, ",", &save); tok; tok = strtok_r(NULL, ",", &save), ++r)
            if (r == sim_rank) {
                long v = atol(tok);
                if (v >= 0) off = (size_t)v;
                break;
            }
        free(copy);
    } else {
        /* offset = base (default 0) + rank * bytes unless DS_PER_RANK_OFFSET says otherwise.
         * (Without DS_BASE_OFFSET the reference adds rank * bytes twice; its run script
         * always exports the base, so the two agree for generated runs.) */
        const char *base = getenv("DS_BASE_OFFSET"), *per = getenv("DS_PER_RANK_OFFSET");
        off = base ? (size_t)atol(base) : 0;
        if (!per || !strcmp(per, "true")) off += (size_t)sim_rank * bytes;
    }
    if (fsize > 0) {
        off %= fsize;
        if (off + chunk > fsize) chunk = fsize - off;
    }
    fseek(fp, (long)off, SEEK_SET);
    size_t got = fread(buf, 1, chunk, fp);
    fclose(fp);
    if (got < bytes) memset((char *)buf + got, 0, bytes - got);
}

static void add_into(void *dst, const void *src, int count, data_type_t t) {
    switch (t) {
        case TYPE_INT: for (int i = 0; i < count; ++i) ((int *)dst)[i] += ((const int *)src)[i]; break;
        case TYPE_FLOAT: for (int i = 0; i < count; ++i) ((float *)dst)[i] += ((const float *)src)[i]; break;
        case TYPE_DOUBLE: for (int i = 0; i < count; ++i) ((double *)dst)[i] += ((const double *)src)[i]; break;
        /* element-type accumulation of a 16-bit float: one rounding per addition */
        case TYPE_BFLOAT16:
            for (int i = 0; i < count; ++i)
                ((uint16_t *)dst)[i] = ccb_float_to_bf16(ccb_bf16_to_float(((uint16_t *)dst)[i]) + ccb_bf16_to_float(((const uint16_t *)src)[i]));
            break;
        case TYPE_HALF:
            for (int i = 0; i < count; ++i)
                ((uint16_t *)dst)[i] = ccb_float_to_half(ccb_half_to_float(((uint16_t *)dst)[i]) + ccb_half_to_float(((const uint16_t *)src)[i]));
            break;
        default: for (int i = 0; i < count; ++i) ((char *)dst)[i] = (char)(((char *)dst)[i] + ((const char *)src)[i]); break;
    }
}

static void *xmalloc(size_t n) {
    void *p = malloc(n ? n : 1);
    if (!p) {
        fprintf(stderr, "[oracle] out of memory (%zu bytes)\n", n);
        exit(1);
    }
    return p;
}

void dummy_allreduce(void *ref, const char *input_file, data_type_t datatype, pattern_type_t pattern_type, int count,
                     int nranks) {
    if (datatype == TYPE_BFLOAT16 || datatype == TYPE_HALF) {
        /* a sum carried in a 16-bit float would be a worse reference than the device's fp32
         * accumulation: these types are summed in float64 and rounded once */
        dummy_allreduce_f64(ref, input_file, datatype, pattern_type, count, nranks);
        return;
    }
    const size_t bytes = (size_t)count * get_element_size(datatype);
    void *tmp = xmalloc(bytes);
    dummy_load_rank_data(input_file, datatype, pattern_type, ref, bytes, 0, nranks);
    for (int r = 1; r < nranks; ++r) {
        dummy_load_rank_data(input_file, datatype, pattern_type, tmp, bytes, r, nranks);
        add_into(ref, tmp, count, datatype);
    }
    free(tmp);
}

void dummy_allreduce_f64(void *ref, const char *input_file, data_type_t datatype, pattern_type_t pattern_type,
                         int count, int nranks) {
    const size_t bytes = (size_t)count * get_element_size(datatype);
    void *tmp = xmalloc(bytes);
    double *acc = (double *)calloc((size_t)(count > 0 ? count : 1), sizeof(double));
    if (!acc) {
        fprintf(stderr, "[oracle] out of memory\n");
        exit(1);
    }
    for (int r = 0; r < nranks; ++r) {
        dummy_load_rank_data(input_file, datatype, pattern_type, tmp, bytes, r, nranks);
        for (int i = 0; i < count; ++i) acc[i] += to_double(tmp, datatype, i);
    }
    for (int i = 0; i < count; ++i) {
        if (datatype == TYPE_INT) ((int *)ref)[i] = (int)acc[i];
        else if (datatype == TYPE_FLOAT) ((float *)ref)[i] = (float)acc[i];
        else if (datatype == TYPE_DOUBLE) ((double *)ref)[i] = acc[i];
        else if (datatype == TYPE_BFLOAT16) ((uint16_t *)ref)[i] = ccb_float_to_bf16((float)acc[i]);
        else if (datatype == TYPE_HALF) ((uint16_t *)ref)[i] = ccb_float_to_half((float)acc[i]);
        else ((char *)ref)[i] = (char)acc[i];
    }
    free(acc);
    free(tmp);
}

void dummy_reduce(void *ref, const char *input_file, data_type_t datatype, pattern_type_t pattern_type, int count,
                  int nranks, int root) {
    (void)root;
    dummy_allreduce(ref, input_file, datatype, pattern_type, count, nranks);
}

/* Rank r's send buffer holds nranks blocks of count_per; block d goes to rank d. */
void dummy_alltoall(void *ref, const char *input_file, data_type_t datatype, pattern_type_t pattern_type,
                    int count_per, int nranks, int rank) {
    const size_t es = get_element_size(datatype), blk = (size_t)count_per * es, full = blk * (size_t)nranks;
    char *tmp = (char *)xmalloc(full);
    for (int s = 0; s < nranks; ++s) {
        dummy_load_rank_data(input_file, datatype, pattern_type, tmp, full, s, nranks);
        memcpy((char *)ref + (size_t)s * blk, tmp + (size_t)rank * blk, blk);
    }
    free(tmp);
}

void dummy_allgather(void *ref, const char *input_file, data_type_t datatype, pattern_type_t pattern_type, int count,
                     int nranks) {
    const size_t blk = (size_t)count * get_element_size(datatype);
    for (int s = 0; s < nranks; ++s)
        dummy_load_rank_data(input_file, datatype, pattern_type, (char *)ref + (size_t)s * blk, blk, s, nranks);
}

void dummy_gather(void *ref, const char *input_file, data_type_t datatype, pattern_type_t pattern_type, int count,
                  int nranks, int root) {
    (void)root;
    dummy_allgather(ref, input_file, datatype, pattern_type, count, nranks);
}

/* Root's send buffer holds nranks blocks of count; rank gets block `rank`. */
void dummy_scatter(void *ref, const char *input_file, data_type_t datatype, pattern_type_t pattern_type, int count,
                   int nranks, int root, int rank) {
    const size_t blk = (size_t)count * get_element_size(datatype), full = blk * (size_t)nranks;
    char *tmp = (char *)xmalloc(full);
    dummy_load_rank_data(input_file, datatype, pattern_type, tmp, full, root, nranks);
    memcpy(ref, tmp + (size_t)rank * blk, blk);
    free(tmp);
}

/* count = elements each rank receives; every rank sends count * nranks. */
void dummy_reduce_scatter(void *ref, const char *input_file, data_type_t datatype, pattern_type_t pattern_type,
                          int count, int nranks, int rank) {
    const size_t es = get_element_size(datatype), blk = (size_t)count * es, full = blk * (size_t)nranks;
    char *tmp = (char *)xmalloc(full);
    memset(ref, 0, blk);
    for (int s = 0; s < nranks; ++s) {
        dummy_load_rank_data(input_file, datatype, pattern_type, tmp, full, s, nranks);
        if (s == 0) memcpy(ref, tmp + (size_t)rank * blk, blk);
        else add_into(ref, tmp + (size_t)rank * blk, count, datatype);
    }
    free(tmp);
}

void dummy_bcast(void *ref, const char *input_file, data_type_t datatype, pattern_type_t pattern_type, int count,
                 int nranks, int root) {
    dummy_load_rank_data(input_file, datatype, pattern_type, ref, (size_t)count * get_element_size(datatype), root,
                         nranks);
}

/* argv front-end, data patterns, file I/O, message-size iterator, oracle cache.
 *
 * Behaviour follows the reference's run_codes/benchmark-core/src/utils.c: option
 * string "d:m:i:w:f:t:vMhe:p:co:L:bB:S:R:A" (utils.c:306), defaults 1:65536:2,
 * 100 iterations, 10 warm-up, tolerance 1e-6, double, rank_linear (utils.c:26-31,
 * 286-303). Differences: -m accepts sizes beyond the int range (the reference parses
 * them with atoi), and -S / -R, which the reference parses but never consumes
 * (utils.c:374-382), are implemented by ref_cache_store / ref_cache_load. */
#define _GNU_SOURCE
#include <errno.h>
#include <getopt.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include <strings.h>
#include <sys/stat.h>

#include "utils.h"
#include "validation.h"

/* ------------------------------------------------------------------ file I/O */
static size_t elem_bytes(data_type_t t) { return get_element_size(t); }

int read_from_file(const char *filename, void *buffer, size_t buffer_size, file_format_t format,
                   data_type_t datatype) {
    FILE *fp = fopen(filename, format == FILE_FORMAT_BINARY ? "rb" : "r");
    if (!fp) {
        fprintf(stderr, "read_from_file: cannot open %s: %s\n", filename, strerror(errno));
        return -1;
    }
    size_t got = 0;
    if (format == FILE_FORMAT_BINARY) {
        got = fread(buffer, 1, buffer_size, fp);
    } else {
        const size_t es = elem_bytes(datatype), n = buffer_size / es;
        size_t i = 0;
        for (; i < n; ++i) {
            int ok;
            if (datatype == TYPE_INT) ok = fscanf(fp, "%d", (int *)buffer + i);
            else if (datatype == TYPE_FLOAT) ok = fscanf(fp, "%f", (float *)buffer + i);
            else if (datatype == TYPE_DOUBLE) ok = fscanf(fp, "%lf", (double *)buffer + i);
            else if (datatype == TYPE_BFLOAT16 || datatype == TYPE_HALF) {
                float f = 0.f;
                ok = fscanf(fp, "%f", &f);
                ((uint16_t *)buffer)[i] = datatype == TYPE_HALF ? ccb_float_to_half(f) : ccb_float_to_bf16(f);
            }
            else {
                int v;
                ok = fscanf(fp, "%d", &v);
                if (ok == 1) ((char *)buffer)[i] = (char)v;
            }
            if (ok != 1) break;
        }
        got = i * es;
    }
    fclose(fp);
    if (got < buffer_size) memset((char *)buffer + got, 0, buffer_size - got);
    return 0;
}

int write_to_file(const char *filename, const void *buffer, size_t buffer_size, file_format_t format,
                  data_type_t datatype) {
    FILE *fp = fopen(filename, format == FILE_FORMAT_BINARY ? "wb" : "w");
    if (!fp) {
        fprintf(stderr, "write_to_file: cannot open %s: %s\n", filename, strerror(errno));
        return -1;
    }
    int rc = 0;
    if (format == FILE_FORMAT_BINARY) {
        if (fwrite(buffer, 1, buffer_size, fp) != buffer_size) rc = -1;
    } else {
        const size_t n = buffer_size / elem_bytes(datatype);
        for (size_t i = 0; i < n; ++i) {
            if (datatype == TYPE_INT) fprintf(fp, "%d\n", ((const int *)buffer)[i]);
            else if (datatype == TYPE_FLOAT) fprintf(fp, "%.9g\n", ((const float *)buffer)[i]);
            else if (datatype == TYPE_DOUBLE) fprintf(fp, "%.17g\n", ((const double *)buffer)[i]);
            else if (datatype == TYPE_BFLOAT16) fprintf(fp, "%.9g\n", ccb_bf16_to_float(((const uint16_t *)buffer)[i]));
            else if (datatype == TYPE_HALF) fprintf(fp, "%.9g\n", ccb_half_to_float(((const uint16_t *)buffer)[i]));
            else fprintf(fp, "%d\n", (int)((const char *)buffer)[i]);
        }
    }
    fclose(fp);
    return rc;
}

void *allocate_aligned_buffer(size_t size, size_t alignment) {
    void *p = NULL;
    if (alignment < sizeof(void *)) alignment = sizeof(void *);
    if (posix_memalign(&p, alignment, size ? size : alignment) != 0) return NULL;
    return p;
}
void free_aligned_buffer(void *ptr) { free(ptr); }

/* ------------------------------------------------------------------ patterns */
pattern_type_t parse_pattern_type(const char *name) {
    static const char *names[] = {"plain", "rank_linear", "rank_product", "sequential"};
    for (int i = 0; i < 4; ++i)
        if (strcasecmp(name, names[i]) == 0) return (pattern_type_t)i;
    fprintf(stderr, "Unknown pattern type: '%s' (options: plain, rank_linear, rank_product, sequential)\n", name);
    exit(1);
}

static inline double pattern_value(pattern_type_t p, int rank, int count, int i) {
    switch (p) {
        case PATTERN_RANK_LINEAR: return (double)(rank + i);
        case PATTERN_RANK_PRODUCT: return (double)((rank + 1) * (i + 1));
        case PATTERN_SEQUENTIAL: return (double)(rank * count + i);
        default: return 1.0;
    }
}

void init_buffer_pattern(void *buffer, int count, data_type_t datatype, pattern_type_t pattern_type, int rank) {
    if (!buffer) return;
    for (int i = 0; i < count; ++i) {
        /* integer arithmetic first, like the reference, so that overflow wraps the same way */
        int iv;
        switch (pattern_type) {
            case PATTERN_RANK_LINEAR: iv = rank + i; break;
            case PATTERN_RANK_PRODUCT: iv = (int)((unsigned)(rank + 1) * (unsigned)(i + 1)); break;
            case PATTERN_SEQUENTIAL: iv = (int)((unsigned)rank * (unsigned)count + (unsigned)i); break;
            default: iv = 1; break;
        }
        (void)pattern_value;
        if (datatype == TYPE_INT) ((int *)buffer)[i] = iv;
        else if (datatype == TYPE_FLOAT) ((float *)buffer)[i] = (float)iv;
        else if (datatype == TYPE_DOUBLE) ((double *)buffer)[i] = (double)iv;
        else if (datatype == TYPE_BFLOAT16) ((uint16_t *)buffer)[i] = ccb_float_to_bf16((float)iv);
        else if (datatype == TYPE_HALF) ((uint16_t *)buffer)[i] = ccb_float_to_half((float)iv);
        else ((char *)buffer)[i] = (char)((rank + i) % 256);
    }
}

void print_buffer(const void *buffer, int count, data_type_t datatype, int max_to_print) {
    if (max_to_print <= 0 || count <= 0) return;
    const int n = count < max_to_print ? count : max_to_print;
    printf("Buffer (first %d of %d): ", n, count);
    for (int i = 0; i < n; ++i) {
        if (datatype == TYPE_INT) printf("%d ", ((const int *)buffer)[i]);
        else if (datatype == TYPE_FLOAT) printf("%.3f ", ((const float *)buffer)[i]);
        else if (datatype == TYPE_DOUBLE) printf("%.6lf ", ((const double *)buffer)[i]);
        else if (datatype == TYPE_BFLOAT16) printf("%.3f ", ccb_bf16_to_float(((const uint16_t *)buffer)[i]));
        else if (datatype == TYPE_HALF) printf("%.3f ", ccb_half_to_float(((const uint16_t *)buffer)[i]));
        else printf("%d ", (int)((const char *)buffer)[i]);
    }
    printf("\n");
}

/* ---------------------------------------------------------------------- argv */
static void usage(const char *prog) {
    printf("Usage: %s [options]\n"
           "Options:\n"
           "  -d TYPE          Data type: float, double, int, char (default: double)\n"
           "  -m MIN:MAX:INCR  Message size range in bytes (default: 1:65536:2)\n"
           "  -A               INCR is added each step instead of multiplied\n"
           "  -L X,Y,Z         Explicit message size list (overrides -m)\n"
           "  -p PATTERN       plain, rank_linear, rank_product, sequential (default: rank_linear)\n"
           "  -i ITER          Measured iterations (default: 100)\n"
           "  -w WARMUP        Warm-up iterations (default: 10)\n"
           "  -f FILE          Input file, or folder when DS_TYPE=folder\n"
           "  -t TOL           Validation tolerance (default: 1e-6)\n"
           "  -v               Validate every iteration against the CPU oracle\n"
           "  -M               Compute all deviation metrics\n"
           "  -e METRICS       Comma-separated metric names, or 'all'\n"
           "  -c               Write a result CSV\n"
           "  -o PATH          CSV path (default: results/<test>.csv)\n"
           "  -b               Dump reference and user results as raw binary\n"
           "  -B PATH          Base path of the binary dumps\n"
           "  -S DIR           Store the oracle's results under DIR\n"
           "  -R DIR           Load the oracle's results from DIR instead of recomputing\n"
           "  -h               This help\n",
           prog);
}

static size_t parse_size(const char *s) {
    char *end = NULL;
    unsigned long long v = strtoull(s, &end, 10);
    if (end && (*end == 'k' || *end == 'K')) v <<= 10;
    else if (end && (*end == 'm' || *end == 'M')) v <<= 20;
    else if (end && (*end == 'g' || *end == 'G')) v <<= 30;
    return (size_t)v;
}

static void copy_path(char *dst, size_t cap, const char *src) {
    strncpy(dst, src, cap - 1);
    dst[cap - 1] = '\0';
}

test_config_t parse_arguments(int argc, char **argv) {
    test_config_t c;
    memset(&c, 0, sizeof(c));
    c.min_message_size = 1;
    c.max_message_size = 65536;
    c.message_size_incr = 2;
    c.iterations = 100;
    c.warmup_iterations = 10;
    c.file_format = FILE_FORMAT_BINARY;
    c.tolerance = 1e-6;
    c.pattern_type = PATTERN_RANK_LINEAR;
    c.data_type = TYPE_DOUBLE;
    optind = 1;
    int opt;
    while ((opt = getopt(argc, argv, "d:m:i:w:f:t:vMhe:p:co:L:bB:S:R:A")) != -1) {
        switch (opt) {
            case 'm': {
                char *save = NULL;
                char *tok = strtok_r(optarg, ":", &save);
                if (tok) c.min_message_size = parse_size(tok);
                if ((tok = strtok_r(NULL, ":", &save))) c.max_message_size = parse_size(tok);
                if ((tok = strtok_r(NULL, ":", &save))) c.message_size_incr = atoi(tok);
                break;
            }
            case 'A': c.message_size_incr_mode = 1; break;
            case 'L': {
                c.use_size_list = 1;
                c.num_sizes = 0;
                size_t lo = (size_t)-1, hi = 0;
                char *save = NULL;
                for (char *tok = strtok_r(optarg, ",", &save); tok && c.num_sizes < 256;
                     tok = strtok_r(NULL, ",", &save)) {
                    size_t v = parse_size(tok);
                    c.size_list[c.num_sizes++] = v;
                    if (v < lo) lo = v;
                    if (v > hi) hi = v;
                }
                if (c.num_sizes) {
                    c.min_message_size = lo;
                    c.max_message_size = hi;
                }
                break;
            }
            case 'i': c.iterations = atoi(optarg); break;
            case 'w': c.warmup_iterations = atoi(optarg); break;
            case 'f': c.input_file = optarg; break;
            case 't': c.tolerance = atof(optarg); break;
            case 'v': c.validate = 1; break;
            case 'M':
                c.compute_metrics = 1;
                c.metrics_mask = validation_registry_count() >= 32 ? 0xffffffffu
                                                                   : ((1u << validation_registry_count()) - 1u);
                break;
            case 'e':
                c.compute_metrics = 1;
                c.metrics_mask = parse_metric_mask(optarg);
                break;
            case 'p': c.pattern_type = parse_pattern_type(optarg); break;
            case 'd':
                if (!strcasecmp(optarg, "float")) c.data_type = TYPE_FLOAT;
                else if (!strcasecmp(optarg, "double")) c.data_type = TYPE_DOUBLE;
                else if (!strcasecmp(optarg, "int")) c.data_type = TYPE_INT;
                else if (!strcasecmp(optarg, "char")) c.data_type = TYPE_CHAR;
                else if (!strcasecmp(optarg, "bfloat16") || !strcasecmp(optarg, "bf16")) c.data_type = TYPE_BFLOAT16;
                else if (!strcasecmp(optarg, "half") || !strcasecmp(optarg, "float16") || !strcasecmp(optarg, "fp16")) c.data_type = TYPE_HALF;
                else {
                    fprintf(stderr, "Unknown data type: '%s' (options: float, double, int, char, bfloat16, half)\n", optarg);
                    exit(1);
                }
                break;
            case 'c': c.save_csv = 1; break;
            case 'o': copy_path(c.csv_path, sizeof(c.csv_path), optarg); break;
            case 'b': c.save_binary = 1; break;
            case 'B': copy_path(c.bin_path, sizeof(c.bin_path), optarg); break;
            case 'S': copy_path(c.save_ref_path, sizeof(c.save_ref_path), optarg); break;
            case 'R': copy_path(c.ref_dir, sizeof(c.ref_dir), optarg); break;
            case 'h': usage(argv[0]); exit(0);
            default: usage(argv[0]); exit(1);
        }
    }
    return c;
}

/* ------------------------------------------------------------- size iterator */
void size_iter_init(size_iter_t *it, const test_config_t *config) {
    memset(it, 0, sizeof(*it));
    it->use_list = config->use_size_list;
    it->num_sizes = config->num_sizes;
    memcpy(it->size_list, config->size_list, sizeof(it->size_list));
    it->min_size = config->min_message_size;
    it->max_size = config->max_message_size;
    it->incr = config->message_size_incr;
    it->incr_mode = config->message_size_incr_mode;
}

int size_iter_next(size_iter_t *it, size_t *size) {
    if (it->use_list) {
        if (it->index >= it->num_sizes) return 0;
        *size = it->size_list[it->index++];
        return 1;
    }
    size_t cur = it->min_size;
    if (it->incr_mode) {
        cur = it->min_size + (size_t)it->index * (size_t)(it->incr > 0 ? it->incr : 1);
    } else {
        const size_t f = it->incr > 1 ? (size_t)it->incr : 2;
        for (int k = 0; k < it->index; ++k) {
            if (cur > it->max_size) break;
            cur = cur ? cur * f : 1;
        }
    }
    if (cur > it->max_size) return 0;
    it->index++;
    *size = cur;
    return 1;
}

/* -------------------------------------------------------------- oracle cache */
static const char *dtype_tag(data_type_t t) {
    return t == TYPE_INT ? "int" : t == TYPE_FLOAT ? "float" : t == TYPE_DOUBLE ? "double" : t == TYPE_BFLOAT16 ? "bfloat16"
           : t == TYPE_HALF ? "half" : "char";
}

static void ref_cache_name(char *out, size_t cap, const char *dir, const test_config_t *cfg, const char *collective,
                           int nranks, int rank, size_t bytes) {
    snprintf(out, cap, "%s/%s_n%d_r%d_%s_p%d_%zu.ref", dir, collective, nranks, rank, dtype_tag(cfg->data_type),
             (int)cfg->pattern_type, bytes);
}

int ref_cache_load(const test_config_t *cfg, const char *collective, int nranks, int rank, void *buf, size_t bytes) {
    if (!cfg->ref_dir[0]) return 0;
    char path[1024];
    ref_cache_name(path, sizeof(path), cfg->ref_dir, cfg, collective, nranks, rank, bytes);
    FILE *f = fopen(path, "rb");
    if (!f) return 0;
    size_t got = fread(buf, 1, bytes, f);
    fclose(f);
    return got == bytes;
}

int ref_cache_store(const test_config_t *cfg, const char *collective, int nranks, int rank, const void *buf,
                    size_t bytes) {
    if (!cfg->save_ref_path[0]) return 0;
    mkdir(cfg->save_ref_path, 0755);
    char path[1024], tmp[1100];
    ref_cache_name(path, sizeof(path), cfg->save_ref_path, cfg, collective, nranks, rank, bytes);
    snprintf(tmp, sizeof(tmp), "%s.tmp", path);
    FILE *f = fopen(tmp, "wb");
    if (!f) return 0;
    size_t put = fwrite(buf, 1, bytes, f);
    fclose(f);
    if (put != bytes) {
        remove(tmp);
        return 0;
    }
    return rename(tmp, path) == 0;
}

int csv_has_size(const char *path, size_t msg_size, int nranks) {
    FILE *f = fopen(path, "r");
    if (!f) return 0;
    char line[2048];
    int found = 0;
    while (fgets(line, sizeof(line), f)) {
        unsigned long long sz = 0;
        int n = 0;
        if (sscanf(line, "%llu,%d,", &sz, &n) == 2 && sz == msg_size && n == nranks) {
            found = 1;
            break;
        }
    }
    fclose(f);
    return found;
}

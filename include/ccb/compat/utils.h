/* Benchmark-core basics: element types, data patterns, file I/O, the argv
 * front-end and the message-size iterator. Source-compatible with the reference's
 * run_codes/benchmark-core/include/utils.h (same type, field and function names), so
 * benchmark drivers and user code written against it compile unchanged. */
#ifndef UTILS_H
#define UTILS_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* The reference has the first four (run_codes/benchmark-core/include/utils.h:13-18); the
 * 16-bit floating types are additions, appended so that the reference's values keep
 * their numbers. `-d bfloat16` (bf16) and `-d half` (float16, fp16) select them. */
typedef enum { TYPE_INT, TYPE_FLOAT, TYPE_DOUBLE, TYPE_CHAR, TYPE_BFLOAT16, TYPE_HALF } data_type_t;

/* 16-bit floats on the host: stored as their bit patterns, converted with round to
 * nearest even, NaN kept. */
static inline float ccb_bf16_to_float(uint16_t h) {
    union { uint32_t u; float f; } v;
    v.u = (uint32_t)h << 16;
    return v.f;
}
static inline uint16_t ccb_float_to_bf16(float f) {
    union { uint32_t u; float f; } v;
    v.f = f;
    if ((v.u & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((v.u >> 16) | 0x40u); /* NaN */
    return (uint16_t)((v.u + 0x7fffu + ((v.u >> 16) & 1u)) >> 16);
}
static inline float ccb_half_to_float(uint16_t h) {
    union { uint32_t u; float f; } v;
    const uint32_t sign = (uint32_t)(h & 0x8000u) << 16, exp = (h >> 10) & 0x1fu, man = h & 0x3ffu;
    if (exp == 0x1fu) v.u = sign | 0x7f800000u | (man << 13);
    else if (exp) v.u = sign | ((exp + 112u) << 23) | (man << 13);
    else if (man) {
        int e = -1;
        uint32_t m = man;
        do { ++e; m <<= 1; } while (!(m & 0x400u));
        v.u = sign | ((uint32_t)(112 - e) << 23) | ((m & 0x3ffu) << 13);
    } else v.u = sign;
    return v.f;
}
static inline uint16_t ccb_float_to_half(float f) {
    union { uint32_t u; float f; } v;
    v.f = f;
    const uint32_t sign = (v.u >> 16) & 0x8000u, a = v.u & 0x7fffffffu;
    if (a > 0x7f800000u) return (uint16_t)(sign | 0x7e00u);                 /* NaN */
    if (a >= 0x477ff000u) return (uint16_t)(sign | 0x7c00u);                /* rounds to infinity */
    if (a < 0x33000001u) return (uint16_t)sign;                             /* rounds to zero */
    if (a < 0x38800000u) {                                                  /* subnormal half */
        const uint32_t shift = 126u - (a >> 23), m = (a & 0x7fffffu) | 0x800000u;
        const uint32_t q = m >> shift, rem = m & ((1u << shift) - 1u), half = 1u << (shift - 1);
        return (uint16_t)(sign | (q + (rem > half || (rem == half && (q & 1u)))));
    }
    const uint32_t q = (a - 0x38000000u) >> 13, rem = a & 0x1fffu;
    return (uint16_t)(sign | (q + (rem > 0x1000u || (rem == 0x1000u && (q & 1u)))));
}

typedef enum {
    PATTERN_PLAIN = 0,        /* every element 1                  */
    PATTERN_RANK_LINEAR = 1,  /* rank + i                         */
    PATTERN_RANK_PRODUCT = 2, /* (rank + 1) * (i + 1)             */
    PATTERN_SEQUENTIAL = 3    /* rank * count + i                 */
} pattern_type_t;

typedef enum { FILE_FORMAT_BINARY, FILE_FORMAT_TEXT } file_format_t;

int read_from_file(const char *filename, void *buffer, size_t buffer_size, file_format_t format,
                   data_type_t datatype);
int write_to_file(const char *filename, const void *buffer, size_t buffer_size, file_format_t format,
                  data_type_t datatype);
void *allocate_aligned_buffer(size_t size, size_t alignment);
void free_aligned_buffer(void *ptr);
pattern_type_t parse_pattern_type(const char *name);
void init_buffer_pattern(void *buffer, int count, data_type_t datatype, pattern_type_t pattern_type, int rank);
void print_buffer(const void *buffer, int count, data_type_t datatype, int max_to_print);

typedef struct {
    int use_list;
    int index;
    int num_sizes;
    size_t size_list[256];
    size_t min_size, max_size;
    int incr;
    int incr_mode; /* 0 = multiply, 1 = add */
} size_iter_t;

typedef struct {
    size_t min_message_size;
    size_t max_message_size;
    int message_size_incr;
    int message_size_incr_mode; /* 0 = multiply, 1 = add (-A) */
    int use_size_list;          /* -L X,Y,Z */
    int num_sizes;
    size_t size_list[256];
    int iterations;
    int warmup_iterations;
    int save_csv;               /* -c */
    char csv_path[512];         /* -o */
    int save_binary;            /* -b */
    char bin_path[512];         /* -B */
    char *input_file;           /* -f */
    file_format_t file_format;
    double tolerance;           /* -t */
    int validate;               /* -v */
    int compute_metrics;        /* -M / -e */
    uint32_t metrics_mask;
    pattern_type_t pattern_type;
    data_type_t data_type;
    char save_ref_path[512];    /* -S DIR: store the oracle's results under DIR */
    char ref_dir[512];          /* -R DIR: load the oracle's results from DIR   */
} test_config_t;

test_config_t parse_arguments(int argc, char **argv);
void size_iter_init(size_iter_t *it, const test_config_t *config);
int size_iter_next(size_iter_t *it, size_t *size);

/* Additions of this implementation. */
/* Oracle cache used by -S / -R: <dir>/<collective>_n<nranks>_r<rank>_<dtype>_<bytes>.ref */
int ref_cache_load(const test_config_t *cfg, const char *collective, int nranks, int rank, void *buf, size_t bytes);
int ref_cache_store(const test_config_t *cfg, const char *collective, int nranks, int rank, const void *buf,
                    size_t bytes);
/* 1 when a result CSV already holds a row for (msg_size, nranks): lets a sweep resume. */
int csv_has_size(const char *path, size_t msg_size, int nranks);

#ifdef __cplusplus
}
#endif
#endif /* UTILS_H */

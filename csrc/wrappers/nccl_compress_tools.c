/* Host-codec transport helpers for NCCL wrappers.
 *
 * Same contract as the reference (run_codes/wrappers/nccl_compress_tools.h:33-38,
 * nccl_compress_tools.c:113-166): `buf` is a CPU (host) buffer; it is compressed with
 * nccl_compress into the fixed-size wire, uploaded to a device staging buffer and sent
 * with ncclSend as bytes; the receive side mirrors it and decompresses straight into
 * the caller's host buffer. exchange = grouped send + receive (:171-229);
 * nccl_reduce_cpu for f32/f64/i32/i64 with sum/prod/max/min (:234-293).
 * Beyond the reference, a DEVICE (or managed) pointer is accepted too: it is staged
 * through pinned host memory on the way in and out (cudaPointerGetAttributes tells the
 * two apart). The reference allocates and frees device and host staging on every call
 * and synchronises twice; here staging is a per-thread cache that only grows, pinned
 * so the copies are asynchronous. */
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include "nccl_compress_tools.h"

size_t nccl_type_size(ncclDataType_t t) {
    switch (t) {
        case ncclInt8: case ncclUint8: return 1;
        case ncclFloat16: return 2;
        case ncclInt32: case ncclUint32: case ncclFloat32: return 4;
        case ncclInt64: case ncclUint64: case ncclFloat64: return 8;
        default: return (int)t == 9 ? 2 : 1; /* 9 = bfloat16 */
    }
}

__attribute__((weak)) int compression_enabled(void) { return 1; }

__attribute__((weak)) int nccl_compress(void *input, size_t input_size, void *output, size_t *output_size) {
    memcpy(output, input, input_size);
    *output_size = input_size;
    return 0;
}
__attribute__((weak)) int nccl_decompress(void *input, size_t input_size, void *output, size_t output_size) {
    memcpy(output, input, input_size < output_size ? input_size : output_size);
    return 0;
}

typedef struct {
    void *host_raw, *host_wire, *dev_wire;
    size_t raw_cap, wire_cap;
} stage_t;
static __thread stage_t g_send, g_recv;

static int stage_reserve(stage_t *s, size_t raw, size_t wire) {
    if (raw > s->raw_cap) {
        if (s->host_raw) cudaFreeHost(s->host_raw);
        if (cudaMallocHost(&s->host_raw, raw) != cudaSuccess) return -1;
        s->raw_cap = raw;
    }
    if (wire > s->wire_cap) {
        if (s->host_wire) cudaFreeHost(s->host_wire);
        if (s->dev_wire) cudaFree(s->dev_wire);
        if (cudaMallocHost(&s->host_wire, wire) != cudaSuccess || cudaMalloc(&s->dev_wire, wire) != cudaSuccess) return -1;
        s->wire_cap = wire;
    }
    return 0;
}

/* 1 when the CUDA runtime knows `p` as device or managed memory, 0 for host memory
 * (pinned, registered or plain malloc). */
static int on_device(const void *p) {
    struct cudaPointerAttributes a;
    if (cudaPointerGetAttributes(&a, p) != cudaSuccess) {
        (void)cudaGetLastError(); /* older runtimes report plain host memory as an error */
        return 0;
    }
    return a.type == cudaMemoryTypeDevice || a.type == cudaMemoryTypeManaged;
}

/* caller's data (host, or device staged through pinned memory) -> wire on the device (in s->dev_wire) */
static int pack(stage_t *s, const void *buf, size_t n, cudaStream_t stream) {
    const size_t wire = nccl_max_wire_size(n);
    const int dev = on_device(buf);
    if (stage_reserve(s, dev ? n : 0, wire)) return -1;
    void *raw = (void *)buf;
    if (dev) {
        if (cudaMemcpyAsync(s->host_raw, buf, n, cudaMemcpyDeviceToHost, stream) != cudaSuccess) return -1;
        if (cudaStreamSynchronize(stream) != cudaSuccess) return -1;
        raw = s->host_raw;
    }
    unsigned char *w = (unsigned char *)s->host_wire;
    size_t out = wire - sizeof(uint64_t);
    if (!compression_enabled() || nccl_compress(raw, n, w + sizeof(uint64_t), &out) != 0 || out > wire - sizeof(uint64_t)) {
        memcpy(w + sizeof(uint64_t), raw, n); /* fall back to the raw bytes */
        out = n;
    }
    uint64_t sz = out;
    memcpy(w, &sz, sizeof(sz));
    memset(w + sizeof(uint64_t) + out, 0, wire - sizeof(uint64_t) - out);
    return cudaMemcpyAsync(s->dev_wire, w, wire, cudaMemcpyHostToDevice, stream) == cudaSuccess ? 0 : -1;
}

/* wire on the device (s->dev_wire) -> caller's data (host directly, device through pinned memory) */
static int unpack(stage_t *s, void *buf, size_t n, cudaStream_t stream) {
    const size_t wire = nccl_max_wire_size(n);
    const int dev = on_device(buf);
    if (dev && stage_reserve(s, n, wire)) return -1;
    if (cudaMemcpyAsync(s->host_wire, s->dev_wire, wire, cudaMemcpyDeviceToHost, stream) != cudaSuccess) return -1;
    if (cudaStreamSynchronize(stream) != cudaSuccess) return -1;
    unsigned char *w = (unsigned char *)s->host_wire;
    uint64_t sz = 0;
    memcpy(&sz, w, sizeof(sz));
    if (sz > wire - sizeof(uint64_t)) return -1;
    void *raw = dev ? s->host_raw : buf;
    if (!compression_enabled()) {
        memcpy(raw, w + sizeof(uint64_t), n);
    } else if (nccl_decompress(w + sizeof(uint64_t), (size_t)sz, raw, n) != 0) {
        return -1;
    }
    if (!dev) return 0;
    if (cudaMemcpyAsync(buf, s->host_raw, n, cudaMemcpyHostToDevice, stream) != cudaSuccess) return -1;
    return cudaStreamSynchronize(stream) == cudaSuccess ? 0 : -1;
}

__attribute__((weak)) int nccl_send_compressed(const void *buf, size_t data_bytes, int peer, ncclComm_t comm, cudaStream_t stream) {
    if (data_bytes == 0) return 0;
    if (pack(&g_send, buf, data_bytes, stream)) return 1;
    if (ncclSend(g_send.dev_wire, nccl_max_wire_size(data_bytes), ncclUint8, peer, comm, stream) != ncclSuccess) return 1;
    return cudaStreamSynchronize(stream) != cudaSuccess;
}

__attribute__((weak)) int nccl_recv_decompress(void *buf, size_t data_bytes, int peer, ncclComm_t comm, cudaStream_t stream) {
    if (data_bytes == 0) return 0;
    if (stage_reserve(&g_recv, 0, nccl_max_wire_size(data_bytes))) return 1;
    if (ncclRecv(g_recv.dev_wire, nccl_max_wire_size(data_bytes), ncclUint8, peer, comm, stream) != ncclSuccess) return 1;
    return unpack(&g_recv, buf, data_bytes, stream) != 0;
}

__attribute__((weak)) int nccl_exchange_compressed(const void *sendbuf, size_t send_bytes, void *recvbuf, size_t recv_bytes, int dst,
                                                   int src, ncclComm_t comm, cudaStream_t stream) {
    if (send_bytes && pack(&g_send, sendbuf, send_bytes, stream)) return 1;
    if (recv_bytes && stage_reserve(&g_recv, 0, nccl_max_wire_size(recv_bytes))) return 1;
    if (ncclGroupStart() != ncclSuccess) return 1;
    int bad = 0;
    if (send_bytes) bad |= ncclSend(g_send.dev_wire, nccl_max_wire_size(send_bytes), ncclUint8, dst, comm, stream) != ncclSuccess;
    if (recv_bytes) bad |= ncclRecv(g_recv.dev_wire, nccl_max_wire_size(recv_bytes), ncclUint8, src, comm, stream) != ncclSuccess;
    bad |= ncclGroupEnd() != ncclSuccess;
    if (bad) return 1;
    if (recv_bytes) return unpack(&g_recv, recvbuf, recv_bytes, stream) != 0;
    return cudaStreamSynchronize(stream) != cudaSuccess;
}

#define REDUCE_LOOP(T)                                                                    \
    do {                                                                                  \
        T *d = (T *)dst;                                                                  \
        const T *s = (const T *)src;                                                      \
        switch (op) {                                                                     \
            case ncclSum: for (size_t i = 0; i < count; ++i) d[i] += s[i]; break;         \
            case ncclProd: for (size_t i = 0; i < count; ++i) d[i] *= s[i]; break;        \
            case ncclMax: for (size_t i = 0; i < count; ++i) if (s[i] > d[i]) d[i] = s[i]; break; \
            case ncclMin: for (size_t i = 0; i < count; ++i) if (s[i] < d[i]) d[i] = s[i]; break; \
            default: return 1;                                                            \
        }                                                                                 \
    } while (0)

int nccl_reduce_cpu(void *dst, const void *src, size_t count, ncclDataType_t dtype, ncclRedOp_t op) {
    switch (dtype) {
        case ncclFloat32: REDUCE_LOOP(float); return 0;
        case ncclFloat64: REDUCE_LOOP(double); return 0;
        case ncclInt32: REDUCE_LOOP(int32_t); return 0;
        case ncclInt64: REDUCE_LOOP(int64_t); return 0;
        default: return 1;
    }
}

"""nccl_send_compressed / nccl_recv_decompress / nccl_exchange_compressed on HOST buffers (the
reference's contract, run_codes/wrappers/nccl_compress_tools.h:33-38), linked on the CPU
against stand-ins for the CUDA runtime and NCCL: "device" memory is malloc'd memory that the
stand-in remembers, ncclSend appends the bytes to a queue and ncclRecv pops them."""
import ctypes
import subprocess
from pathlib import Path

import numpy as np
import pytest

ROOT = Path(__file__).resolve().parent.parent

FAKE = r'''
#include <stdlib.h>
#include <string.h>
#include <stdint.h>
#include <cuda_runtime.h>
#include <nccl.h>
static void *dev_ptrs[64]; static size_t dev_sizes[64]; static int ndev;
static unsigned char *queue[16]; static size_t qsize[16]; static int qhead, qtail;
static int d2h_copies, h2d_copies;
cudaError_t cudaMalloc(void **p, size_t n) { *p = malloc(n); dev_ptrs[ndev] = *p; dev_sizes[ndev++] = n; return cudaSuccess; }
cudaError_t cudaFree(void *p) { for (int i = 0; i < ndev; ++i) if (dev_ptrs[i] == p) dev_ptrs[i] = 0; free(p); return cudaSuccess; }
cudaError_t cudaMallocHost(void **p, size_t n) { *p = malloc(n); return cudaSuccess; }
cudaError_t cudaFreeHost(void *p) { free(p); return cudaSuccess; }
cudaError_t cudaStreamSynchronize(cudaStream_t s) { (void)s; return cudaSuccess; }
cudaError_t cudaGetLastError(void) { return cudaSuccess; }
static int is_dev(const void *p) {
    for (int i = 0; i < ndev; ++i)
        if (dev_ptrs[i] && (const char *)p >= (char *)dev_ptrs[i] && (const char *)p < (char *)dev_ptrs[i] + dev_sizes[i]) return 1;
    return 0;
}
cudaError_t cudaPointerGetAttributes(struct cudaPointerAttributes *a, const void *p) {
    memset(a, 0, sizeof(*a));
    a->type = is_dev(p) ? cudaMemoryTypeDevice : cudaMemoryTypeUnregistered;
    return cudaSuccess;
}
cudaError_t cudaMemcpyAsync(void *d, const void *s, size_t n, enum cudaMemcpyKind k, cudaStream_t st) {
    (void)st;
    if (k == cudaMemcpyDeviceToHost) { if (!is_dev(s) || is_dev(d)) return cudaErrorInvalidValue; ++d2h_copies; }
    if (k == cudaMemcpyHostToDevice) { if (is_dev(s) || !is_dev(d)) return cudaErrorInvalidValue; ++h2d_copies; }
    memcpy(d, s, n);
    return cudaSuccess;
}
ncclResult_t ncclSend(const void *b, size_t n, ncclDataType_t t, int peer, ncclComm_t c, cudaStream_t s) {
    (void)peer; (void)c; (void)s;
    if (t != ncclUint8 || !is_dev(b)) return ncclInvalidArgument;
    queue[qtail % 16] = malloc(n); memcpy(queue[qtail % 16], b, n); qsize[qtail % 16] = n; ++qtail;
    return ncclSuccess;
}
ncclResult_t ncclRecv(void *b, size_t n, ncclDataType_t t, int peer, ncclComm_t c, cudaStream_t s) {
    (void)peer; (void)c; (void)s;
    if (t != ncclUint8 || !is_dev(b) || qhead == qtail || qsize[qhead % 16] != n) return ncclInvalidArgument;
    memcpy(b, queue[qhead % 16], n); free(queue[qhead % 16]); ++qhead;
    return ncclSuccess;
}
ncclResult_t ncclGroupStart(void) { return ncclSuccess; }
ncclResult_t ncclGroupEnd(void) { return ncclSuccess; }
/* test access */
size_t fake_queued_size(void) { return qhead == qtail ? 0 : qsize[qhead % 16]; }
const unsigned char *fake_queued(void) { return qhead == qtail ? 0 : queue[qhead % 16]; }
int fake_copies(void) { return d2h_copies * 1000 + h2d_copies; }
void *fake_device_alloc(size_t n) { void *p; cudaMalloc(&p, n); return p; }
/* a halving "codec": keeps every second byte, proves that the hooks are called */
int nccl_compress(void *in, size_t n, void *out, size_t *outn) {
    for (size_t i = 0; i < n / 2; ++i) ((unsigned char *)out)[i] = ((unsigned char *)in)[2 * i];
    *outn = n / 2; return 0;
}
int nccl_decompress(void *in, size_t n, void *out, size_t outn) {
    for (size_t i = 0; i < n && 2 * i + 1 < outn + 1; ++i) { ((unsigned char *)out)[2 * i] = ((unsigned char *)in)[i]; if (2 * i + 1 < outn) ((unsigned char *)out)[2 * i + 1] = 0; }
    return 0;
}
'''


@pytest.fixture(scope="module")
def tools(tmp_path_factory):
    d = tmp_path_factory.mktemp("ct")
    (d / "fake.c").write_text(FAKE)
    so = d / "libtools_cpu.so"
    inc = ["-I" + str(ROOT / "include/ccb/compat"), "-I/usr/local/cuda/include"]
    subprocess.run(["gcc", "-shared", "-fPIC", "-O1", "-Wl,-Bsymbolic", *inc, str(d / "fake.c"), str(ROOT / "csrc/wrappers/nccl_compress_tools.c"),
                    "-o", str(so)], check=True)
    L = ctypes.CDLL(str(so))
    L.fake_queued.restype = ctypes.POINTER(ctypes.c_ubyte)
    L.fake_queued_size.restype = ctypes.c_size_t
    L.fake_device_alloc.restype = ctypes.c_void_p
    L.fake_device_alloc.argtypes = [ctypes.c_size_t]
    for f in (L.nccl_send_compressed, L.nccl_recv_decompress):
        f.argtypes = [ctypes.c_void_p, ctypes.c_size_t, ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p]
    L.nccl_exchange_compressed.argtypes = [ctypes.c_void_p, ctypes.c_size_t, ctypes.c_void_p, ctypes.c_size_t, ctypes.c_int,
                                           ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p]
    return L


def _wire_size(n):
    return n + 8 + 64 + n // 16


def test_host_buffers_round_trip_through_the_fixed_wire(tools):
    n = 1000
    src = np.arange(n, dtype=np.uint8)
    dst = np.full(n, 255, dtype=np.uint8)
    before = tools.fake_copies()
    assert tools.nccl_send_compressed(src.ctypes.data, n, 1, None, None) == 0
    assert tools.fake_queued_size() == _wire_size(n)
    wire = np.ctypeslib.as_array(tools.fake_queued(), shape=(_wire_size(n),)).copy()
    assert int.from_bytes(wire[:8].tobytes(), "little") == n // 2          # [u64 compressed size]
    assert np.array_equal(wire[8:8 + n // 2], src[::2])                     # [payload]
    assert not wire[8 + n // 2:].any()                                      # [zero pad]
    assert tools.nccl_recv_decompress(dst.ctypes.data, n, 0, None, None) == 0
    assert np.array_equal(dst[::2], src[::2]) and not dst[1::2].any()
    # host buffers are used in place: one upload of the wire, one download, no staging of the data
    assert tools.fake_copies() - before == 1000 + 1


def test_device_buffers_are_staged(tools):
    n = 512
    dsrc, ddst = tools.fake_device_alloc(n), tools.fake_device_alloc(n)
    ctypes.memmove(dsrc, bytes(range(256)) * 2, n)
    before = tools.fake_copies()
    assert tools.nccl_send_compressed(dsrc, n, 1, None, None) == 0
    assert tools.nccl_recv_decompress(ddst, n, 0, None, None) == 0
    got = np.frombuffer(ctypes.string_at(ddst, n), dtype=np.uint8)
    assert np.array_equal(got[::2], np.frombuffer(bytes(range(256)) * 2, dtype=np.uint8)[::2])
    assert tools.fake_copies() - before == 2000 + 2   # data down + wire up, wire down + data up


def test_exchange_on_host_buffers(tools):
    n = 300
    a = (np.arange(n) * 7 % 251).astype(np.uint8)
    b = np.zeros(n, dtype=np.uint8)
    assert tools.nccl_exchange_compressed(a.ctypes.data, n, b.ctypes.data, n, 1, 1, None, None) == 0
    assert np.array_equal(b[::2], a[::2])

// ccb_all_reduce_noalloc: the two-shot fused AllReduce of ccb_reduce.cuh, played for
// up to CCB_NOALLOC_MAX_RANKS ranks on one GPU, with its staging arenas and flags in a
// static __device__ array instead of allocated memory. See include/ccb/ccb_noalloc.h
// for who this is for and for the rules of use.
//
// The array's name is only a host-side handle in host code: passing it to a kernel
// would hand the kernel a host address. The device address is looked up once per
// device with cudaGetSymbolAddress, with that device current, and kept.
#include <cuda_runtime.h>
#include <string.h>

#include <mutex>

#include "../rt/ccb_rt_internal.h"
#include "ccb/ccb_noalloc.h"
#include "ccb_reduce.cuh"

namespace ccb {

static __device__ __align__(256) unsigned char g_noalloc_scratch[CCB_NOALLOC_TOTAL_BYTES];

constexpr int kMaxDevices = 64;
struct DeviceSlot {
  char* base = nullptr;   // device address of g_noalloc_scratch on this device
  uint32_t epoch = 0;     // call counter that orders the flag words
  int num_sms = 0;
};
static DeviceSlot g_slots[kMaxDevices];
static std::mutex g_slots_lock;

// First use on `dev` (which is current): find the array and zero its flag regions.
static int setup_device(int dev, DeviceSlot** out) {
  if (dev < 0 || dev >= kMaxDevices) {
    set_error("device index %d out of range", dev);
    return CCB_ERR_ARG;
  }
  std::lock_guard<std::mutex> g(g_slots_lock);
  DeviceSlot& s = g_slots[dev];
  if (!s.base) {
    void* p = nullptr;
    cudaError_t e = cudaGetSymbolAddress(&p, g_noalloc_scratch);
    if (e != cudaSuccess || !p) {
      set_error("cudaGetSymbolAddress(scratch) failed: %s", cudaGetErrorString(e));
      return CCB_ERR_CUDA;
    }
    for (int r = 0; r < CCB_NOALLOC_MAX_RANKS; ++r) {
      e = cudaMemset(static_cast<char*>(p) + (size_t)r * CCB_NOALLOC_ARENA_BYTES, 0, CCB_DATA_OFFSET);
      if (e != cudaSuccess) {
        set_error("clearing the flag words failed: %s", cudaGetErrorString(e));
        return CCB_ERR_CUDA;
      }
    }
    // cudaMemset is asynchronous to the host and runs on the legacy stream: a kernel
    // launched right after on a non-blocking stream would not be ordered behind it, and a
    // zero landing on a flag that was just set would make a wait run out. Wait for it.
    e = cudaDeviceSynchronize();
    if (e != cudaSuccess) {
      set_error("clearing the flag words failed: %s", cudaGetErrorString(e));
      return CCB_ERR_CUDA;
    }
    e = cudaDeviceGetAttribute(&s.num_sms, cudaDevAttrMultiProcessorCount, dev);
    if (e != cudaSuccess || s.num_sms < 1) {
      set_error("cannot read the SM count: %s", cudaGetErrorString(e));
      return CCB_ERR_CUDA;
    }
    s.base = static_cast<char*>(p);
  }
  *out = &s;
  return CCB_OK;
}

static const void* twoshot_fn(int dtype, int codec) {
#define CCB_NA_CODEC(T)                                                                                         \
  switch (codec) {                                                                                              \
    case CCB_CODEC_NONE: return reinterpret_cast<const void*>(&reduce_kernel<T, CodecNone<T>, kTwoShot>);       \
    case CCB_CODEC_INT8: return reinterpret_cast<const void*>(&reduce_kernel<T, CodecInt8<128>, kTwoShot>);     \
    case CCB_CODEC_INT8_G256: return reinterpret_cast<const void*>(&reduce_kernel<T, CodecInt8<256>, kTwoShot>); \
    case CCB_CODEC_FP8: return reinterpret_cast<const void*>(&reduce_kernel<T, CodecFp8, kTwoShot>);            \
    case CCB_CODEC_INT4: return reinterpret_cast<const void*>(&reduce_kernel<T, CodecInt4, kTwoShot>);          \
    default: return nullptr;                                                                                    \
  }
  switch (dtype) {
    case CCB_F32: CCB_NA_CODEC(float)
    case CCB_BF16: CCB_NA_CODEC(__nv_bfloat16)
    case CCB_F16: CCB_NA_CODEC(__half)
  }
#undef CCB_NA_CODEC
  return nullptr;
}

// Status words of the calls on this device: spare control words of rank 0's part of the
// array (the kernels use words 0 and 64..72 of that region).
constexpr int kStatusCtrlWord = 128;
static uint32_t* status_words(DeviceSlot* s) {
  return reinterpret_cast<uint32_t*>(s->base + CCB_CTRL_OFFSET) + kStatusCtrlWord;
}

constexpr size_t kHalfBytes = ((CCB_NOALLOC_ARENA_BYTES - CCB_DATA_OFFSET) / 2) & ~(size_t)255;

static size_t shard_for(size_t count, int n) {
  const size_t per = (count + n - 1) / n;
  return (per + kWarpElems - 1) / kWarpElems * kWarpElems;
}
static bool fits(size_t count, int n, int dtype, int codec) {
  return 2 * (size_t)n * codec_slot_bytes(codec, dtype, shard_for(count, n)) <= kHalfBytes;
}

}  // namespace ccb

using namespace ccb;

extern "C" uint64_t ccb_noalloc_max_count(int nranks, int dtype, int codec) {
  if (nranks < 1 || nranks > CCB_NOALLOC_MAX_RANKS || !twoshot_fn(dtype, codec)) return 0;
  // slot bytes grow with the shard size in steps of 512 elements: search the largest shard
  size_t shard = 0;
  while (2 * (size_t)nranks * codec_slot_bytes(codec, dtype, shard + kWarpElems) <= kHalfBytes) shard += kWarpElems;
  return (uint64_t)shard * (uint64_t)nranks;
}

extern "C" int ccb_noalloc_status(uint32_t* words) {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess || dev < 0 || dev >= kMaxDevices) {
    set_error("cudaGetDevice failed: %s", cudaGetErrorString(e));
    return CCB_ERR_CUDA;
  }
  DeviceSlot* slot = &g_slots[dev];
  uint32_t w[CCB_STATUS_WORDS] = {};
  {
    std::lock_guard<std::mutex> g(g_slots_lock);
    if (!slot->base) {  // no call was made on this device yet
      if (words) memset(words, 0, sizeof(w));
      return CCB_OK;
    }
  }
  e = cudaMemcpy(w, status_words(slot), sizeof(w), cudaMemcpyDeviceToHost);
  if (e != cudaSuccess) {
    set_error("reading the status words failed: %s", cudaGetErrorString(e));
    return CCB_ERR_CUDA;
  }
  if (words) memcpy(words, w, sizeof(w));
  if (w[CCB_STATUS_FLAGS]) {
    set_error("a device-side wait of an earlier ccb_all_reduce_noalloc call gave up (status 0x%x, where 0x%x)",
              w[CCB_STATUS_FLAGS], w[CCB_STATUS_WHERE]);
    return CCB_ERR_TIMEOUT;
  }
  return CCB_OK;
}

extern "C" int ccb_all_reduce_noalloc(const void* const* send, void* const* recv, int nranks, uint64_t count, int dtype,
                                      int codec, ccb_stream_t stream_) {
  if (!send || !recv || nranks < 1 || nranks > CCB_NOALLOC_MAX_RANKS) {
    set_error("ccb_all_reduce_noalloc: 1 to %d ranks and non-null pointer arrays are required", CCB_NOALLOC_MAX_RANKS);
    return CCB_ERR_ARG;
  }
  const void* fn = twoshot_fn(dtype, codec);
  if (!fn) {
    set_error("ccb_all_reduce_noalloc: unsupported dtype %d / codec %d", dtype, codec);
    return CCB_ERR_UNSUPPORTED;
  }
  if (count == 0) return CCB_OK;
  if (!fits(count, nranks, dtype, codec)) {
    set_error("ccb_all_reduce_noalloc: %llu elements exceed the built-in scratch; the limit for %d ranks is %llu",
              (unsigned long long)count, nranks, (unsigned long long)ccb_noalloc_max_count(nranks, dtype, codec));
    return CCB_ERR_CAPACITY;
  }
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) {
    set_error("cudaGetDevice failed: %s", cudaGetErrorString(e));
    return CCB_ERR_CUDA;
  }
  DeviceSlot* slot = nullptr;
  int rc = setup_device(dev, &slot);
  if (rc) return rc;

  ReduceArgs a;
  memset(&a, 0, sizeof(a));
  uint32_t epoch;
  {
    std::lock_guard<std::mutex> g(g_slots_lock);
    epoch = ++slot->epoch;
    if (epoch == 0) epoch = slot->epoch = 2;  // 0 means "never signalled"
  }
  for (int r = 0; r < nranks; ++r) {
    a.c.arena[r] = slot->base + (size_t)r * CCB_NOALLOC_ARENA_BYTES;
    a.send[r] = send[r];
    a.recv[r] = recv[r];
  }
  a.c.mc_arena = nullptr;
  a.c.status = status_words(slot);  // read back by ccb_noalloc_status()
  a.c.trace = nullptr;
  a.c.timeout_ns = 10ull * 1000000000ull;
  a.c.half_bytes = kHalfBytes;
  a.c.epoch = epoch;
  a.c.nranks = nranks;
  a.count = count;
  a.shard_elems = shard_for(count, nranks);
  a.shard_pad = a.shard_elems;
  a.slot_bytes = codec_slot_bytes(codec, dtype, a.shard_pad);
  a.rank0 = 0;
  a.nlocal = nranks;
  a.op = CCB_OP_SUM;
  a.mode = CCB_MODE_ALLREDUCE;
  a.waves = 1;
  // every CTA of every rank must be resident at once: at most one CTA per SM in total
  const size_t units = (a.shard_elems < count ? a.shard_elems : (size_t)count + kWarpElems - 1) / kWarpElems;
  int cap = slot->num_sms / nranks;
  if (cap < 1) cap = 1;
  int tw = kWarps;
  while (tw > 1 && units / (size_t)tw < (size_t)cap) tw >>= 1;
  a.tile_warps = tw;
  size_t tiles = (units + tw - 1) / tw;
  if (tiles < 1) tiles = 1;
  const int ctas = tiles < (size_t)cap ? (int)tiles : cap;
  dim3 grid((unsigned)ctas, (unsigned)nranks, 1), block(kThreads, 1, 1);
  void* params[] = {&a};
  e = cudaLaunchCooperativeKernel(fn, grid, block, params, 0, static_cast<cudaStream_t>(stream_));
  if (e != cudaSuccess) {
    set_error("ccb_all_reduce_noalloc: launch failed: %s", cudaGetErrorString(e));
    return CCB_ERR_CUDA;
  }
  count_launch();
  return CCB_OK;
}

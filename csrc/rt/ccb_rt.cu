// Host runtime of libccb.so: communicator set-up (symmetric VMM arenas mapped on
// every rank, optional NVLS multicast mapping), call sequencing (epochs), grid
// sizing for co-residency, and the launchers of the fused kernels.
//
// The reference has no runtime of this kind: its wrapper keeps a per-communicator
// cudaMalloc scratch and drives every hop from the host
// (plain_nccl_compress.cu:368-436 communicator wrap, :330-360 kernel launches).
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdarg.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include <unistd.h>

#include <atomic>
#include <mutex>
#include <string>
#include <vector>

#include "../kernels/ccb_exchange.cuh"
#include "../kernels/ccb_nvls.cuh"
#include "../kernels/ccb_p2p.cuh"
#include "../kernels/ccb_linkprobe.cuh"
#include "../kernels/ccb_reduce.cuh"
#include "../kernels/ccb_ring.cuh"
#include "ccb/ccb.h"
#include "ccb_bootstrap.h"
#include "ccb_rt_internal.h"

namespace ccb {

static thread_local char g_err[512];
static std::atomic<uint64_t> g_launches{0};

void set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
  if (getenv("CCB_DEBUG")) fprintf(stderr, "[ccb] %s\n", g_err);
}
void count_launch() { g_launches.fetch_add(1, std::memory_order_relaxed); }

// ---- driver entry points, fetched through the runtime so that the library has
// ---- no link-time dependency on libcuda (it must load on hosts without a GPU).
struct Driver {
  CUresult (*MemGetAllocationGranularity)(size_t*, const CUmemAllocationProp*, CUmemAllocationGranularity_flags);
  CUresult (*MemCreate)(CUmemGenericAllocationHandle*, size_t, const CUmemAllocationProp*, unsigned long long);
  CUresult (*MemRelease)(CUmemGenericAllocationHandle);
  CUresult (*MemAddressReserve)(CUdeviceptr*, size_t, size_t, CUdeviceptr, unsigned long long);
  CUresult (*MemAddressFree)(CUdeviceptr, size_t);
  CUresult (*MemMap)(CUdeviceptr, size_t, size_t, CUmemGenericAllocationHandle, unsigned long long);
  CUresult (*MemUnmap)(CUdeviceptr, size_t);
  CUresult (*MemSetAccess)(CUdeviceptr, size_t, const CUmemAccessDesc*, size_t);
  CUresult (*MemExportToShareableHandle)(void*, CUmemGenericAllocationHandle, CUmemAllocationHandleType, unsigned long long);
  CUresult (*MemImportFromShareableHandle)(CUmemGenericAllocationHandle*, void*, CUmemAllocationHandleType);
  CUresult (*MulticastCreate)(CUmemGenericAllocationHandle*, const CUmulticastObjectProp*);
  CUresult (*MulticastAddDevice)(CUmemGenericAllocationHandle, CUdevice);
  CUresult (*MulticastBindMem)(CUmemGenericAllocationHandle, size_t, CUmemGenericAllocationHandle, size_t, size_t, unsigned long long);
  CUresult (*MulticastGetGranularity)(size_t*, const CUmulticastObjectProp*, CUmulticastGranularity_flags);
  CUresult (*MulticastUnbind)(CUmemGenericAllocationHandle, CUdevice, size_t, size_t);
  CUresult (*GetErrorString)(CUresult, const char**);
  CUresult (*DeviceGetAttribute)(int*, CUdevice_attribute, CUdevice);
  bool ok = false;
};

static Driver& driver() {
  static Driver d;
  static std::once_flag once;
  std::call_once(once, [] {
    bool all = true;
    auto get = [&](const char* name, void** fn, bool required) {
      cudaDriverEntryPointQueryResult q;
      *fn = nullptr;
      if (cudaGetDriverEntryPoint(name, fn, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess || !*fn) {
        *fn = nullptr;
        if (required) all = false;
        (void)cudaGetLastError();
      }
    };
#define CCB_GET(sym, req) get("cu" #sym, reinterpret_cast<void**>(&d.sym), req)
    CCB_GET(MemGetAllocationGranularity, true);
    CCB_GET(MemCreate, true);
    CCB_GET(MemRelease, true);
    CCB_GET(MemAddressReserve, true);
    CCB_GET(MemAddressFree, true);
    CCB_GET(MemMap, true);
    CCB_GET(MemUnmap, true);
    CCB_GET(MemSetAccess, true);
    CCB_GET(MemExportToShareableHandle, true);
    CCB_GET(MemImportFromShareableHandle, true);
    CCB_GET(GetErrorString, true);
    CCB_GET(DeviceGetAttribute, true);
    CCB_GET(MulticastCreate, false);
    CCB_GET(MulticastAddDevice, false);
    CCB_GET(MulticastBindMem, false);
    CCB_GET(MulticastGetGranularity, false);
    CCB_GET(MulticastUnbind, false);
#undef CCB_GET
    d.ok = all;
  });
  return d;
}

static const char* cu_err(CUresult r) {
  const char* s = nullptr;
  if (driver().GetErrorString) driver().GetErrorString(r, &s);
  return s ? s : "unknown driver error";
}

#define CU_TRY(call)                                              \
  do {                                                            \
    CUresult _r = (call);                                         \
    if (_r != CUDA_SUCCESS) {                                     \
      set_error("%s failed: %s", #call, cu_err(_r));              \
      return CCB_ERR_CUDA;                                        \
    }                                                             \
  } while (0)
#define RT_TRY(call)                                              \
  do {                                                            \
    cudaError_t _e = (call);                                      \
    if (_e != cudaSuccess) {                                      \
      set_error("%s failed: %s", #call, cudaGetErrorString(_e));  \
      return CCB_ERR_CUDA;                                        \
    }                                                             \
  } while (0)

static size_t round_up(size_t x, size_t m) { return (x + m - 1) / m * m; }

}  // namespace ccb

using namespace ccb;

struct ccb_comm {
  int rank0 = 0, nlocal = 1, nranks = 1, device = 0;
  size_t arena_bytes = 0;   // per rank, mapped size
  size_t half_bytes = 0;
  int call_overlap = 0;     // consecutive pipelined calls may overlap tail and head (caller's promise: disjoint buffers)
  size_t symm_top = 0;      // symmetric allocations grow down from here
  size_t symm_limit = 0;    // top of the allocatable part (below the point-to-point mailboxes)
  size_t p2p_offset = 0;    // mailboxes of ccb_p2p: [source][lane][half][p2p_lane_bytes]; 0 = none
  unsigned int p2p_lane_bytes = 0;
  unsigned int p2p_sent[CCB_MAX_RANKS] = {}, p2p_rcvd[CCB_MAX_RANKS] = {};  // rounds exchanged so far, per peer and direction
  char* arena[CCB_MAX_RANKS] = {};
  char* mc_arena = nullptr;
  uint32_t* status_host = nullptr;
  uint32_t* status_dev = nullptr;
  uint64_t timeout_ns = 10ull * 1000000000ull;
  uint32_t epoch = 0;
  int num_sms = 0;
  int max_ctas = 0;
  int waves = 0;  // 0 = choose per call
  int noncoop_ctas = 0;     // grids of at most this many CTAs are launched without the cooperative attribute
  int pipe_mode = 1;        // 0 = never use the pipelined two-shot kernel, 1 = when large enough, 2 = always
  int pipe_min_chunks = 4;  // chunks (4096 elements) per CTA from which it is used
  int pipe_link_warps = 20; // of the 31 data warps of a CTA, how many store over NVLink
  int pipe_mc = 0;          // phase 2 through the NVLS multicast mapping (measured slower at 2 and 4 GPUs: off)
  unsigned long long* trace = nullptr;  // device buffer, CCB_MAX_CTAS * nlocal * CCB_TRACE_SLOTS
  bool dead = false;
  // ownership
  bool vmm = false;
  CUdeviceptr va_base = 0;
  size_t va_size = 0;
  CUmemGenericAllocationHandle handles[CCB_MAX_RANKS] = {};
  bool mapped[CCB_MAX_RANKS] = {};
  CUmemGenericAllocationHandle mc_handle = 0;
  CUdeviceptr mc_va = 0;
  bool mc_bound = false;
  void* local_alloc[CCB_MAX_RANKS] = {};  // cudaMalloc'd arenas (local / ipc modes)
  bool ipc_opened[CCB_MAX_RANKS] = {};
};

namespace ccb {

static uint64_t env_u64(const char* name, uint64_t dflt) {
  const char* e = getenv(name);
  if (!e || !*e) return dflt;
  return strtoull(e, nullptr, 10);
}

static int finish_common(ccb_comm* c) {
  cudaDeviceProp prop;
  RT_TRY(cudaGetDeviceProperties(&prop, c->device));
  c->num_sms = prop.multiProcessorCount;
  c->timeout_ns = env_u64("CCB_TIMEOUT_MS", 10000) * 1000000ull;
  c->max_ctas = (int)env_u64("CCB_MAX_CTAS", 0);
  c->waves = (int)env_u64("CCB_WAVES", 0);
  c->noncoop_ctas = (int)env_u64("CCB_NONCOOP_CTAS", 0);
  c->pipe_mode = (int)env_u64("CCB_PIPE", 1);
  c->pipe_min_chunks = (int)env_u64("CCB_PIPE_MIN_CHUNKS", 4);
  c->pipe_link_warps = (int)env_u64("CCB_PIPE_LINK_WARPS", 20);
  if (c->pipe_link_warps < 1) c->pipe_link_warps = 1;
  if (c->pipe_link_warps > 30) c->pipe_link_warps = 30;
  c->pipe_mc = (int)env_u64("CCB_PIPE_MC", 0);
  RT_TRY(cudaHostAlloc(reinterpret_cast<void**>(&c->status_host), CCB_STATUS_WORDS * 4, cudaHostAllocMapped));
  memset(c->status_host, 0, CCB_STATUS_WORDS * 4);
  RT_TRY(cudaHostGetDevicePointer(reinterpret_cast<void**>(&c->status_dev), c->status_host, 0));
  // Point-to-point mailboxes at the top of the arena (1/64 of it per source, at most 8 MiB):
  // two halves per (source, lane). Communicators with one rank, or playing several ranks
  // in one process, have none.
  c->symm_limit = c->arena_bytes;
  if (c->nranks > 1 && c->nlocal == 1) {
    size_t lane = c->arena_bytes / 64 / (2 * kP2pLanes);
    if (lane > (256u << 10)) lane = 256u << 10;
    lane &= ~(size_t)255;
    const size_t total = (size_t)CCB_MAX_RANKS * kP2pLanes * 2 * lane;
    if (lane >= 4096 && total + CCB_DATA_OFFSET < c->arena_bytes / 2) {
      c->p2p_lane_bytes = (unsigned int)lane;
      c->p2p_offset = (c->arena_bytes - total) & ~(size_t)4095;
      c->symm_limit = c->p2p_offset;
    }
  }
  c->symm_top = c->symm_limit;
  c->half_bytes = ((c->symm_top - CCB_DATA_OFFSET) / 2) & ~(size_t)255;
  return CCB_OK;
}

CommDev comm_dev(ccb_comm* c, uint32_t epoch) {
  CommDev d;
  memset(&d, 0, sizeof(d));
  for (int i = 0; i < c->nranks; ++i) d.arena[i] = c->arena[i];
  d.mc_arena = c->mc_arena;
  d.status = c->status_dev;
  d.trace = c->trace;
  d.timeout_ns = c->timeout_ns;
  d.half_bytes = c->half_bytes;
  d.epoch = epoch;
  d.nranks = c->nranks;
  return d;
}

uint32_t next_epoch(ccb_comm* c) {
  ++c->epoch;
  if (c->epoch == 0) c->epoch = 2;  // keep parity alternating across the wrap; 0 is "never"
  return c->epoch;
}

// How many CTAs per rank may be launched so that every CTA of every local rank is
// resident at once (CTAs spin on flags written by same-numbered CTAs elsewhere).
int grid_cap(ccb_comm* c, const void* kernel, int threads) {
  int per_sm = 0;
  if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, threads, 0) != cudaSuccess || per_sm < 1) {
    (void)cudaGetLastError();
    per_sm = 1;
  }
  if (per_sm > 2) per_sm = 2;
  int cap = per_sm * c->num_sms / c->nlocal;
  if (cap > CCB_MAX_CTAS) cap = CCB_MAX_CTAS;
  if (c->max_ctas > 0 && cap > c->max_ctas) cap = c->max_ctas;
  return cap < 1 ? 1 : cap;
}

int launch(ccb_comm* c, const void* kernel, int ctas, void* args, cudaStream_t stream, int threads, bool may_overlap) {
  dim3 grid((unsigned)ctas, (unsigned)c->nlocal, 1), block((unsigned)threads, 1, 1);
  void* params[] = {args};
  // Consecutive calls may overlap tail and head (ccb_comm_set_call_overlap): the launch is
  // plain and carries the programmatic-serialisation attribute, so its CTAs start on the SMs
  // that the CTAs of the call before leave, instead of after the slowest of them. The kernel
  // says "dependents may launch" at its start and never waits for the grid before it: the
  // caller has promised that consecutive calls touch different user buffers, and the staging
  // halves and flags alternate by epoch. One CTA of 1024 threads fills an SM, so the call
  // after the next cannot start before this one has left the device.
  if (may_overlap && c->call_overlap && c->nlocal == 1) {
    cudaLaunchConfig_t cfg;
    memset(&cfg, 0, sizeof(cfg));
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.stream = stream;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    cudaError_t e = cudaLaunchKernelExC(&cfg, kernel, params);
    if (e != cudaSuccess) {
      set_error("kernel launch failed: %s", cudaGetErrorString(e));
      return CCB_ERR_CUDA;
    }
    count_launch();
    return CCB_OK;
  }
  // A cooperative launch starts only when the WHOLE grid fits beside what is running, so
  // behind a stream of GEMMs it waits for a full wave to drain. With one rank per launch
  // no CTA waits on another CTA of its own grid (only on the same-numbered CTA of the
  // peers, whose GPUs make progress independently), so a small grid may be launched
  // plainly: its CTAs start one by one as SMs free up. Launches that play several ranks
  // (CTAs of one grid wait on each other) always stay cooperative.
  const bool plain = c->nlocal == 1 && c->noncoop_ctas > 0 && ctas <= c->noncoop_ctas;
  cudaError_t e = plain ? cudaLaunchKernel(kernel, grid, block, params, 0, stream)
                        : cudaLaunchCooperativeKernel(kernel, grid, block, params, 0, stream);
  if (e != cudaSuccess) {
    set_error("kernel launch failed: %s", cudaGetErrorString(e));
    return CCB_ERR_CUDA;
  }
  count_launch();
  return CCB_OK;
}

int check_alive(ccb_comm* c) {
  if (!c) {
    set_error("null communicator");
    return CCB_ERR_ARG;
  }
  if (c->dead || (c->status_host && c->status_host[CCB_STATUS_FLAGS] != 0)) {
    c->dead = true;
    set_error("communicator is dead: a device-side wait gave up (status 0x%x, where 0x%x)",
              c->status_host[CCB_STATUS_FLAGS], c->status_host[CCB_STATUS_WHERE]);
    return CCB_ERR_TIMEOUT;
  }
  return CCB_OK;
}

size_t elem_size(int dtype) { return dtype == CCB_F32 ? 4 : 2; }

size_t codec_slot_bytes(int codec, int dtype, size_t pad) {
  size_t b;
  switch (codec) {
    case CCB_CODEC_INT8: b = pad + pad / 128 * 4; break;
    case CCB_CODEC_INT8_G256: b = pad + pad / 256 * 4; break;
    case CCB_CODEC_FP8: b = pad + pad / 32; break;
    case CCB_CODEC_INT4: b = pad / 2 + pad / 128 * 4; break;
    default: b = pad * elem_size(dtype); break;
  }
  return round_up(b, 256);
}

}  // namespace ccb

// =============================================================== creation ====
extern "C" int ccb_comm_create_local(ccb_comm** out, int nranks, uint64_t arena_bytes) {
  if (!out || nranks < 1 || nranks > CCB_MAX_RANKS) {
    set_error("nranks must be in [1, %d]", CCB_MAX_RANKS);
    return CCB_ERR_ARG;
  }
  ccb_comm* c = new ccb_comm();
  c->rank0 = 0;
  c->nlocal = c->nranks = nranks;
  RT_TRY(cudaGetDevice(&c->device));
  if (arena_bytes == 0) arena_bytes = env_u64("CCB_ARENA_MB", 256) << 20;
  c->arena_bytes = round_up(arena_bytes, 2u << 20);
  for (int r = 0; r < nranks; ++r) {
    RT_TRY(cudaMalloc(&c->local_alloc[r], c->arena_bytes));
    RT_TRY(cudaMemset(c->local_alloc[r], 0, CCB_DATA_OFFSET));
    c->arena[r] = static_cast<char*>(c->local_alloc[r]);
  }
  int rc = finish_common(c);
  if (rc != CCB_OK) return rc;
  RT_TRY(cudaDeviceSynchronize());
  *out = c;
  return CCB_OK;
}

namespace ccb {

static int setup_vmm(ccb_comm* c, Bootstrap& boot, int flags) {
  Driver& d = driver();
  if (!d.ok) {
    set_error("CUDA virtual memory management entry points are unavailable");
    return CCB_ERR_UNSUPPORTED;
  }
  const int n = c->nranks, r = c->rank0;
  CUmemAllocationProp prop;
  memset(&prop, 0, sizeof(prop));
  prop.type = CU_MEM_ALLOCATION_TYPE_PINNED;
  prop.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  prop.location.id = c->device;
  prop.requestedHandleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
  size_t gran = 0;
  CU_TRY(d.MemGetAllocationGranularity(&gran, &prop, CU_MEM_ALLOC_GRANULARITY_RECOMMENDED));
  bool want_mc = (flags & 1) && d.MulticastCreate && d.MulticastGetGranularity && n > 1;
  CUmulticastObjectProp mcp;
  memset(&mcp, 0, sizeof(mcp));
  if (want_mc) {
    int supported = 0;
    if (d.DeviceGetAttribute(&supported, CU_DEVICE_ATTRIBUTE_MULTICAST_SUPPORTED, c->device) != CUDA_SUCCESS || !supported)
      want_mc = false;
  }
  if (want_mc) {
    mcp.numDevices = (unsigned)n;
    mcp.handleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
    mcp.size = round_up(c->arena_bytes, gran);
    size_t mgran = 0;
    if (d.MulticastGetGranularity(&mgran, &mcp, CU_MULTICAST_GRANULARITY_RECOMMENDED) == CUDA_SUCCESS && mgran > gran)
      gran = mgran;
  }
  c->arena_bytes = round_up(c->arena_bytes, gran);
  mcp.size = c->arena_bytes;
  c->va_size = c->arena_bytes * (size_t)n;
  CU_TRY(d.MemCreate(&c->handles[r], c->arena_bytes, &prop, 0));
  CU_TRY(d.MemAddressReserve(&c->va_base, c->va_size, gran, 0, 0));
  c->vmm = true;
  CUmemAccessDesc acc;
  memset(&acc, 0, sizeof(acc));
  acc.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  acc.location.id = c->device;
  acc.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
  CU_TRY(d.MemMap(c->va_base + (size_t)r * c->arena_bytes, c->arena_bytes, 0, c->handles[r], 0));
  c->mapped[r] = true;
  CU_TRY(d.MemSetAccess(c->va_base + (size_t)r * c->arena_bytes, c->arena_bytes, &acc, 1));
  for (int p = 0; p < n; ++p) c->arena[p] = reinterpret_cast<char*>(c->va_base + (size_t)p * c->arena_bytes);
  RT_TRY(cudaMemset(c->arena[r], 0, CCB_DATA_OFFSET));
  RT_TRY(cudaDeviceSynchronize());

  int fd = -1;
  CU_TRY(d.MemExportToShareableHandle(&fd, c->handles[r], CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0));
  std::vector<BootMsg> msgs;
  uint64_t mysize = c->arena_bytes;
  bool okx = boot.all_gather(1, 0, &mysize, sizeof(mysize), fd, &msgs);
  ::close(fd);
  if (!okx) {
    set_error("handle exchange failed: %s", boot.error().c_str());
    return CCB_ERR_BOOTSTRAP;
  }
  for (int p = 0; p < n; ++p) {
    if (p == r) continue;
    BootMsg& m = msgs[(size_t)p];
    uint64_t psize = 0;
    if (m.payload.size() == sizeof(psize)) memcpy(&psize, m.payload.data(), sizeof(psize));
    if (m.fd < 0 || psize != c->arena_bytes) {
      set_error("rank %d sent no usable arena handle (size %llu, expected %llu)", p, (unsigned long long)psize,
                (unsigned long long)c->arena_bytes);
      return CCB_ERR_BOOTSTRAP;
    }
    CUresult ir = d.MemImportFromShareableHandle(&c->handles[p], reinterpret_cast<void*>(static_cast<uintptr_t>(m.fd)),
                                                 CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR);
    ::close(m.fd);
    m.fd = -1;
    if (ir != CUDA_SUCCESS) {
      set_error("cuMemImportFromShareableHandle(rank %d) failed: %s", p, cu_err(ir));
      return CCB_ERR_CUDA;
    }
    CU_TRY(d.MemMap(c->va_base + (size_t)p * c->arena_bytes, c->arena_bytes, 0, c->handles[p], 0));
    c->mapped[p] = true;
    CU_TRY(d.MemSetAccess(c->va_base + (size_t)p * c->arena_bytes, c->arena_bytes, &acc, 1));
  }

  // ---- optional NVLS multicast mapping of the same physical arenas ----------
  // Every rank must reach the same verdict, so each step is followed by a vote.
  if (n > 1) {
    int vote = want_mc ? 1 : 0;
    std::vector<BootMsg> votes;
    if (!boot.all_gather(2, 0, &vote, sizeof(vote), -1, &votes)) {
      set_error("multicast vote failed: %s", boot.error().c_str());
      return CCB_ERR_BOOTSTRAP;
    }
    for (int p = 0; p < n; ++p)
      if (p != r && (votes[(size_t)p].payload.size() != sizeof(int) || *reinterpret_cast<int*>(votes[(size_t)p].payload.data()) == 0))
        want_mc = false;
  }
  if (want_mc) {
    int good = 1;
    if (r == 0) {
      int mfd = -1;
      if (d.MulticastCreate(&c->mc_handle, &mcp) != CUDA_SUCCESS ||
          d.MemExportToShareableHandle(&mfd, c->mc_handle, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0) != CUDA_SUCCESS) {
        good = 0;
        c->mc_handle = 0;
      }
      for (int p = 1; p < n; ++p) boot.send(p, 3, 0, &good, sizeof(good), good ? mfd : -1);
      if (mfd >= 0) ::close(mfd);
    } else {
      BootMsg m;
      if (!boot.recv(3, 0, 0, &m)) {
        set_error("multicast handle exchange failed: %s", boot.error().c_str());
        return CCB_ERR_BOOTSTRAP;
      }
      good = (m.payload.size() == sizeof(int)) ? *reinterpret_cast<int*>(m.payload.data()) : 0;
      if (good && m.fd >= 0) {
        if (d.MemImportFromShareableHandle(&c->mc_handle, reinterpret_cast<void*>(static_cast<uintptr_t>(m.fd)),
                                           CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR) != CUDA_SUCCESS) {
          good = 0;
          c->mc_handle = 0;
        }
      } else {
        good = 0;
      }
      if (m.fd >= 0) ::close(m.fd);
    }
    auto vote_all = [&](int seq, int mine) -> int {
      std::vector<BootMsg> vs;
      if (!boot.all_gather(4, seq, &mine, sizeof(mine), -1, &vs)) return -1;
      int all = mine;
      for (int p = 0; p < n; ++p)
        if (p != r && (vs[(size_t)p].payload.size() != sizeof(int) || *reinterpret_cast<int*>(vs[(size_t)p].payload.data()) == 0)) all = 0;
      return all;
    };
    int all = vote_all(0, good);
    if (all < 0) {
      set_error("multicast vote failed: %s", boot.error().c_str());
      return CCB_ERR_BOOTSTRAP;
    }
    if (all) {
      good = d.MulticastAddDevice(c->mc_handle, c->device) == CUDA_SUCCESS;
      all = vote_all(1, good);  // every device must be added before anyone binds
      if (all < 0) return CCB_ERR_BOOTSTRAP;
    }
    if (all) {
      good = d.MulticastBindMem(c->mc_handle, 0, c->handles[r], 0, c->arena_bytes, 0) == CUDA_SUCCESS;
      if (good) c->mc_bound = true;
      if (good) {
        good = d.MemAddressReserve(&c->mc_va, c->arena_bytes, gran, 0, 0) == CUDA_SUCCESS &&
               d.MemMap(c->mc_va, c->arena_bytes, 0, c->mc_handle, 0) == CUDA_SUCCESS &&
               d.MemSetAccess(c->mc_va, c->arena_bytes, &acc, 1) == CUDA_SUCCESS;
      }
      all = vote_all(2, good);
      if (all < 0) return CCB_ERR_BOOTSTRAP;
      if (all) c->mc_arena = reinterpret_cast<char*>(c->mc_va);
    }
  }
  return CCB_OK;
}

static int setup_ipc(ccb_comm* c, Bootstrap& boot) {
  const int n = c->nranks, r = c->rank0;
  c->arena_bytes = round_up(c->arena_bytes, 2u << 20);
  RT_TRY(cudaMalloc(&c->local_alloc[r], c->arena_bytes));
  RT_TRY(cudaMemset(c->local_alloc[r], 0, CCB_DATA_OFFSET));
  RT_TRY(cudaDeviceSynchronize());
  c->arena[r] = static_cast<char*>(c->local_alloc[r]);
  cudaIpcMemHandle_t h;
  RT_TRY(cudaIpcGetMemHandle(&h, c->local_alloc[r]));
  std::vector<BootMsg> msgs;
  if (!boot.all_gather(5, 0, &h, sizeof(h), -1, &msgs)) {
    set_error("ipc handle exchange failed: %s", boot.error().c_str());
    return CCB_ERR_BOOTSTRAP;
  }
  for (int p = 0; p < n; ++p) {
    if (p == r) continue;
    if (msgs[(size_t)p].payload.size() != sizeof(h)) {
      set_error("rank %d sent a malformed ipc handle", p);
      return CCB_ERR_BOOTSTRAP;
    }
    cudaIpcMemHandle_t ph;
    memcpy(&ph, msgs[(size_t)p].payload.data(), sizeof(ph));
    void* ptr = nullptr;
    RT_TRY(cudaIpcOpenMemHandle(&ptr, ph, cudaIpcMemLazyEnablePeerAccess));
    c->arena[p] = static_cast<char*>(ptr);
    c->ipc_opened[p] = true;
  }
  return CCB_OK;
}

}  // namespace ccb

extern "C" int ccb_comm_create(ccb_comm** out, int rank, int nranks, const char* tag, uint64_t arena_bytes, int flags) {
  if (!out || nranks < 1 || nranks > CCB_MAX_RANKS || rank < 0 || rank >= nranks || !tag) {
    set_error("bad arguments (rank %d of %d, at most %d ranks)", rank, nranks, CCB_MAX_RANKS);
    return CCB_ERR_ARG;
  }
  ccb_comm* c = new ccb_comm();
  c->rank0 = rank;
  c->nlocal = 1;
  c->nranks = nranks;
  RT_TRY(cudaGetDevice(&c->device));
  RT_TRY(cudaFree(0));
  if (arena_bytes == 0) arena_bytes = env_u64("CCB_ARENA_MB", 2048) << 20;
  c->arena_bytes = arena_bytes;
  int rc;
  {
    Bootstrap boot(rank, nranks, tag, (int)env_u64("CCB_BOOTSTRAP_TIMEOUT_MS", 60000));
    if (!boot.ok()) {
      set_error("rendezvous: %s", boot.error().c_str());
      delete c;
      return CCB_ERR_BOOTSTRAP;
    }
    const char* mem = getenv("CCB_MEM");
    if (mem && !strcmp(mem, "ipc")) rc = setup_ipc(c, boot);
    else rc = setup_vmm(c, boot, flags);
    if (rc == CCB_OK && nranks > 1 && !boot.barrier(100)) {
      set_error("rendezvous barrier: %s", boot.error().c_str());
      rc = CCB_ERR_BOOTSTRAP;
    }
  }
  if (rc == CCB_OK) rc = finish_common(c);
  if (rc != CCB_OK) {
    ccb_comm_destroy(c);
    return rc;
  }
  *out = c;
  return CCB_OK;
}

extern "C" int ccb_comm_destroy(ccb_comm* c) {
  if (!c) return CCB_OK;
  cudaDeviceSynchronize();
  Driver& d = driver();
  if (c->mc_va) {
    d.MemUnmap(c->mc_va, c->arena_bytes);
    d.MemAddressFree(c->mc_va, c->arena_bytes);
  }
  if (c->mc_bound && d.MulticastUnbind) d.MulticastUnbind(c->mc_handle, c->device, 0, c->arena_bytes);
  if (c->mc_handle) d.MemRelease(c->mc_handle);
  if (c->vmm) {
    for (int p = 0; p < c->nranks; ++p) {
      if (c->mapped[p]) d.MemUnmap(c->va_base + (size_t)p * c->arena_bytes, c->arena_bytes);
      if (c->handles[p]) d.MemRelease(c->handles[p]);
    }
    if (c->va_base) d.MemAddressFree(c->va_base, c->va_size);
  }
  for (int p = 0; p < CCB_MAX_RANKS; ++p) {
    if (c->ipc_opened[p]) cudaIpcCloseMemHandle(c->arena[p]);
    if (c->local_alloc[p]) cudaFree(c->local_alloc[p]);
  }
  if (c->status_host) cudaFreeHost(c->status_host);
  if (c->trace) cudaFree(c->trace);
  (void)cudaGetLastError();
  delete c;
  return CCB_OK;
}

extern "C" int ccb_comm_rank(const ccb_comm* c) { return c ? c->rank0 : -1; }
extern "C" int ccb_comm_nranks(const ccb_comm* c) { return c ? c->nranks : -1; }
extern "C" int ccb_comm_nlocal(const ccb_comm* c) { return c ? c->nlocal : -1; }
extern "C" int ccb_comm_has_nvls(const ccb_comm* c) { return c && c->mc_arena ? 1 : 0; }
extern "C" uint64_t ccb_comm_arena_bytes(const ccb_comm* c) { return c ? c->arena_bytes : 0; }
extern "C" int ccb_comm_set_timeout_ms(ccb_comm* c, uint64_t ms) {
  if (!c) return CCB_ERR_ARG;
  c->timeout_ns = ms * 1000000ull;
  return CCB_OK;
}
extern "C" int ccb_comm_set_max_ctas(ccb_comm* c, int ctas) {
  if (!c) return CCB_ERR_ARG;
  c->max_ctas = ctas;
  return CCB_OK;
}
// ---- symmetric allocations: user buffers inside the arena, same offset on every rank ----
extern "C" int ccb_comm_symm_alloc(ccb_comm* c, uint64_t bytes, uint64_t* offset) {
  if (!c || !offset || bytes == 0) return CCB_ERR_ARG;
  const size_t need = round_up(bytes, 4096);
  // staging keeps at least a quarter of the arena
  if (need > c->symm_top || c->symm_top - need < CCB_DATA_OFFSET + c->arena_bytes / 4) {
    set_error("symmetric allocation of %llu bytes does not fit (arena %llu bytes, %llu already taken)", (unsigned long long)bytes,
              (unsigned long long)c->arena_bytes, (unsigned long long)(c->symm_limit - c->symm_top));
    return CCB_ERR_CAPACITY;
  }
  RT_TRY(cudaDeviceSynchronize());  // no call may be using the staging that shrinks
  c->symm_top -= need;
  c->half_bytes = ((c->symm_top - CCB_DATA_OFFSET) / 2) & ~(size_t)255;
  *offset = c->symm_top;
  return CCB_OK;
}
extern "C" void* ccb_comm_symm_ptr(ccb_comm* c, uint64_t offset) {
  if (!c || offset < c->symm_top || offset >= c->symm_limit) return nullptr;
  return c->arena[c->rank0] + offset;
}
extern "C" int ccb_comm_symm_free_all(ccb_comm* c) {
  if (!c) return CCB_ERR_ARG;
  RT_TRY(cudaDeviceSynchronize());
  // Point-to-point mailboxes at the top of the arena (1/64 of it per source, at most 8 MiB):
  // two halves per (source, lane). Communicators with one rank, or playing several ranks
  // in one process, have none.
  c->symm_limit = c->arena_bytes;
  if (c->nranks > 1 && c->nlocal == 1) {
    size_t lane = c->arena_bytes / 64 / (2 * kP2pLanes);
    if (lane > (256u << 10)) lane = 256u << 10;
    lane &= ~(size_t)255;
    const size_t total = (size_t)CCB_MAX_RANKS * kP2pLanes * 2 * lane;
    if (lane >= 4096 && total + CCB_DATA_OFFSET < c->arena_bytes / 2) {
      c->p2p_lane_bytes = (unsigned int)lane;
      c->p2p_offset = (c->arena_bytes - total) & ~(size_t)4095;
      c->symm_limit = c->p2p_offset;
    }
  }
  c->symm_top = c->symm_limit;
  c->half_bytes = ((c->symm_top - CCB_DATA_OFFSET) / 2) & ~(size_t)255;
  return CCB_OK;
}
extern "C" int ccb_all_reduce_symm(ccb_comm* c, uint64_t send_off, uint64_t recv_off, uint64_t count, int dtype, ccb_stream_t stream_) {
  int rc = check_alive(c);
  if (rc) return rc;
  if (!c->mc_arena || c->nlocal != 1) {
    set_error("in-place NVLS all-reduce needs a communicator with a multicast mapping and one rank per process");
    return CCB_ERR_UNSUPPORTED;
  }
  const size_t bytes = round_up(count * elem_size(dtype), 16);
  if (count == 0) return CCB_OK;
  if (send_off < c->symm_top || recv_off < c->symm_top || send_off + bytes > c->symm_limit || recv_off + bytes > c->symm_limit ||
      (send_off & 15) || (recv_off & 15)) {
    set_error("buffers of an in-place all-reduce must come from ccb_comm_symm_alloc");
    return CCB_ERR_ARG;
  }
  const void* fn = dtype == CCB_F32    ? reinterpret_cast<const void*>(&nvls_inplace_kernel<float>)
                   : dtype == CCB_BF16 ? reinterpret_cast<const void*>(&nvls_inplace_kernel<__nv_bfloat16>)
                   : dtype == CCB_F16  ? reinterpret_cast<const void*>(&nvls_inplace_kernel<__half>)
                                       : nullptr;
  if (!fn) return CCB_ERR_UNSUPPORTED;
  ReduceArgs a;
  memset(&a, 0, sizeof(a));
  a.c = comm_dev(c, next_epoch(c));
  a.count = count;
  a.shard_elems = send_off;  // the in-place kernel reads these two fields as arena byte offsets
  a.shard_pad = recv_off;
  a.rank0 = c->rank0;
  a.nlocal = 1;
  const size_t vecs = bytes / 16, per = (vecs + c->nranks - 1) / c->nranks;
  const size_t tiles = (per + kThreads * 4 - 1) / (kThreads * 4);
  const int cap = grid_cap(c, fn);
  return launch(c, fn, tiles < (size_t)cap ? (int)(tiles ? tiles : 1) : cap, &a, static_cast<cudaStream_t>(stream_));
}
// ---- link probe ---------------------------------------------------------------------------
// Writes `bytes` from this rank into the data area of `peer`'s arena with the given store
// method (see ccb_linkprobe.cuh). No collective may be in flight on the communicator; the
// staging areas are overwritten. Time it with events on `stream`.
extern "C" int ccb_link_probe(ccb_comm* c, int method, int peer, uint64_t bytes, ccb_stream_t stream_) {
  int rc = check_alive(c);
  if (rc) return rc;
  if (method < 0 || method > 2 || peer < 0 || peer >= c->nranks || c->nlocal != 1) {
    set_error("ccb_link_probe: method 0..2, a peer rank, one rank per process");
    return CCB_ERR_ARG;
  }
  bytes &= ~(uint64_t)8191;
  if (bytes == 0 || bytes > 2 * c->half_bytes) {
    set_error("ccb_link_probe: %llu bytes do not fit the data area (%llu)", (unsigned long long)bytes, (unsigned long long)(2 * c->half_bytes));
    return CCB_ERR_CAPACITY;
  }
  LinkProbeArgs a;
  a.dst = c->arena[peer] + CCB_DATA_OFFSET;
  a.bytes = bytes;
  a.method = method;
  const size_t smem = method == 0 ? 0 : (size_t)(kProbeThreads / 32) * kProbeStages * (method == 1 ? 512 : 2048);
  static bool attr_set = false;
  if (!attr_set) {
    cudaFuncSetAttribute(link_probe_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (kProbeThreads / 32) * kProbeStages * 2048);
    attr_set = true;
  }
  int sms = 148;
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, c->device);
  link_probe_kernel<<<sms, kProbeThreads, smem, static_cast<cudaStream_t>(stream_)>>>(a);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    set_error("link probe launch failed: %s", cudaGetErrorString(e));
    return CCB_ERR_CUDA;
  }
  count_launch();
  return CCB_OK;
}

// ---- point-to-point over the peer arenas --------------------------------------------------
// ops: `nops` sends and receives of THIS rank, all launched as one kernel (what an
// ncclGroupStart/End holds, or one call). Message sizes must match at the two ends.
static int p2p_flush(ccb_comm* c, P2pArgs& a, cudaStream_t stream) {
  if (a.nops == 0) return CCB_OK;
  dim3 grid(kP2pLanes, (unsigned)a.nops, 1), block(kThreads, 1, 1);
  void* params[] = {&a};
  // the lanes of one operation do not wait on each other, and the two ends of a transfer
  // run on different GPUs: a plain launch is enough
  cudaError_t e = cudaLaunchKernel(reinterpret_cast<const void*>(&p2p_kernel), grid, block, params, 0, stream);
  a.nops = 0;
  if (e != cudaSuccess) {
    set_error("p2p launch failed: %s", cudaGetErrorString(e));
    return CCB_ERR_CUDA;
  }
  count_launch();
  return CCB_OK;
}
extern "C" int ccb_p2p(ccb_comm* c, const ccb_p2p_op* ops, int nops, ccb_stream_t stream_) {
  int rc = check_alive(c);
  if (rc) return rc;
  if (!ops || nops < 1) {
    set_error("ccb_p2p: no operations");
    return CCB_ERR_ARG;
  }
  if (!c->p2p_offset) {
    set_error("this communicator has no point-to-point mailboxes (one rank per process and an arena of at least 64 MiB are needed)");
    return CCB_ERR_UNSUPPORTED;
  }
  for (int i = 0; i < nops; ++i)
    if (ops[i].peer < 0 || ops[i].peer >= c->nranks || ops[i].peer == c->rank0 || (!ops[i].buf && ops[i].bytes)) {
      set_error("ccb_p2p: bad peer %d or null buffer", ops[i].peer);
      return CCB_ERR_ARG;
    }
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  P2pArgs a;
  memset(&a, 0, sizeof(a));
  a.c = comm_dev(c, c->epoch ? c->epoch : 1);   // point-to-point does not advance the collectives' epoch
  a.box_offset = c->p2p_offset;
  a.lane_bytes = c->p2p_lane_bytes;
  a.rank = c->rank0;
  const size_t round_bytes = (size_t)kP2pLanes * c->p2p_lane_bytes;
  for (int i = 0; i < nops; ++i) {
    const ccb_p2p_op& o = ops[i];
    if (o.bytes == 0) continue;
    // Two transfers of one direction between one pair share mailboxes and counters: the
    // second goes into a later launch (both ends split at the same place, since they see
    // the same sequence for the pair). A full batch is launched too.
    bool clash = a.nops == kP2pMaxOps;
    for (int k = 0; k < a.nops && !clash; ++k) clash = a.op[k].peer == o.peer && a.op[k].is_recv == (o.is_recv ? 1 : 0);
    if (clash && (rc = p2p_flush(c, a, stream)) != CCB_OK) return rc;
    unsigned int* ctr = o.is_recv ? &c->p2p_rcvd[o.peer] : &c->p2p_sent[o.peer];
    P2pOp& d = a.op[a.nops++];
    d.buf = o.buf;
    d.bytes = o.bytes;
    d.peer = o.peer;
    d.is_recv = o.is_recv ? 1 : 0;
    d.first_round = *ctr;
    *ctr += (unsigned int)((o.bytes + round_bytes - 1) / round_bytes);
  }
  return p2p_flush(c, a, stream);
}
extern "C" int ccb_send(ccb_comm* c, const void* buf, uint64_t bytes, int peer, ccb_stream_t stream) {
  ccb_p2p_op o = {const_cast<void*>(buf), bytes, peer, 0};
  return ccb_p2p(c, &o, 1, stream);
}
extern "C" int ccb_recv(ccb_comm* c, void* buf, uint64_t bytes, int peer, ccb_stream_t stream) {
  ccb_p2p_op o = {buf, bytes, peer, 1};
  return ccb_p2p(c, &o, 1, stream);
}
extern "C" int ccb_comm_set_call_overlap(ccb_comm* c, int on) {
  if (!c) return CCB_ERR_ARG;
  c->call_overlap = on ? 1 : 0;
  return CCB_OK;
}
extern "C" int ccb_comm_set_noncooperative(ccb_comm* c, int ctas) {
  if (!c || ctas < 0) return CCB_ERR_ARG;
  c->noncoop_ctas = ctas;
  return CCB_OK;
}
extern "C" int ccb_comm_set_trace(ccb_comm* c, int on) {
  if (!c) return CCB_ERR_ARG;
  const size_t bytes = (size_t)CCB_MAX_CTAS * CCB_MAX_RANKS * CCB_TRACE_SLOTS * sizeof(unsigned long long);
  if (on && !c->trace) {
    RT_TRY(cudaMalloc(reinterpret_cast<void**>(&c->trace), bytes));
    RT_TRY(cudaMemset(c->trace, 0, bytes));
  } else if (!on && c->trace) {
    cudaDeviceSynchronize();
    cudaFree(c->trace);
    c->trace = nullptr;
  }
  return CCB_OK;
}
/* Copies the timestamps of the last traced call: out[cta * CCB_TRACE_SLOTS + k]. */
extern "C" int ccb_comm_read_trace(ccb_comm* c, unsigned long long* out, int ctas) {
  if (!c || !c->trace || ctas < 1 || ctas > CCB_MAX_CTAS * CCB_MAX_RANKS) return CCB_ERR_ARG;
  RT_TRY(cudaMemcpy(out, c->trace, (size_t)ctas * CCB_TRACE_SLOTS * sizeof(unsigned long long), cudaMemcpyDeviceToHost));
  return CCB_OK;
}
extern "C" int ccb_comm_set_waves(ccb_comm* c, int waves) {
  if (!c || waves < 0 || waves > CCB_MAX_SLOTS / 2) return CCB_ERR_ARG;
  c->waves = waves;
  return CCB_OK;
}
/* Pipelined two-shot kernel: mode 0 never / 1 when the message is large enough / 2 always;
 * link_warps in [1, 30] (0 keeps the current value); mc != 0 lets phase 2 use the NVLS mapping. */
extern "C" int ccb_comm_set_pipeline(ccb_comm* c, int mode, int link_warps, int mc) {
  if (!c || mode < 0 || mode > 2 || link_warps < 0 || link_warps > 30) return CCB_ERR_ARG;
  c->pipe_mode = mode;
  if (link_warps > 0) c->pipe_link_warps = link_warps;
  c->pipe_mc = mc ? 1 : 0;
  return CCB_OK;
}
extern "C" int ccb_comm_status(ccb_comm* c, uint32_t* words) {
  if (!c) return CCB_ERR_ARG;
  if (words) memcpy(words, c->status_host, CCB_STATUS_WORDS * 4);
  if (c->status_host[CCB_STATUS_FLAGS]) {
    c->dead = true;
    return CCB_ERR_TIMEOUT;
  }
  return CCB_OK;
}
extern "C" uint64_t ccb_wire_bytes(int codec, int dtype, uint64_t count) {
  return codec_slot_bytes(codec, dtype, round_up(count, kWarpElems));
}
extern "C" uint64_t ccb_launch_count(void) { return g_launches.load(); }
extern "C" const char* ccb_last_error(void) { return g_err; }

// ============================================================== launchers ====
namespace ccb {


#define CCB_DISPATCH_TC(dtype, codec, EXPR)                                          \
  [&]() -> const void* {                                                             \
    switch (dtype) {                                                                 \
      case CCB_F32: CCB_DISPATCH_C(float, codec, EXPR)                               \
      case CCB_BF16: CCB_DISPATCH_C(__nv_bfloat16, codec, EXPR)                      \
      case CCB_F16: CCB_DISPATCH_C(__half, codec, EXPR)                              \
    }                                                                                \
    return nullptr;                                                                  \
  }()
#define CCB_DISPATCH_C(T, codec, EXPR)                                               \
  switch (codec) {                                                                   \
    case CCB_CODEC_NONE: { using TT = T; using CC = CodecNone<T>; return EXPR; }      \
    case CCB_CODEC_INT8: { using TT = T; using CC = CodecInt8<128>; return EXPR; }    \
    case CCB_CODEC_INT8_G256: { using TT = T; using CC = CodecInt8<256>; return EXPR; } \
    case CCB_CODEC_FP8: { using TT = T; using CC = CodecFp8; return EXPR; }           \
    case CCB_CODEC_INT4: { using TT = T; using CC = CodecInt4; return EXPR; }         \
    default: return nullptr;                                                         \
  }

static const void* reduce_fn(int dtype, int codec, int shape) {
  if (shape == kOneShot) return CCB_DISPATCH_TC(dtype, codec, (reinterpret_cast<const void*>(&reduce_kernel<TT, CC, kOneShot>)));
  return CCB_DISPATCH_TC(dtype, codec, (reinterpret_cast<const void*>(&reduce_kernel<TT, CC, kTwoShot>)));
}
static const void* exchange_fn(int dtype, int codec) {
  return CCB_DISPATCH_TC(dtype, codec, (reinterpret_cast<const void*>(&exchange_kernel<TT, CC>)));
}
static const void* ring_fn(int dtype, int codec) {
  return CCB_DISPATCH_TC(dtype, codec, (reinterpret_cast<const void*>(&ring_kernel<TT, CC>)));
}
static const void* tree_fn(int dtype, int codec) {
  return CCB_DISPATCH_TC(dtype, codec, (reinterpret_cast<const void*>(&tree_kernel<TT, CC>)));
}

// Picks the tile width (in warps, a power of two up to 16) and the number of CTAs per
// rank for `elems` elements per shard: the widest tile that still gives every
// resident CTA work, so that mid-size messages are not served by a handful of CTAs.
static int ctas_for(ccb_comm* c, const void* fn, size_t elems, int* tile_warps) {
  const int cap = grid_cap(c, fn);
  const size_t units = (elems + kWarpElems - 1) / kWarpElems;
  int tw = kWarps;
  while (tw > 1 && units / (size_t)tw < (size_t)cap) tw >>= 1;
  *tile_warps = tw;
  size_t tiles = (units + tw - 1) / tw;
  if (tiles < 1) tiles = 1;
  return tiles < (size_t)cap ? (int)tiles : cap;
}

// One launch of the reduce family on `count` elements starting at element `base`
// of every buffer (base is a multiple of 512, so vector alignment is preserved).
static int reduce_launch(ccb_comm* c, const void* const* send, void* const* recv, float* const* ef, size_t base,
                         size_t recv_base, size_t count, size_t shard_elems, int dtype, int op, int codec, int mode,
                         int root, int shape, cudaStream_t stream) {
  const void* fn = reduce_fn(dtype, codec, shape);
  if (!fn) {
    set_error("unsupported dtype %d / codec %d", dtype, codec);
    return CCB_ERR_UNSUPPORTED;
  }
  // Large two-shot AllReduce / ReduceScatter calls go to the warp-specialised pipelined
  // kernel: it needs a few chunks (8 units of 512 elements) per CTA and wave to pay.
  int pipe_waves = 0, pipe_ctas = 0;
  if (shape == kTwoShot && mode != CCB_MODE_REDUCE && c->nranks > 1 && c->pipe_mode != 0) {
    const void* pfn = pipe_kernel_fn(dtype, codec);
    const int cap = pfn ? grid_cap(c, pfn, pipe_kernel_threads()) : 1;
    const size_t per = shard_elems < count ? shard_elems : count;
    const size_t chunks = (per + kPipeChunkElems - 1) / kPipeChunkElems;
    const size_t ctas = chunks < (size_t)cap ? chunks : (size_t)cap;
    const size_t per_cta = ctas ? chunks / ctas : 0;
    if (pfn && (per_cta >= (size_t)c->pipe_min_chunks || c->pipe_mode == 2)) {
      // Measured at 256 MiB: two ranks are fastest with 6 waves (272 us against 283 with 8; a
      // wave is then a quarter of the data and each costs two fence-and-flag rounds), four
      // ranks with 8 (386 against 392 with 4).
      int w = c->waves > 0 ? c->waves : (int)(per_cta / 2);
      const int most = c->waves > 0 ? CCB_MAX_SLOTS / 2 : (c->nranks <= 2 ? 6 : CCB_MAX_SLOTS / 2);
      if (w > most) w = most;
      if (w > CCB_MAX_SLOTS / 2) w = CCB_MAX_SLOTS / 2;
      // overlapping calls alternate between the two halves of the flag rows: 4 waves each
      if (c->call_overlap && c->nlocal == 1 && w > CCB_MAX_SLOTS / 4) w = CCB_MAX_SLOTS / 4;
      if (w < 1) w = 1;
      pipe_waves = w;
      pipe_ctas = (int)(ctas ? ctas : 1);
      fn = pfn;
    }
  }
  ReduceArgs a;
  memset(&a, 0, sizeof(a));
  a.c = comm_dev(c, next_epoch(c));
  const size_t es = elem_size(dtype);
  for (int i = 0; i < c->nlocal; ++i) {
    a.send[i] = static_cast<const char*>(send[i]) + base * es;
    a.recv[i] = static_cast<char*>(recv[i]) + recv_base * es;
    a.ef[i] = (ef && ef[i]) ? ef[i] + base : nullptr;
  }
  a.count = count;
  a.shard_elems = shard_elems;
  a.shard_pad = round_up(shard_elems, kWarpElems);
  a.slot_bytes = codec_slot_bytes(codec, dtype, a.shard_pad);
  a.rank0 = c->rank0;
  a.nlocal = c->nlocal;
  a.op = op;
  a.root = root;
  a.mode = mode;
  if (pipe_waves) {
    a.waves = pipe_waves;
    a.tile_warps = kWarps;
    a.link_warps = c->pipe_link_warps;
    a.row_base = (c->call_overlap && c->nlocal == 1 && (a.c.epoch & 1u)) ? CCB_MAX_SLOTS / 2 : 0;
    a.use_mc = (c->mc_arena && c->nlocal == 1 && c->pipe_mc) ? 1 : 0;
    return launch(c, fn, pipe_ctas, &a, stream, pipe_kernel_threads(), true);
  }
  const int ctas = ctas_for(c, fn, shard_elems < count ? shard_elems : count, &a.tile_warps);
  // Each extra wave of the non-specialised kernel costs a pipeline drain (fence + flag
  // round trip) on the data warps that outweighs the overlap it buys, so it runs one wave
  // unless asked otherwise; the pipelined kernel above is the one that overlaps phases.
  int waves = c->waves > 0 ? c->waves : 1;
  if (waves > CCB_MAX_SLOTS / 2) waves = CCB_MAX_SLOTS / 2;
  a.waves = shape == kTwoShot ? waves : 1;
  return launch(c, fn, ctas, &a, stream);
}

int nvls_all_reduce(ccb_comm* c, const void* const* send, void* const* recv, uint64_t count, int dtype, int op,
                    cudaStream_t stream) {
  if (!c->mc_arena || c->nlocal != 1) {
    set_error("this communicator has no NVLS multicast mapping");
    return CCB_ERR_UNSUPPORTED;
  }
  if (op != CCB_OP_SUM) {
    set_error("the NVLS path supports sum only");
    return CCB_ERR_UNSUPPORTED;
  }
  const void* fn = dtype == CCB_F32    ? reinterpret_cast<const void*>(&nvls_allreduce_kernel<float>)
                   : dtype == CCB_BF16 ? reinterpret_cast<const void*>(&nvls_allreduce_kernel<__nv_bfloat16>)
                                       : reinterpret_cast<const void*>(&nvls_allreduce_kernel<__half>);
  const int n = c->nranks;
  const size_t es = elem_size(dtype);
  size_t done = 0;
  while (done < count) {
    size_t left = count - done, slice = left, shard;
    for (;;) {
      shard = round_up((slice + n - 1) / n, kWarpElems);
      if (2 * (size_t)n * round_up(shard * es, 256) <= c->half_bytes) break;
      slice = round_up(slice / 2, (size_t)kWarpElems * n);
      if (slice <= (size_t)kWarpElems * n) break;
    }
    if (slice > left) slice = left;
    shard = round_up((slice + n - 1) / n, kWarpElems);
    ReduceArgs a;
    memset(&a, 0, sizeof(a));
    a.c = comm_dev(c, next_epoch(c));
    a.send[0] = static_cast<const char*>(send[0]) + done * es;
    a.recv[0] = static_cast<char*>(recv[0]) + done * es;
    a.count = slice;
    a.shard_elems = shard;
    a.shard_pad = shard;
    a.slot_bytes = round_up(shard * es, 256);
    if (2 * (size_t)n * a.slot_bytes > c->half_bytes) {
      set_error("arena too small for this call");
      return CCB_ERR_CAPACITY;
    }
    a.rank0 = c->rank0;
    a.nlocal = 1;
    a.op = op;
    size_t tiles = (shard * es / 16 + kThreads * 4 - 1) / (kThreads * 4);
    int cap = grid_cap(c, fn);
    int rc = launch(c, fn, tiles < (size_t)cap ? (int)(tiles ? tiles : 1) : cap, &a, stream);
    if (rc) return rc;
    done += slice;
  }
  return CCB_OK;
}

}  // namespace ccb

extern "C" int ccb_all_reduce(ccb_comm* c, const void* const* send, void* const* recv, uint64_t count, int dtype,
                              int op, int codec, int algo, float* const* ef, ccb_stream_t stream_) {
  int rc = check_alive(c);
  if (rc) return rc;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  if (count == 0) return CCB_OK;
  if (codec != CCB_CODEC_NONE && op != CCB_OP_SUM) {
    set_error("lossy codecs support sum only");
    return CCB_ERR_UNSUPPORTED;
  }
  const int n = c->nranks;
  const size_t es = elem_size(dtype);
  if (algo == CCB_ALGO_AUTO) {
    // One-shot has one exchange instead of two (about 10 us less latency) but every rank
    // sends its whole message to every peer: (n-1) * S wire bytes against 2(n-1)/n * S.
    // It wins while the extra (n-1)(1-2/n) * S bytes cost less than that latency at the
    // ~600 GB/s an SM-driven NVLink stream sustains, i.e. below about
    // 6 MB / ((n-1)(1-2/n)) of wire bytes; with two ranks both shapes move the same
    // bytes and one-shot stays ahead until the pipelined two-shot kernel overtakes it
    // (measured: int8 95 against 110 us at 35 MB of wire, 351 against 265 us at 138 MB;
    // uncompressed 62 against 76 us at 17 MB, 146 against 140 us at 67 MB): 48 MiB.
    const size_t wire = codec_slot_bytes(codec, dtype, round_up(count, kWarpElems));
    size_t limit = n <= 2 ? ((size_t)48 << 20) : (size_t)(6.0e6 / ((n - 1) * (1.0 - 2.0 / n)));
    limit = (size_t)env_u64("CCB_ONESHOT_MAX_BYTES", limit);
    const bool fits = (size_t)n * wire <= c->half_bytes;
    algo = (n > 1 && fits && wire <= limit) ? CCB_ALGO_ONESHOT : CCB_ALGO_TWOSHOT;
  }
  if (algo == CCB_ALGO_NVLS) return nvls_all_reduce(c, send, recv, count, dtype, op, stream);
  if (algo == CCB_ALGO_RING || algo == CCB_ALGO_TREE) {
    const void* fn = algo == CCB_ALGO_RING ? ring_fn(dtype, codec) : tree_fn(dtype, codec);
    if (!fn) {
      set_error("unsupported dtype %d / codec %d", dtype, codec);
      return CCB_ERR_UNSUPPORTED;
    }
    // Ring: 2(n-1) slots of one shard. Tree: ceil(log2 n) + 1 slots of the whole message.
    int levels = 0;
    while ((1 << levels) < n) ++levels;
    const size_t nslots = algo == CCB_ALGO_RING ? (size_t)(2 * (n - 1)) : (size_t)(levels + 1);
    if (nslots > CCB_MAX_SLOTS) {
      set_error("too many steps for the flag table");
      return CCB_ERR_UNSUPPORTED;
    }
    size_t done = 0;
    while (done < count) {
      // Largest slice (multiple of 512 * n) whose slots fit in half an arena.
      size_t left = count - done;
      size_t slice = left;
      for (;;) {
        size_t unit = algo == CCB_ALGO_RING ? round_up((slice + n - 1) / n, kWarpElems) : round_up(slice, kWarpElems);
        size_t need = (nslots ? nslots : 1) * codec_slot_bytes(codec, dtype, unit);
        if (need <= c->half_bytes) break;
        slice = round_up(slice / 2, (size_t)kWarpElems * n);
        if (slice <= (size_t)kWarpElems * n) break;
      }
      if (slice > left) slice = left;
      ReduceArgs a;
      memset(&a, 0, sizeof(a));
      a.c = comm_dev(c, next_epoch(c));
      for (int i = 0; i < c->nlocal; ++i) {
        a.send[i] = static_cast<const char*>(send[i]) + done * es;
        a.recv[i] = static_cast<char*>(recv[i]) + done * es;
        a.ef[i] = (ef && ef[i]) ? ef[i] + done : nullptr;
      }
      a.count = slice;
      a.shard_elems = algo == CCB_ALGO_RING ? round_up((slice + n - 1) / n, kWarpElems) : round_up(slice, kWarpElems);
      a.shard_pad = a.shard_elems;
      a.slot_bytes = codec_slot_bytes(codec, dtype, a.shard_pad);
      if ((nslots ? nslots : 1) * a.slot_bytes > c->half_bytes) {
        set_error("arena too small for this call");
        return CCB_ERR_CAPACITY;
      }
      a.rank0 = c->rank0;
      a.nlocal = c->nlocal;
      a.op = op;
      a.mode = CCB_MODE_ALLREDUCE;
      const int ctas = ctas_for(c, fn, a.shard_elems < slice ? a.shard_elems : slice, &a.tile_warps);
      rc = launch(c, fn, ctas, &a, stream);
      if (rc) return rc;
      done += slice;
    }
    return CCB_OK;
  }
  const int shape = algo == CCB_ALGO_ONESHOT ? kOneShot : kTwoShot;
  size_t done = 0;
  while (done < count) {
    size_t left = count - done, slice = left, shard;
    for (;;) {
      shard = shape == kOneShot ? round_up(slice, kWarpElems) : round_up((slice + n - 1) / n, kWarpElems);
      size_t need = (shape == kOneShot ? 1 : 2) * (size_t)n * codec_slot_bytes(codec, dtype, shard);
      if (need <= c->half_bytes) break;
      slice = round_up(slice / 2, (size_t)kWarpElems * n);
      if (slice <= (size_t)kWarpElems * n) break;
    }
    if (slice > left) slice = left;
    shard = shape == kOneShot ? round_up(slice, kWarpElems) : round_up((slice + n - 1) / n, kWarpElems);
    if ((shape == kOneShot ? 1 : 2) * (size_t)n * codec_slot_bytes(codec, dtype, shard) > c->half_bytes) {
      set_error("arena too small for this call");
      return CCB_ERR_CAPACITY;
    }
    rc = reduce_launch(c, send, recv, ef, done, done, slice, shard, dtype, op, codec, CCB_MODE_ALLREDUCE, 0, shape, stream);
    if (rc) return rc;
    done += slice;
  }
  return CCB_OK;
}

extern "C" int ccb_reduce_scatter(ccb_comm* c, const void* const* send, void* const* recv, uint64_t recvcount,
                                  int dtype, int op, int codec, float* const* ef, ccb_stream_t stream_) {
  int rc = check_alive(c);
  if (rc) return rc;
  if (recvcount == 0) return CCB_OK;
  if (codec != CCB_CODEC_NONE && op != CCB_OP_SUM) {
    set_error("lossy codecs support sum only");
    return CCB_ERR_UNSUPPORTED;
  }
  const int n = c->nranks;
  const size_t pad = round_up(recvcount, kWarpElems);
  if ((size_t)n * codec_slot_bytes(codec, dtype, pad) > c->half_bytes) {
    set_error("arena too small: reduce_scatter of %llu elements per rank needs %llu bytes of staging",
              (unsigned long long)recvcount, (unsigned long long)((size_t)n * codec_slot_bytes(codec, dtype, pad)));
    return CCB_ERR_CAPACITY;
  }
  return reduce_launch(c, send, recv, ef, 0, 0, (size_t)recvcount * n, recvcount, dtype, op, codec,
                       CCB_MODE_REDUCESCATTER, 0, kTwoShot, static_cast<cudaStream_t>(stream_));
}

extern "C" int ccb_reduce(ccb_comm* c, const void* const* send, void* const* recv, uint64_t count, int dtype, int op,
                          int root, int codec, ccb_stream_t stream_) {
  int rc = check_alive(c);
  if (rc) return rc;
  if (count == 0) return CCB_OK;
  if (root < 0 || root >= c->nranks) {
    set_error("bad root %d", root);
    return CCB_ERR_ARG;
  }
  if (codec != CCB_CODEC_NONE && op != CCB_OP_SUM) {
    set_error("lossy codecs support sum only");
    return CCB_ERR_UNSUPPORTED;
  }
  const size_t pad = round_up(count, kWarpElems);
  if ((size_t)c->nranks * codec_slot_bytes(codec, dtype, pad) > c->half_bytes) {
    set_error("arena too small for reduce of %llu elements", (unsigned long long)count);
    return CCB_ERR_CAPACITY;
  }
  return reduce_launch(c, send, recv, nullptr, 0, 0, count, pad, dtype, op, codec, CCB_MODE_REDUCE, root, kTwoShot,
                       static_cast<cudaStream_t>(stream_));
}

extern "C" int ccb_exchange(ccb_comm* c, const void* const* send, void* const* recv, const uint64_t* cnt,
                            const uint64_t* send_off, const uint64_t* recv_off, int dtype, int codec,
                            ccb_stream_t stream_) {
  int rc = check_alive(c);
  if (rc) return rc;
  const int n = c->nranks;
  const void* fn = exchange_fn(dtype, codec);
  if (!fn) {
    set_error("unsupported dtype %d / codec %d", dtype, codec);
    return CCB_ERR_UNSUPPORTED;
  }
  ExchangeArgs a;
  memset(&a, 0, sizeof(a));
  size_t maxcnt = 0;
  bool full = true;
  for (int s = 0; s < n; ++s)
    for (int d = 0; d < n; ++d) {
      a.cnt[s][d] = cnt[s * n + d];
      a.send_off[s][d] = send_off[s * n + d];
      a.recv_off[d][s] = recv_off[d * n + s];
      if (a.cnt[s][d] > maxcnt) maxcnt = a.cnt[s][d];
      if (s != d && a.cnt[s][d] == 0) full = false;
    }
  if (maxcnt == 0) return CCB_OK;
  a.slot_pad = round_up(maxcnt, kWarpElems);
  a.slot_bytes = codec_slot_bytes(codec, dtype, a.slot_pad);
  if ((size_t)n * a.slot_bytes > c->half_bytes) {
    set_error("arena too small: exchange blocks of %llu elements need %llu bytes of staging", (unsigned long long)maxcnt,
              (unsigned long long)((size_t)n * a.slot_bytes));
    return CCB_ERR_CAPACITY;
  }
  a.c = comm_dev(c, next_epoch(c));
  for (int i = 0; i < c->nlocal; ++i) {
    a.send[i] = send[i];
    a.recv[i] = recv[i];
  }
  a.rank0 = c->rank0;
  a.nlocal = c->nlocal;
  a.ack = full ? 0 : 1;
  const int ctas = ctas_for(c, fn, maxcnt, &a.tile_warps);
  return launch(c, fn, ctas, &a, static_cast<cudaStream_t>(stream_));
}

namespace {
struct Mats {
  uint64_t cnt[CCB_MAX_RANKS * CCB_MAX_RANKS] = {}, so[CCB_MAX_RANKS * CCB_MAX_RANKS] = {}, ro[CCB_MAX_RANKS * CCB_MAX_RANKS] = {};
};
}  // namespace

extern "C" int ccb_all_gather(ccb_comm* c, const void* const* send, void* const* recv, uint64_t sendcount, int dtype,
                              int codec, ccb_stream_t stream) {
  if (!c) return CCB_ERR_ARG;
  const int n = c->nranks;
  Mats m;
  for (int s = 0; s < n; ++s)
    for (int d = 0; d < n; ++d) {
      m.cnt[s * n + d] = sendcount;
      m.so[s * n + d] = 0;
      m.ro[d * n + s] = (uint64_t)s * sendcount;
    }
  return ccb_exchange(c, send, recv, m.cnt, m.so, m.ro, dtype, codec, stream);
}

extern "C" int ccb_broadcast(ccb_comm* c, const void* const* send, void* const* recv, uint64_t count, int dtype,
                             int root, int codec, ccb_stream_t stream) {
  if (!c || root < 0 || root >= c->nranks) return CCB_ERR_ARG;
  const int n = c->nranks;
  Mats m;
  for (int d = 0; d < n; ++d) m.cnt[root * n + d] = count;
  return ccb_exchange(c, send, recv, m.cnt, m.so, m.ro, dtype, codec, stream);
}

extern "C" int ccb_all_to_all(ccb_comm* c, const void* const* send, void* const* recv, uint64_t count, int dtype,
                              int codec, ccb_stream_t stream) {
  if (!c) return CCB_ERR_ARG;
  const int n = c->nranks;
  Mats m;
  for (int s = 0; s < n; ++s)
    for (int d = 0; d < n; ++d) {
      m.cnt[s * n + d] = count;
      m.so[s * n + d] = (uint64_t)d * count;
      m.ro[d * n + s] = (uint64_t)s * count;
    }
  return ccb_exchange(c, send, recv, m.cnt, m.so, m.ro, dtype, codec, stream);
}

extern "C" int ccb_scatter(ccb_comm* c, const void* const* send, void* const* recv, uint64_t recvcount, int dtype,
                           int root, int codec, ccb_stream_t stream) {
  if (!c || root < 0 || root >= c->nranks) return CCB_ERR_ARG;
  const int n = c->nranks;
  Mats m;
  for (int d = 0; d < n; ++d) {
    m.cnt[root * n + d] = recvcount;
    m.so[root * n + d] = (uint64_t)d * recvcount;
  }
  return ccb_exchange(c, send, recv, m.cnt, m.so, m.ro, dtype, codec, stream);
}

extern "C" int ccb_gather(ccb_comm* c, const void* const* send, void* const* recv, uint64_t sendcount, int dtype,
                          int root, int codec, ccb_stream_t stream) {
  if (!c || root < 0 || root >= c->nranks) return CCB_ERR_ARG;
  const int n = c->nranks;
  Mats m;
  for (int s = 0; s < n; ++s) {
    m.cnt[s * n + root] = sendcount;
    m.ro[root * n + s] = (uint64_t)s * sendcount;
  }
  return ccb_exchange(c, send, recv, m.cnt, m.so, m.ro, dtype, codec, stream);
}

// Test hook: launch a two-shot fp32 AllReduce that plays only the first
// `ranks_played` ranks of a local communicator. The flags of the absent ranks are
// never written, so the waits of the played ranks run out their limit and report
// through the status words. Used to test the time-out path without any fault.
extern "C" int ccb_test_partial_all_reduce(ccb_comm* c, const void* send, void* recv, uint64_t count, int ranks_played,
                                           ccb_stream_t stream) {
  int rc = check_alive(c);
  if (rc) return rc;
  if (c->nlocal != c->nranks || ranks_played < 1 || ranks_played >= c->nranks) {
    set_error("needs a local communicator and 1 <= ranks_played < nranks");
    return CCB_ERR_ARG;
  }
  if (!send || !recv || count == 0) {
    set_error("send, recv and a positive count are required");
    return CCB_ERR_ARG;
  }
  if (2 * (size_t)c->nranks * codec_slot_bytes(CCB_CODEC_NONE, CCB_F32, round_up((count + c->nranks - 1) / c->nranks, kWarpElems)) > c->half_bytes) {
    set_error("arena too small for this call");
    return CCB_ERR_CAPACITY;
  }
  const void* fn = reinterpret_cast<const void*>(&reduce_kernel<float, CodecNone<float>, kTwoShot>);
  ReduceArgs a;
  memset(&a, 0, sizeof(a));
  a.c = comm_dev(c, next_epoch(c));
  for (int i = 0; i < ranks_played; ++i) {
    a.send[i] = send;
    a.recv[i] = recv;
  }
  a.count = count;
  a.shard_elems = round_up((count + c->nranks - 1) / c->nranks, kWarpElems);
  a.shard_pad = a.shard_elems;
  a.slot_bytes = codec_slot_bytes(CCB_CODEC_NONE, CCB_F32, a.shard_pad);
  a.rank0 = 0;
  a.nlocal = ranks_played;
  a.mode = CCB_MODE_ALLREDUCE;
  a.waves = 1;
  a.tile_warps = kWarps;
  dim3 grid(1, (unsigned)ranks_played, 1), block(kThreads, 1, 1);
  void* params[] = {&a};
  cudaError_t e = cudaLaunchCooperativeKernel(fn, grid, block, params, 0, static_cast<cudaStream_t>(stream));
  if (e != cudaSuccess) {
    set_error("kernel launch failed: %s", cudaGetErrorString(e));
    return CCB_ERR_CUDA;
  }
  count_launch();
  return CCB_OK;
}

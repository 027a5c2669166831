// Native symmetric arena: one physical allocation per rank made with the virtual-memory-management
// driver API, exported as a POSIX file descriptor, imported and mapped by every peer of the node.
//
//   rank r:  cuMemCreate(size, shareable as fd)  ->  map at a reserved address, read/write for r
//            export fd  --(Unix socket, csrc/runtime/fd_exchange.cpp)-->  every peer
//   peer p:  cuMemImportFromShareableHandle(fd)  ->  map at its own reserved address,
//            read/write for device p (the access travels over NVLink)
//
// The kernels in this directory take the table of the `world` base addresses (PeerTable) plus byte
// offsets that are identical on every rank.  No multicast object is created here: the arena offers
// plain peer loads and stores only.
//
// This is the counterpart of the reference's buffer pool + device context singletons
// (rumus/src/backend/gpu/pool.rs:23-101, rumus/src/backend/gpu/context.rs:750-757,916-995), which
// have no peer mappings at all ("WebGPU has no peer-to-peer DMA", rumus/src/tensor/core.rs:1175).
//
// The driver entry points are looked up through the runtime, so the library does not link libcuda.
#include <cuda.h>
#include <cuda_runtime.h>

#include <cstdio>
#include <cstring>
#include <unistd.h>

namespace {

constexpr int kMaxRanks = 8;

struct Driver {
  CUresult (*MemGetAllocationGranularity)(size_t*, const CUmemAllocationProp*, CUmemAllocationGranularity_flags);
  CUresult (*MemCreate)(CUmemGenericAllocationHandle*, size_t, const CUmemAllocationProp*, unsigned long long);
  CUresult (*MemAddressReserve)(CUdeviceptr*, size_t, size_t, CUdeviceptr, unsigned long long);
  CUresult (*MemMap)(CUdeviceptr, size_t, size_t, CUmemGenericAllocationHandle, unsigned long long);
  CUresult (*MemSetAccess)(CUdeviceptr, size_t, const CUmemAccessDesc*, size_t);
  CUresult (*MemExportToShareableHandle)(void*, CUmemGenericAllocationHandle, CUmemAllocationHandleType, unsigned long long);
  CUresult (*MemImportFromShareableHandle)(CUmemGenericAllocationHandle*, void*, CUmemAllocationHandleType);
  CUresult (*MemUnmap)(CUdeviceptr, size_t);
  CUresult (*MemRelease)(CUmemGenericAllocationHandle);
  CUresult (*MemAddressFree)(CUdeviceptr, size_t);
  bool ok = false;
};

template <typename F>
bool load(const char* name, F* fn) {
  void* p = nullptr;
  cudaDriverEntryPointQueryResult q;
  if (cudaGetDriverEntryPoint(name, &p, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess || !p)
    return false;
  *fn = reinterpret_cast<F>(p);
  return true;
}

Driver& driver() {
  static Driver d = [] {
    Driver x{};
    x.ok = load("cuMemGetAllocationGranularity", &x.MemGetAllocationGranularity) &&
           load("cuMemCreate", &x.MemCreate) && load("cuMemAddressReserve", &x.MemAddressReserve) &&
           load("cuMemMap", &x.MemMap) && load("cuMemSetAccess", &x.MemSetAccess) &&
           load("cuMemExportToShareableHandle", &x.MemExportToShareableHandle) &&
           load("cuMemImportFromShareableHandle", &x.MemImportFromShareableHandle) &&
           load("cuMemUnmap", &x.MemUnmap) && load("cuMemRelease", &x.MemRelease) &&
           load("cuMemAddressFree", &x.MemAddressFree);
    return x;
  }();
  return d;
}

struct Arena {
  int device = 0, rank = 0, world = 1;
  size_t bytes = 0;                                  // rounded up to the allocation granularity
  CUmemGenericAllocationHandle handle[kMaxRanks] = {};
  CUdeviceptr base[kMaxRanks] = {};
  bool mapped[kMaxRanks] = {};
  bool have_handle[kMaxRanks] = {};
};

CUmemAllocationProp props(int device) {
  CUmemAllocationProp p{};
  p.type = CU_MEM_ALLOCATION_TYPE_PINNED;
  p.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  p.location.id = device;
  p.requestedHandleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
  return p;
}

// Reserve an address range, map `h` there and give `device` read/write access.
int map_handle(Arena* a, int slot, CUmemGenericAllocationHandle h) {
  Driver& d = driver();
  CUdeviceptr va = 0;
  if (d.MemAddressReserve(&va, a->bytes, 0, 0, 0) != CUDA_SUCCESS) return 11;
  if (d.MemMap(va, a->bytes, 0, h, 0) != CUDA_SUCCESS) {
    d.MemAddressFree(va, a->bytes);
    return 12;
  }
  CUmemAccessDesc acc{};
  acc.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  acc.location.id = a->device;
  acc.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
  if (d.MemSetAccess(va, a->bytes, &acc, 1) != CUDA_SUCCESS) {
    d.MemUnmap(va, a->bytes);
    d.MemAddressFree(va, a->bytes);
    return 13;
  }
  a->base[slot] = va;
  a->mapped[slot] = true;
  return 0;
}

}  // namespace

extern "C" {

// Creates this rank's allocation (at least `bytes`, rounded up to the granularity) on `device` and
// maps it locally.  Error codes: 1 bad arguments, 2 driver entry points unavailable, 3 granularity
// query failed, 4 allocation failed, 11-13 reserve / map / set-access failed.
int rb_arena_create(long long bytes, int device, int rank, int world, void** out) {
  if (bytes <= 0 || world < 1 || world > kMaxRanks || rank < 0 || rank >= world || !out) return 1;
  Driver& d = driver();
  if (!d.ok) return 2;
  cudaSetDevice(device);
  cudaFree(nullptr);   // make sure the primary context exists
  CUmemAllocationProp p = props(device);
  size_t gran = 0;
  if (d.MemGetAllocationGranularity(&gran, &p, CU_MEM_ALLOC_GRANULARITY_RECOMMENDED) != CUDA_SUCCESS || gran == 0)
    return 3;
  Arena* a = new Arena;
  a->device = device; a->rank = rank; a->world = world;
  a->bytes = ((size_t)bytes + gran - 1) / gran * gran;
  if (d.MemCreate(&a->handle[rank], a->bytes, &p, 0) != CUDA_SUCCESS) { delete a; return 4; }
  a->have_handle[rank] = true;
  const int rc = map_handle(a, rank, a->handle[rank]);
  if (rc) {
    d.MemRelease(a->handle[rank]);
    delete a;
    return rc;
  }
  *out = a;
  return 0;
}

long long rb_arena_bytes(void* h) { return (long long)static_cast<Arena*>(h)->bytes; }

// A new file descriptor for this rank's allocation (the caller closes it after the exchange).
int rb_arena_export_fd(void* h, int* fd) {
  Arena* a = static_cast<Arena*>(h);
  int out = -1;
  if (driver().MemExportToShareableHandle(&out, a->handle[a->rank], CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0) != CUDA_SUCCESS)
    return 21;
  *fd = out;
  return 0;
}

// Maps the allocation behind `fd` (exported by rank `peer`) into this process.  The descriptor is
// not closed here.
int rb_arena_import_peer(void* h, int peer, int fd) {
  Arena* a = static_cast<Arena*>(h);
  if (peer < 0 || peer >= a->world || peer == a->rank || a->mapped[peer]) return 1;
  Driver& d = driver();
  if (d.MemImportFromShareableHandle(&a->handle[peer], (void*)(uintptr_t)fd, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR) != CUDA_SUCCESS)
    return 22;
  a->have_handle[peer] = true;
  return map_handle(a, peer, a->handle[peer]);
}

// Base address of rank `r`'s arena in this process (0 if not mapped).
unsigned long long rb_arena_base(void* h, int r) {
  Arena* a = static_cast<Arena*>(h);
  return (r >= 0 && r < a->world && a->mapped[r]) ? (unsigned long long)a->base[r] : 0ull;
}

// Unmaps everything and drops the handles.  The caller makes sure (stream synchronisation plus a
// barrier across the ranks) that no kernel of any rank still touches the memory.
int rb_arena_destroy(void* h) {
  Arena* a = static_cast<Arena*>(h);
  if (!a) return 0;
  Driver& d = driver();
  for (int r = 0; r < a->world; ++r) {
    if (a->mapped[r]) {
      d.MemUnmap(a->base[r], a->bytes);
      d.MemAddressFree(a->base[r], a->bytes);
    }
    if (a->have_handle[r]) d.MemRelease(a->handle[r]);
  }
  delete a;
  return 0;
}
}

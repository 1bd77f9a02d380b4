// Symmetric memory over the CUDA virtual-memory API: each rank creates one physical chunk,
// exports it (POSIX fd or 64-byte fabric handle), imports every peer's chunk and maps all of
// them read/write into ONE contiguous virtual range, chunk r at base + r * chunk_bytes.
// Optionally the chunks are also bound to an NVSwitch multicast object and mapped a second
// time, so that a `multimem` store reaches every rank.
//
// Host-only code; C++ counterpart of the reference's csrc/nvl_shared_buffer.cuh
// (capability probe :41-66, granularity :68-118, export/import :158-217, local allocation
// :227-273, all-rank mapping :284-356, multicast :383-544). Differences: errors are returned
// (never exit()), resources are owned by explicit handles that Python releases in a defined
// order, and one heap chunk carries all of a Buffer's sub-buffers (one exchange per Buffer).
#include "driver_api.h"
#include "launch.h"
#include <string.h>
#include <unistd.h>
#include <vector>

namespace mep {

enum HandleKind { kHandleFd = 0, kHandleFabric = 1 };

static CUmemAllocationHandleType cu_type(int kind) {
  return kind == kHandleFabric ? CU_MEM_HANDLE_TYPE_FABRIC : CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
}

static CUmemAllocationProp alloc_prop(int dev, int kind) {
  CUmemAllocationProp p = {};
  p.type = CU_MEM_ALLOCATION_TYPE_PINNED;
  p.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  p.location.id = dev;
  p.requestedHandleTypes = cu_type(kind);
  return p;
}

struct LocalChunk {
  int dev; size_t bytes; int kind;
  CUmemGenericAllocationHandle handle;   // kept for multicast binding
  bool handle_live;
};

struct Mapping {
  int dev; int world; size_t chunk_bytes;
  CUdeviceptr base;
  std::vector<bool> mapped;
};

// [fresh local memory | an existing chunk] in one virtual range, see mep_alias_map
struct AliasMap {
  int dev; CUdeviceptr va; size_t local_bytes, tail_bytes;
  CUmemGenericAllocationHandle local; bool local_live, local_mapped, tail_mapped;
};

struct Multicast {
  int dev; size_t bytes;
  CUmemGenericAllocationHandle mc; bool mc_live;
  CUdeviceptr va; bool mapped; bool bound;
};

}  // namespace mep

using namespace mep;

extern "C" {

// 1 if this device can export fabric handles (attribute AND a trial allocation succeed).
int mep_fabric_supported(int dev, int* out) {
  *out = 0;
  const DriverApi* d = driver(); if (!d) return -1;
  CUdevice cd; MEP_CU_CHECK(d->DeviceGet(&cd, dev));
  int attr = 0;
  if (d->DeviceGetAttribute(&attr, CU_DEVICE_ATTRIBUTE_HANDLE_TYPE_FABRIC_SUPPORTED, cd) != CUDA_SUCCESS || !attr) return 0;
  CUmemAllocationProp p = alloc_prop(dev, kHandleFabric);
  size_t gran = 0;
  if (d->MemGetAllocationGranularity(&gran, &p, CU_MEM_ALLOC_GRANULARITY_RECOMMENDED) != CUDA_SUCCESS) return 0;
  CUmemGenericAllocationHandle h;
  if (d->MemCreate(&h, gran, &p, 0) != CUDA_SUCCESS) return 0;
  d->MemRelease(h);
  *out = 1;
  return 0;
}

int mep_multicast_supported(int dev, int* out) {
  *out = 0;
  const DriverApi* d = driver(); if (!d) return -1;
  CUdevice cd; MEP_CU_CHECK(d->DeviceGet(&cd, dev));
  int attr = 0;
  if (d->DeviceGetAttribute(&attr, CU_DEVICE_ATTRIBUTE_MULTICAST_SUPPORTED, cd) == CUDA_SUCCESS) *out = attr;
  return 0;
}

// Recommended mapping granularity for one handle kind.
int mep_vmm_granularity(int dev, int kind, size_t* out) {
  const DriverApi* d = driver(); if (!d) return -1;
  CUmemAllocationProp p = alloc_prop(dev, kind);
  MEP_CU_CHECK(d->MemGetAllocationGranularity(out, &p, CU_MEM_ALLOC_GRANULARITY_RECOMMENDED));
  return 0;
}

int mep_multicast_granularity(int dev, int world, int kind, size_t bytes, size_t* out) {
  const DriverApi* d = driver(); if (!d) return -1;
  CUmulticastObjectProp mp = {};
  mp.numDevices = world; mp.size = bytes; mp.handleTypes = cu_type(kind);
  MEP_CU_CHECK(d->MulticastGetGranularity(out, &mp, CU_MULTICAST_GRANULARITY_RECOMMENDED));
  return 0;
}

// Create this rank's physical chunk. `bytes` must be a multiple of the granularity.
// `shareable` receives either an int fd (first 4 bytes) or the 64-byte fabric handle.
int mep_chunk_create(int dev, size_t bytes, int kind, void** chunk_out, unsigned char shareable[64]) {
  const DriverApi* d = driver(); if (!d) return -1;
  CUmemAllocationProp p = alloc_prop(dev, kind);
  size_t gran = 0;
  MEP_CU_CHECK(d->MemGetAllocationGranularity(&gran, &p, CU_MEM_ALLOC_GRANULARITY_RECOMMENDED));
  MEP_REQUIRE(bytes > 0 && bytes % gran == 0, "chunk size %zu is not a multiple of the granularity %zu", bytes, gran);
  LocalChunk* c = new LocalChunk{dev, bytes, kind, 0, false};
  CUresult r = d->MemCreate(&c->handle, bytes, &p, 0);
  if (r != CUDA_SUCCESS) {
    delete c;
    size_t fr = 0, tot = 0; cudaMemGetInfo(&fr, &tot);
    const char* es = nullptr; d->GetErrorString(r, &es);
    return set_error("cuMemCreate(%zu bytes) failed: %s (device %d: %zu MiB free of %zu MiB)", bytes, es ? es : "?", dev,
                     fr >> 20, tot >> 20);
  }
  c->handle_live = true;
  memset(shareable, 0, 64);
  if (kind == kHandleFabric) {
    CUmemFabricHandle fh;
    r = d->MemExportToShareableHandle(&fh, c->handle, CU_MEM_HANDLE_TYPE_FABRIC, 0);
    if (r == CUDA_SUCCESS) memcpy(shareable, &fh, sizeof fh);
  } else {
    int fd = -1;
    r = d->MemExportToShareableHandle(&fd, c->handle, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0);
    if (r == CUDA_SUCCESS) memcpy(shareable, &fd, sizeof fd);
  }
  if (r != CUDA_SUCCESS) { d->MemRelease(c->handle); delete c; MEP_CU_CHECK(r); }
  *chunk_out = c;
  return 0;
}

// Drop the owned physical handle (mappings keep the memory alive). Idempotent.
int mep_chunk_release(void* chunk) {
  LocalChunk* c = static_cast<LocalChunk*>(chunk);
  if (!c) return 0;
  const DriverApi* d = driver();
  if (d && c->handle_live) { d->MemRelease(c->handle); c->handle_live = false; }
  delete c;
  return 0;
}

// Map all ranks' chunks contiguously. `shareables` is world x 64 bytes (fd ints or fabric
// handles; entry `my_rank` is not imported: the local chunk's own handle is used). With fd
// handles this call CONSUMES every descriptor of the table, on success and on failure alike:
// peers' descriptors are closed once imported, entry `my_rank` (the copy of the caller's own
// descriptor that came back through the exchange; negative = none) is closed unused, and after a
// failed import the descriptors of the ranks not reached yet are closed too. On failure
// everything mapped so far is undone.
int mep_map_all(int dev, int world, int my_rank, void* local_chunk, const unsigned char* shareables,
                void** mapping_out, unsigned long long* base_out) {
  const DriverApi* d = driver(); if (!d) return -1;
  LocalChunk* lc = static_cast<LocalChunk*>(local_chunk);
  MEP_REQUIRE(lc && lc->handle_live, "map_all: local chunk already released");
  MEP_REQUIRE(world >= 1 && my_rank >= 0 && my_rank < world, "map_all: bad rank %d of %d", my_rank, world);
  const size_t cb = lc->bytes;
  CUmemAllocationProp p = alloc_prop(dev, lc->kind);
  size_t gran = 0;
  MEP_CU_CHECK(d->MemGetAllocationGranularity(&gran, &p, CU_MEM_ALLOC_GRANULARITY_RECOMMENDED));
  Mapping* m = new Mapping{dev, world, cb, 0, std::vector<bool>(world, false)};
  CUresult r = d->MemAddressReserve(&m->base, cb * world, gran, 0, 0);
  if (r != CUDA_SUCCESS) { delete m; MEP_CU_CHECK(r); }
  CUmemAccessDesc acc = {};
  acc.location.type = CU_MEM_LOCATION_TYPE_DEVICE; acc.location.id = dev; acc.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
  const char* what = "";
  int consumed = 0;      // fd handles: table entries [0, consumed) have been closed
  for (int i = 0; i < world && r == CUDA_SUCCESS; ++i) {
    CUmemGenericAllocationHandle h; bool imported = false;
    if (i == my_rank) {
      h = lc->handle;
      if (lc->kind != kHandleFabric) { int fd; memcpy(&fd, shareables + 64 * i, sizeof fd); if (fd >= 0) close(fd); }
      consumed = i + 1;
    }
    else if (lc->kind == kHandleFabric) {
      CUmemFabricHandle fh; memcpy(&fh, shareables + 64 * i, sizeof fh);
      r = d->MemImportFromShareableHandle(&h, &fh, CU_MEM_HANDLE_TYPE_FABRIC); what = "import(fabric)"; imported = r == CUDA_SUCCESS;
    } else {
      int fd; memcpy(&fd, shareables + 64 * i, sizeof fd);
      r = d->MemImportFromShareableHandle(&h, (void*)(uintptr_t)fd, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR);
      what = "import(fd)"; imported = r == CUDA_SUCCESS;
      close(fd);
      consumed = i + 1;
    }
    if (r != CUDA_SUCCESS) break;
    r = d->MemMap(m->base + (size_t)i * cb, cb, 0, h, 0); what = "map";
    if (r == CUDA_SUCCESS) m->mapped[i] = true;
    if (imported) d->MemRelease(h);
  }
  if (r == CUDA_SUCCESS) { r = d->MemSetAccess(m->base, cb * world, &acc, 1); what = "set_access"; }
  if (r != CUDA_SUCCESS) {
    if (lc->kind != kHandleFabric)
      for (int i = consumed; i < world; ++i) { int fd; memcpy(&fd, shareables + 64 * i, sizeof fd); if (fd >= 0) close(fd); }
    for (int i = 0; i < world; ++i) if (m->mapped[i]) d->MemUnmap(m->base + (size_t)i * cb, cb);
    d->MemAddressFree(m->base, cb * world);
    delete m;
    const char* s = nullptr; d->GetErrorString(r, &s);
    return set_error("map_all: %s failed: %s", what, s ? s : "?");
  }
  *mapping_out = m; *base_out = (unsigned long long)m->base;
  return 0;
}

// Map ONE chunk that another process owns (single-owner tensors): import its shareable handle
// (fd: consumed; fabric: 64 bytes) and map it read-write at a fresh address. The result is released
// with mep_unmap_all like any other mapping.
int mep_map_remote_one(int dev, int kind, size_t bytes, const unsigned char* shareable,
                       void** mapping_out, unsigned long long* base_out) {
  const DriverApi* d = driver(); if (!d) return -1;
  MEP_REQUIRE(bytes > 0 && shareable != nullptr, "map_remote_one: empty chunk");
  CUmemAllocationProp p = alloc_prop(dev, kind);
  size_t gran = 0;
  MEP_CU_CHECK(d->MemGetAllocationGranularity(&gran, &p, CU_MEM_ALLOC_GRANULARITY_RECOMMENDED));
  MEP_REQUIRE(bytes % gran == 0, "map_remote_one: %zu bytes is not a multiple of the granularity %zu", bytes, gran);
  CUmemGenericAllocationHandle h;
  if (kind == kHandleFabric) {
    CUmemFabricHandle fh; memcpy(&fh, shareable, sizeof fh);
    MEP_CU_CHECK(d->MemImportFromShareableHandle(&h, &fh, CU_MEM_HANDLE_TYPE_FABRIC));
  } else {
    int fd; memcpy(&fd, shareable, sizeof fd);
    const CUresult ri = d->MemImportFromShareableHandle(&h, (void*)(uintptr_t)fd, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR);
    close(fd);
    MEP_CU_CHECK(ri);
  }
  Mapping* m = new Mapping{dev, 1, bytes, 0, std::vector<bool>(1, false)};
  const char* what = "reserve";
  CUresult r = d->MemAddressReserve(&m->base, bytes, gran, 0, 0);
  if (r == CUDA_SUCCESS) {
    r = d->MemMap(m->base, bytes, 0, h, 0); what = "map";
    if (r == CUDA_SUCCESS) {
      m->mapped[0] = true;
      CUmemAccessDesc acc = {};
      acc.location.type = CU_MEM_LOCATION_TYPE_DEVICE; acc.location.id = dev; acc.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
      r = d->MemSetAccess(m->base, bytes, &acc, 1); what = "set_access";
    }
  }
  d->MemRelease(h);          // the mapping keeps the allocation alive
  if (r != CUDA_SUCCESS) {
    if (m->mapped[0]) d->MemUnmap(m->base, bytes);
    if (m->base) d->MemAddressFree(m->base, bytes);
    delete m;
    const char* s = nullptr; d->GetErrorString(r, &s);
    return set_error("map_remote_one: %s failed: %s", what, s ? s : "?");
  }
  *mapping_out = m; *base_out = (unsigned long long)m->base;
  return 0;
}

// One virtual range [local_bytes | chunk]: the first part is backed by NEW physical memory, the
// second part maps the physical memory of `tail_chunk` a second time. This is how several layers
// share one set of prefetch / reduce slots: each layer's compute view is [its own experts | the
// shared slots], contiguous for the grouped GEMM, while the slots exist once (and peers reach them
// through the slot heap's all-rank mapping). `local_bytes` must be a multiple of the granularity.
int mep_alias_map(int dev, size_t local_bytes, void* tail_chunk, void** alias_out, unsigned long long* va_out) {
  const DriverApi* d = driver(); if (!d) return -1;
  LocalChunk* lc = static_cast<LocalChunk*>(tail_chunk);
  MEP_REQUIRE(lc && lc->handle_live, "alias_map: the chunk to alias has been released");
  CUmemAllocationProp p = alloc_prop(dev, lc->kind);
  size_t gran = 0;
  MEP_CU_CHECK(d->MemGetAllocationGranularity(&gran, &p, CU_MEM_ALLOC_GRANULARITY_RECOMMENDED));
  MEP_REQUIRE(local_bytes > 0 && local_bytes % gran == 0,
              "alias_map: %zu local bytes are not a multiple of the mapping granularity %zu", local_bytes, gran);
  AliasMap* a = new AliasMap{dev, 0, local_bytes, lc->bytes, 0, false, false, false};
  const char* what = "reserve";
  CUresult r = d->MemAddressReserve(&a->va, local_bytes + lc->bytes, gran, 0, 0);
  if (r == CUDA_SUCCESS) { r = d->MemCreate(&a->local, local_bytes, &p, 0); what = "create"; a->local_live = r == CUDA_SUCCESS; }
  if (r == CUDA_SUCCESS) { r = d->MemMap(a->va, local_bytes, 0, a->local, 0); what = "map(local)"; a->local_mapped = r == CUDA_SUCCESS; }
  if (r == CUDA_SUCCESS) { r = d->MemMap(a->va + local_bytes, lc->bytes, 0, lc->handle, 0); what = "map(alias)"; a->tail_mapped = r == CUDA_SUCCESS; }
  if (r == CUDA_SUCCESS) {
    CUmemAccessDesc acc = {};
    acc.location.type = CU_MEM_LOCATION_TYPE_DEVICE; acc.location.id = dev; acc.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
    r = d->MemSetAccess(a->va, local_bytes + lc->bytes, &acc, 1); what = "set_access";
  }
  if (r != CUDA_SUCCESS) {
    const char* es = nullptr; d->GetErrorString(r, &es);
    size_t fr = 0, tot = 0; cudaMemGetInfo(&fr, &tot);
    const size_t lb = a->local_bytes;
    if (a->tail_mapped) d->MemUnmap(a->va + a->local_bytes, a->tail_bytes);
    if (a->local_mapped) d->MemUnmap(a->va, a->local_bytes);
    if (a->local_live) d->MemRelease(a->local);
    if (a->va) d->MemAddressFree(a->va, a->local_bytes + a->tail_bytes);
    delete a;
    return set_error("alias_map: %s failed: %s (%zu local bytes, %zu MiB free of %zu MiB)", what, es ? es : "?", lb, fr >> 20, tot >> 20);
  }
  *alias_out = a; *va_out = (unsigned long long)a->va;
  return 0;
}

// Undo mep_alias_map (the aliased chunk itself is untouched). Caller must have synchronised the device.
int mep_alias_unmap(void* alias) {
  AliasMap* a = static_cast<AliasMap*>(alias);
  if (!a) return 0;
  const DriverApi* d = driver();
  if (d) {
    if (a->tail_mapped) d->MemUnmap(a->va + a->local_bytes, a->tail_bytes);
    if (a->local_mapped) d->MemUnmap(a->va, a->local_bytes);
    if (a->local_live) d->MemRelease(a->local);
    d->MemAddressFree(a->va, a->local_bytes + a->tail_bytes);
  }
  delete a;
  return 0;
}

// Unmap every chunk and free the range. Caller must have synchronised the device.
int mep_unmap_all(void* mapping) {
  Mapping* m = static_cast<Mapping*>(mapping);
  if (!m) return 0;
  const DriverApi* d = driver();
  if (d) {
    for (int i = 0; i < m->world; ++i) if (m->mapped[i]) d->MemUnmap(m->base + (size_t)i * m->chunk_bytes, m->chunk_bytes);
    d->MemAddressFree(m->base, m->chunk_bytes * m->world);
  }
  delete m;
  return 0;
}

// ---- NVSwitch multicast. Order required by the driver: root creates + exports; everyone
// imports; everyone adds its device; (barrier); everyone binds its OWNED chunk handle;
// (barrier); only then is the multicast mapping used.
int mep_mc_create(int dev, int world, size_t bytes, int kind, void** mc_out, unsigned char shareable[64]) {
  const DriverApi* d = driver(); if (!d) return -1;
  CUmulticastObjectProp mp = {};
  mp.numDevices = world; mp.size = bytes; mp.handleTypes = cu_type(kind);
  Multicast* m = new Multicast{dev, bytes, 0, false, 0, false, false};
  CUresult r = d->MulticastCreate(&m->mc, &mp);
  if (r != CUDA_SUCCESS) { delete m; MEP_CU_CHECK(r); }
  m->mc_live = true;
  memset(shareable, 0, 64);
  if (kind == kHandleFabric) {
    CUmemFabricHandle fh; r = d->MemExportToShareableHandle(&fh, m->mc, CU_MEM_HANDLE_TYPE_FABRIC, 0);
    if (r == CUDA_SUCCESS) memcpy(shareable, &fh, sizeof fh);
  } else {
    int fd = -1; r = d->MemExportToShareableHandle(&fd, m->mc, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0);
    if (r == CUDA_SUCCESS) memcpy(shareable, &fd, sizeof fd);
  }
  if (r != CUDA_SUCCESS) { d->MemRelease(m->mc); delete m; MEP_CU_CHECK(r); }
  *mc_out = m;
  return 0;
}

int mep_mc_import(int dev, size_t bytes, int kind, const unsigned char shareable[64], void** mc_out) {
  const DriverApi* d = driver(); if (!d) return -1;
  Multicast* m = new Multicast{dev, bytes, 0, false, 0, false, false};
  CUresult r;
  if (kind == kHandleFabric) {
    CUmemFabricHandle fh; memcpy(&fh, shareable, sizeof fh);
    r = d->MemImportFromShareableHandle(&m->mc, &fh, CU_MEM_HANDLE_TYPE_FABRIC);
  } else {
    int fd; memcpy(&fd, shareable, sizeof fd);
    r = d->MemImportFromShareableHandle(&m->mc, (void*)(uintptr_t)fd, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR);
    close(fd);
  }
  if (r != CUDA_SUCCESS) { delete m; MEP_CU_CHECK(r); }
  m->mc_live = true;
  *mc_out = m;
  return 0;
}

int mep_mc_add_device(void* mc) {
  const DriverApi* d = driver(); if (!d) return -1;
  Multicast* m = static_cast<Multicast*>(mc);
  CUdevice cd; MEP_CU_CHECK(d->DeviceGet(&cd, m->dev));
  MEP_CU_CHECK(d->MulticastAddDevice(m->mc, cd));
  return 0;
}

// Bind this rank's owned chunk and map the multicast object. Returns the multicast VA.
int mep_mc_bind_map(void* mc, void* local_chunk, unsigned long long* va_out) {
  const DriverApi* d = driver(); if (!d) return -1;
  Multicast* m = static_cast<Multicast*>(mc);
  LocalChunk* lc = static_cast<LocalChunk*>(local_chunk);
  MEP_REQUIRE(lc && lc->handle_live, "mc_bind_map: the owned chunk handle is required (imported mappings cannot be bound)");
  MEP_REQUIRE(lc->bytes == m->bytes, "mc_bind_map: chunk %zu B != multicast object %zu B", lc->bytes, m->bytes);
  MEP_CU_CHECK(d->MulticastBindMem(m->mc, 0, lc->handle, 0, m->bytes, 0));
  m->bound = true;
  CUmemAllocationProp p = alloc_prop(m->dev, lc->kind);
  size_t gran = 0;
  MEP_CU_CHECK(d->MemGetAllocationGranularity(&gran, &p, CU_MEM_ALLOC_GRANULARITY_RECOMMENDED));
  MEP_CU_CHECK(d->MemAddressReserve(&m->va, m->bytes, gran, 0, 0));
  CUresult r = d->MemMap(m->va, m->bytes, 0, m->mc, 0);
  if (r != CUDA_SUCCESS) { d->MemAddressFree(m->va, m->bytes); m->va = 0; MEP_CU_CHECK(r); }
  m->mapped = true;
  CUmemAccessDesc acc = {};
  acc.location.type = CU_MEM_LOCATION_TYPE_DEVICE; acc.location.id = m->dev; acc.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
  MEP_CU_CHECK(d->MemSetAccess(m->va, m->bytes, &acc, 1));
  *va_out = (unsigned long long)m->va;
  return 0;
}

int mep_mc_destroy(void* mc) {
  Multicast* m = static_cast<Multicast*>(mc);
  if (!m) return 0;
  const DriverApi* d = driver();
  if (d) {
    if (m->mapped) { d->MemUnmap(m->va, m->bytes); d->MemAddressFree(m->va, m->bytes); }
    if (m->bound) { CUdevice cd; if (d->DeviceGet(&cd, m->dev) == CUDA_SUCCESS) d->MulticastUnbind(m->mc, cd, 0, m->bytes); }
    if (m->mc_live) d->MemRelease(m->mc);
  }
  delete m;
  return 0;
}

}  // extern "C"

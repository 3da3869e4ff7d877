// Caching device allocator: memory is reserved from the backend in large chunks; requests are rounded to
// 512-byte multiples and served best-fit from an address-ordered free list per chunk; freed blocks coalesce
// with their neighbours; chunks that become entirely free can be handed back (shrink), as the runtime does
// before a graph allocates its plan. Backend 1 resolves cudaMalloc / cudaFree from libcudart at run time so
// that this library links without CUDA; backend 0 uses the host heap (unit tests).
// The same functions are exported in the signature torch's pluggable-allocator hook expects
// (ofc_torch_alloc / ofc_torch_free), so the framework can run on this allocator.
//
// Reference: the VM's BinAllocator (oneflow/core/vm/bin_allocator.h, 448 lines) and ShrinkAllMem
// (oneflow/core/vm/virtual_machine.cpp:177-193).
#include <dlfcn.h>

#include <cstdlib>
#include <map>
#include <mutex>
#include <set>
#include <vector>

#include "common.h"
#include "ofc_core.h"

namespace {

constexpr int64_t kAlign = 512;

struct Backend {
  int kind;
  int (*cuda_malloc)(void**, size_t) = nullptr;
  int (*cuda_free)(void*) = nullptr;
  bool init() {
    if (kind == 0) return true;
    void* h = dlopen("libcudart.so", RTLD_NOW | RTLD_GLOBAL);
    if (!h) h = dlopen("libcudart.so.12", RTLD_NOW | RTLD_GLOBAL);
    if (!h) return false;
    cuda_malloc = reinterpret_cast<int (*)(void**, size_t)>(dlsym(h, "cudaMalloc"));
    cuda_free = reinterpret_cast<int (*)(void*)>(dlsym(h, "cudaFree"));
    return cuda_malloc && cuda_free;
  }
  void* alloc(size_t n) {
    if (kind == 0) {
      void* p = nullptr;
      return posix_memalign(&p, 4096, n) == 0 ? p : nullptr;
    }
    void* p = nullptr;
    return cuda_malloc(&p, n) == 0 ? p : nullptr;
  }
  void release(void* p) {
    if (kind == 0) std::free(p); else cuda_free(p);
  }
};

struct Block {
  char* ptr;
  int64_t size;
  bool free;
  int chunk;
};

struct Allocator {
  Backend be;
  int64_t chunk_bytes;
  std::mutex mu;
  std::map<char*, Block> blocks;                       // every block, address ordered
  std::multimap<int64_t, char*> free_by_size;          // best fit
  std::vector<std::pair<char*, int64_t>> chunks;       // base, size (base null when released)
  int64_t reserved = 0, in_use = 0;

  void erase_free(const Block& b) {
    auto r = free_by_size.equal_range(b.size);
    for (auto it = r.first; it != r.second; ++it)
      if (it->second == b.ptr) { free_by_size.erase(it); return; }
  }
  bool grow(int64_t need) {
    int64_t sz = need > chunk_bytes ? need : chunk_bytes;
    sz = (sz + kAlign - 1) / kAlign * kAlign;
    char* base = static_cast<char*>(be.alloc(static_cast<size_t>(sz)));
    if (!base) return false;
    const int id = static_cast<int>(chunks.size());
    chunks.emplace_back(base, sz);
    blocks[base] = Block{base, sz, true, id};
    free_by_size.emplace(sz, base);
    reserved += sz;
    return true;
  }
  void* alloc(int64_t bytes) {
    if (bytes <= 0) bytes = 1;
    const int64_t need = (bytes + kAlign - 1) / kAlign * kAlign;
    std::lock_guard<std::mutex> g(mu);
    auto it = free_by_size.lower_bound(need);
    if (it == free_by_size.end()) {
      if (!grow(need)) return nullptr;
      it = free_by_size.lower_bound(need);
    }
    char* p = it->second;
    free_by_size.erase(it);
    Block& b = blocks[p];
    if (b.size - need >= kAlign) {
      Block rest{p + need, b.size - need, true, b.chunk};
      b.size = need;
      blocks[rest.ptr] = rest;
      free_by_size.emplace(rest.size, rest.ptr);
    }
    b.free = false;
    in_use += b.size;
    return p;
  }
  int free_block(void* ptr) {
    std::lock_guard<std::mutex> g(mu);
    auto it = blocks.find(static_cast<char*>(ptr));
    if (it == blocks.end() || it->second.free) return ofc::fail("allocator: pointer was not allocated here (or double free)");
    in_use -= it->second.size;
    it->second.free = true;
    // merge with the next block
    auto nx = std::next(it);
    if (nx != blocks.end() && nx->second.free && nx->second.chunk == it->second.chunk && it->first + it->second.size == nx->first) {
      erase_free(nx->second);
      it->second.size += nx->second.size;
      blocks.erase(nx);
    }
    // merge with the previous block
    if (it != blocks.begin()) {
      auto pv = std::prev(it);
      if (pv->second.free && pv->second.chunk == it->second.chunk && pv->first + pv->second.size == it->first) {
        erase_free(pv->second);
        pv->second.size += it->second.size;
        blocks.erase(it);
        it = pv;
      }
    }
    free_by_size.emplace(it->second.size, it->first);
    return 0;
  }
  int shrink() {
    std::lock_guard<std::mutex> g(mu);
    int n = 0;
    for (auto& c : chunks) {
      if (!c.first) continue;
      auto it = blocks.find(c.first);
      if (it != blocks.end() && it->second.free && it->second.size == c.second) {
        erase_free(it->second);
        blocks.erase(it);
        be.release(c.first);
        reserved -= c.second;
        c.first = nullptr;
        ++n;
      }
    }
    return n;
  }
};

Allocator* g_torch_allocator = nullptr;

}  // namespace

OFC_API void* ofc_allocator_create(int backend, int64_t chunk_bytes) {
  auto* a = new Allocator();
  a->be.kind = backend;
  a->chunk_bytes = chunk_bytes > 0 ? chunk_bytes : (int64_t{1} << 30);
  if (!a->be.init()) {
    ofc::fail("allocator: the CUDA runtime library could not be loaded");
    delete a;
    return nullptr;
  }
  return a;
}
OFC_API void ofc_allocator_destroy(void* p) {
  auto* a = static_cast<Allocator*>(p);
  for (auto& c : a->chunks)
    if (c.first) a->be.release(c.first);
  if (g_torch_allocator == a) g_torch_allocator = nullptr;
  delete a;
}
OFC_API void* ofc_allocator_alloc(void* a, int64_t bytes) {
  void* p = static_cast<Allocator*>(a)->alloc(bytes);
  if (!p) ofc::fail("allocator: out of memory");
  return p;
}
OFC_API int ofc_allocator_free(void* a, void* ptr) { return static_cast<Allocator*>(a)->free_block(ptr); }
OFC_API int ofc_allocator_shrink(void* a) { return static_cast<Allocator*>(a)->shrink(); }
OFC_API void ofc_allocator_stats(void* p, int64_t* reserved, int64_t* in_use, int64_t* n_chunks, int64_t* n_free_blocks) {
  auto* a = static_cast<Allocator*>(p);
  std::lock_guard<std::mutex> g(a->mu);
  if (reserved) *reserved = a->reserved;
  if (in_use) *in_use = a->in_use;
  if (n_chunks) {
    int64_t n = 0;
    for (auto& c : a->chunks) n += c.first != nullptr;
    *n_chunks = n;
  }
  if (n_free_blocks) *n_free_blocks = static_cast<int64_t>(a->free_by_size.size());
}

// torch.cuda.memory.CUDAPluggableAllocator(path, "ofc_torch_alloc", "ofc_torch_free") entry points.
extern "C" __attribute__((visibility("default"))) void* ofc_torch_alloc(size_t size, int device, void* stream) {
  (void)device;
  (void)stream;
  if (!g_torch_allocator) g_torch_allocator = static_cast<Allocator*>(ofc_allocator_create(1, int64_t{2} << 30));
  return g_torch_allocator ? g_torch_allocator->alloc(static_cast<int64_t>(size)) : nullptr;
}
extern "C" __attribute__((visibility("default"))) void ofc_torch_free(void* ptr, size_t size, int device, void* stream) {
  (void)size;
  (void)device;
  (void)stream;
  if (g_torch_allocator && ptr) g_torch_allocator->free_block(ptr);
}

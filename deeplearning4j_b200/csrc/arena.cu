// Workspace arena: one slab per workspace, bump allocation inside a cycle, spill blocks when the slab is full, learning of the
// cycle's high-water mark so that the slab can be re-created at the right size.  This is the native half of the workspace
// machinery (libnd4j/include/memory/Workspace.h, impl/Workspace.cpp): the Python MemoryWorkspace drives the policies, the arena
// owns the memory and hands out aligned addresses, so that tensors of one training step come out of one preallocated block
// instead of the general allocator.
//
// kind: 0 = host (malloc), 1 = pinned host (cudaMallocHost), 2 = device (cudaMalloc on the current device).
#include "common.cuh"

#include <cstdlib>
#include <mutex>
#include <vector>

namespace {

struct Arena {
  int kind = 0;
  char* slab = nullptr;
  size_t capacity = 0, offset = 0;
  size_t cycle_bytes = 0, max_cycle = 0, spilled_bytes = 0;
  unsigned long long generation = 0, cycles = 0;
  std::vector<std::pair<void*, size_t>> spills;
  std::mutex mu;
};

void* raw_alloc(int kind, size_t n) {
  void* p = nullptr;
  if (n == 0) return nullptr;
  if (kind == 0) {
    if (posix_memalign(&p, 256, n) != 0) return nullptr;
  } else if (kind == 1) {
    if (cudaMallocHost(&p, n) != cudaSuccess) return nullptr;
  } else {
    if (cudaMalloc(&p, n) != cudaSuccess) return nullptr;
  }
  return p;
}

void raw_free(int kind, void* p) {
  if (!p) return;
  if (kind == 0) free(p);
  else if (kind == 1) cudaFreeHost(p);
  else cudaFree(p);
}

}  // namespace

DL4J_API void* dl4j_arena_create(int kind, long long initial_bytes) {
  if (kind < 0 || kind > 2 || initial_bytes < 0) return nullptr;
  Arena* a = new Arena();
  a->kind = kind;
  if (initial_bytes > 0) {
    a->slab = static_cast<char*>(raw_alloc(kind, (size_t)initial_bytes));
    if (!a->slab) { delete a; return nullptr; }
    a->capacity = (size_t)initial_bytes;
  }
  return a;
}

DL4J_API void dl4j_arena_destroy(void* h) {
  Arena* a = static_cast<Arena*>(h);
  if (!a) return;
  for (auto& s : a->spills) raw_free(a->kind, s.first);
  raw_free(a->kind, a->slab);
  delete a;
}

// Address of `bytes` bytes aligned to `align` (a power of two, at least 16).  Inside the slab when it fits; otherwise, with
// allow_spill, a separate block that lives until the end of the cycle; otherwise null.  *spilled tells which.
DL4J_API void* dl4j_arena_alloc(void* h, long long bytes, int align, int allow_spill, int* spilled) {
  Arena* a = static_cast<Arena*>(h);
  if (!a || bytes < 0 || align < 16 || (align & (align - 1))) return nullptr;
  std::lock_guard<std::mutex> lk(a->mu);
  const size_t n = ((size_t)bytes + (size_t)align - 1) & ~((size_t)align - 1);
  a->cycle_bytes += n;
  if (spilled) *spilled = 0;
  if (a->slab) {
    const size_t base = reinterpret_cast<uintptr_t>(a->slab);
    const size_t start = ((base + a->offset + (size_t)align - 1) & ~((size_t)align - 1)) - base;
    if (start + n <= a->capacity) {
      a->offset = start + n;
      return a->slab + start;
    }
  }
  if (!allow_spill) return nullptr;
  void* p = raw_alloc(a->kind, n ? n : (size_t)align);
  if (!p) return nullptr;
  a->spills.emplace_back(p, n);
  a->spilled_bytes += n;
  if (spilled) *spilled = 1;
  return p;
}

// End of a cycle: spill blocks are released, the bump pointer returns to the start, the high-water mark is updated.
DL4J_API void dl4j_arena_reset(void* h) {
  Arena* a = static_cast<Arena*>(h);
  if (!a) return;
  std::lock_guard<std::mutex> lk(a->mu);
  if (a->cycle_bytes > a->max_cycle) a->max_cycle = a->cycle_bytes;
  for (auto& s : a->spills) raw_free(a->kind, s.first);
  a->spills.clear();
  a->spilled_bytes = 0;
  a->offset = 0;
  a->cycle_bytes = 0;
  a->generation++;
  a->cycles++;
}

// Replaces the slab by one of `bytes` bytes (only between cycles: nothing handed out earlier stays valid).  Returns 0 on success.
DL4J_API int dl4j_arena_resize(void* h, long long bytes) {
  Arena* a = static_cast<Arena*>(h);
  if (!a || bytes < 0) return -1;
  std::lock_guard<std::mutex> lk(a->mu);
  if (a->offset != 0 || !a->spills.empty()) return -2;
  char* s = bytes ? static_cast<char*>(raw_alloc(a->kind, (size_t)bytes)) : nullptr;
  if (bytes && !s) return -3;
  raw_free(a->kind, a->slab);
  a->slab = s;
  a->capacity = (size_t)bytes;
  return 0;
}

// out[0..7] = capacity, offset, bytes requested this cycle, largest cycle so far, spilled bytes, generation, cycles, spill blocks
DL4J_API void dl4j_arena_stats(void* h, long long* out) {
  Arena* a = static_cast<Arena*>(h);
  if (!a || !out) return;
  std::lock_guard<std::mutex> lk(a->mu);
  out[0] = (long long)a->capacity; out[1] = (long long)a->offset; out[2] = (long long)a->cycle_bytes; out[3] = (long long)a->max_cycle;
  out[4] = (long long)a->spilled_bytes; out[5] = (long long)a->generation; out[6] = (long long)a->cycles; out[7] = (long long)a->spills.size();
}

DL4J_API void* dl4j_arena_base(void* h) {
  Arena* a = static_cast<Arena*>(h);
  return a ? a->slab : nullptr;
}

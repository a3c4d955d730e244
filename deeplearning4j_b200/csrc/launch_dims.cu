// Launch table and device validation (reference: libnd4j execution/cuda/LaunchDims.h:14-222 — a name -> {grid, block, shared
// memory} map whose entries can be overridden with GRID_SIZE_<NAME> / BLOCK_SIZE_<NAME> / SHARED_MEM_SIZE_<NAME>, and
// execution/cuda/DeviceValidator.cu — limits checked before a launch).
//
// Here the table holds the free launch parameters of the grid-stride kernels: `grid` is the number of blocks per SM the host
// entry point aims for (the kernels derive their row slabs from it), `block` and `shmem` are informational for kernels whose
// block shape is fixed at compile time (an override that contradicts a compile-time shape is rejected by the validator instead
// of being applied).  Everything in this file is host code; nothing touches a device unless a validator query asks for the
// current device's limits.
#include "common.cuh"

#include <cctype>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>

namespace {

struct Entry {
  const char* name;       // upper-case, as used in the environment variable
  int grid, block, shmem; // defaults
  int fixed_block;        // 1: the kernel's block size is a compile-time constant
  int cur[3];             // resolved values (defaults overridden by the environment)
  int resolved;
};

Entry g_table[] = {
    {"LAYER_NORM_FWD", 4, 256, 0, 1, {0, 0, 0}, 0},
    {"LAYER_NORM_BWD_DX", 4, 256, 0, 1, {0, 0, 0}, 0},
    {"LAYER_NORM_BWD_COLS", 6, 256, 16896, 1, {0, 0, 0}, 0},
    {"BIAS_ACT_BWD", 6, 256, 8448, 1, {0, 0, 0}, 0},
    {"SCATTER_ADD_ROWS", 16, 256, 0, 1, {0, 0, 0}, 0},
    {"SOFTMAX_XENT", 0, 256, 32, 1, {0, 0, 0}, 0},          // grid = rows
    {"LSTM_CELL", 8, 256, 0, 1, {0, 0, 0}, 0},
    {"FUSED_UPDATE", 8, 256, 0, 1, {0, 0, 0}, 0},
    {"GEMM_TCGEN05", 1, 192, 230656, 1, {0, 0, 0}, 0},      // persistent: one CTA per SM
    {"FLASH_ATTN_FWD", 2, 320, 101000, 1, {0, 0, 0}, 0},
    {"FLASH_ATTN_BWD", 1, 576, 165000, 1, {0, 0, 0}, 0},
};
constexpr int N_ENTRIES = sizeof(g_table) / sizeof(g_table[0]);
std::mutex g_mu;

int env_int(const char* prefix, const char* name, int fallback) {
  char key[128];
  snprintf(key, sizeof(key), "%s%s", prefix, name);
  const char* v = getenv(key);
  if (!v || !*v) return fallback;
  char* end = nullptr;
  const long x = strtol(v, &end, 10);
  if (end == v || x < 0 || x > (1L << 30)) return fallback;     // malformed or absurd values are ignored
  return (int)x;
}

Entry* find(const char* name) {
  if (!name) return nullptr;
  char up[96];
  size_t n = strlen(name);
  if (n >= sizeof(up)) return nullptr;
  for (size_t i = 0; i <= n; ++i) up[i] = (char)toupper((unsigned char)name[i]);
  for (int i = 0; i < N_ENTRIES; ++i)
    if (strcmp(g_table[i].name, up) == 0) return &g_table[i];
  return nullptr;
}

void resolve(Entry* e) {
  if (e->resolved) return;
  e->cur[0] = env_int("GRID_SIZE_", e->name, e->grid);
  e->cur[1] = env_int("BLOCK_SIZE_", e->name, e->block);
  e->cur[2] = env_int("SHARED_MEM_SIZE_", e->name, e->shmem);
  e->resolved = 1;
}

}  // namespace

// Blocks per SM that a host entry point should aim for (internal; falls back to `fallback` for unknown names).
int dl4j_launch_grid(const char* name, int fallback) {
  std::lock_guard<std::mutex> lk(g_mu);
  Entry* e = find(name);
  if (!e) return fallback;
  resolve(e);
  return e->cur[0] > 0 ? e->cur[0] : fallback;
}

// out[0..2] = grid (blocks per SM, 0 = data dependent), block, shared memory bytes; out[3] = 1 when the block size is fixed at
// compile time.  Returns 0, or -1 for an unknown kernel name.
DL4J_API int dl4j_launch_dims(const char* name, int* out) {
  std::lock_guard<std::mutex> lk(g_mu);
  Entry* e = find(name);
  if (!e || !out) return -1;
  resolve(e);
  out[0] = e->cur[0]; out[1] = e->cur[1]; out[2] = e->cur[2]; out[3] = e->fixed_block;
  return 0;
}

// Forget resolved values so that the environment is read again (used by tests and after Environment changes).
DL4J_API void dl4j_launch_dims_reload() {
  std::lock_guard<std::mutex> lk(g_mu);
  for (int i = 0; i < N_ENTRIES; ++i) g_table[i].resolved = 0;
}

DL4J_API int dl4j_launch_dims_count() { return N_ENTRIES; }
DL4J_API const char* dl4j_launch_dims_name(int i) { return (i >= 0 && i < N_ENTRIES) ? g_table[i].name : nullptr; }

// Validation against explicit limits {max threads per block, max shared memory per block, max grid x, warp size}: 0 = fits,
// otherwise a bit set: 1 block too large / not a warp multiple, 2 shared memory, 4 grid, 8 contradicts a compile-time block shape.
DL4J_API int dl4j_validate_launch(const char* name, long long grid, int block, int shmem, const int* limits) {
  int bad = 0;
  if (!limits) return -1;
  if (block <= 0 || block > limits[0] || (limits[3] > 0 && block % limits[3] != 0)) bad |= 1;
  if (shmem < 0 || shmem > limits[1]) bad |= 2;
  if (grid <= 0 || grid > (long long)limits[2]) bad |= 4;
  std::lock_guard<std::mutex> lk(g_mu);
  Entry* e = find(name);
  if (e && e->fixed_block && block != e->block) bad |= 8;
  return bad;
}

// Limits of the current device in the layout dl4j_validate_launch takes; returns a CUDA error code.
DL4J_API int dl4j_device_limits(int* limits) {
  if (!limits) return -1;
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return (int)e;
  cudaDeviceGetAttribute(&limits[0], cudaDevAttrMaxThreadsPerBlock, dev);
  cudaDeviceGetAttribute(&limits[1], cudaDevAttrMaxSharedMemoryPerBlockOptin, dev);
  cudaDeviceGetAttribute(&limits[2], cudaDevAttrMaxGridDimX, dev);
  cudaDeviceGetAttribute(&limits[3], cudaDevAttrWarpSize, dev);
  return 0;
}

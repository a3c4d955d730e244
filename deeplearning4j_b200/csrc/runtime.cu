// Library runtime: driver entry points obtained without linking libcuda, the per-device status
// word that bounded waits report into, and small queries used by the Python side.
#include "common.cuh"

#include <mutex>

static std::mutex g_mu;
static dl4j_PFN_encodeTiled g_encode = nullptr;
static int* g_status[64] = {nullptr};

dl4j_PFN_encodeTiled dl4j_get_encode_tiled() {
  std::lock_guard<std::mutex> lk(g_mu);
  if (g_encode) return g_encode;
  void* fn = nullptr;
  cudaDriverEntryPointQueryResult q;
  if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q) != cudaSuccess ||
      q != cudaDriverEntryPointSuccess)
    return nullptr;
  g_encode = reinterpret_cast<dl4j_PFN_encodeTiled>(fn);
  return g_encode;
}

int* dl4j_status_word(int device) {
  std::lock_guard<std::mutex> lk(g_mu);
  if (device < 0 || device >= 64) return nullptr;
  if (!g_status[device]) {
    int* p = nullptr;
    if (cudaMalloc(&p, 256) != cudaSuccess) return nullptr;
    cudaMemset(p, 0, 256);
    g_status[device] = p;
  }
  return g_status[device];
}

// Returns the status word's value (0 = no bounded wait has expired) and clears it.
DL4J_API int dl4j_read_status(int reset) {
  int dev = 0;
  cudaGetDevice(&dev);
  int* p = dl4j_status_word(dev);
  if (!p) return -1;
  int v = 0;
  if (cudaMemcpy(&v, p, sizeof(int), cudaMemcpyDeviceToHost) != cudaSuccess) return -2;
  if (reset && v != 0) cudaMemset(p, 0, sizeof(int));
  return v;
}

// Queues an asynchronous copy of the status word into `pinned_host` (4 bytes of page-locked memory) on `stream`:
// the host learns of an expired wait one step later without synchronising the device.
DL4J_API int dl4j_status_snapshot(void* pinned_host, void* stream) {
  int dev = 0;
  cudaGetDevice(&dev);
  int* p = dl4j_status_word(dev);
  if (!p || !pinned_host) return -1;
  return (int)cudaMemcpyAsync(pinned_host, p, sizeof(int), cudaMemcpyDeviceToHost, (cudaStream_t)stream);
}

DL4J_API void* dl4j_status_ptr() {
  int dev = 0;
  cudaGetDevice(&dev);
  return dl4j_status_word(dev);
}

DL4J_API int dl4j_num_sms() {
  int dev = 0, n = 0;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
  return n;
}

DL4J_API int dl4j_abi_version() { return 1; }

#ifdef DL4J_DEBUG_BOUNDS
__device__ unsigned long long dl4j_dbg_bounds[4] = {0ULL, 0ULL, 0ULL, 0ULL};
#endif

// Debug-bounds build only: copies {failures, source line, offset, extent of the first failure} into out[4] (synchronises) and
// clears the record when `reset` is set.  Returns 0, or -1 in a build without the checks.
DL4J_API int dl4j_debug_bounds(unsigned long long* out, int reset) {
#ifdef DL4J_DEBUG_BOUNDS
  if (cudaMemcpyFromSymbol(out, dl4j_dbg_bounds, 4 * sizeof(unsigned long long)) != cudaSuccess) return -2;
  if (reset && out[0] != 0ULL) {
    const unsigned long long z[4] = {0ULL, 0ULL, 0ULL, 0ULL};
    if (cudaMemcpyToSymbol(dl4j_dbg_bounds, z, sizeof(z)) != cudaSuccess) return -2;
  }
  return 0;
#else
  (void)out; (void)reset;
  return -1;
#endif
}

// Binds `device`'s primary context to the calling thread for this library's runtime instance.  The
// library is linked against its own (static) CUDA runtime; a thread that has only used another runtime
// instance so far (e.g. an autograd worker thread) may have no context bound yet, and driver entry
// points such as cuTensorMapEncodeTiled then fail with CUDA_ERROR_INVALID_CONTEXT.
DL4J_API int dl4j_bind_device(int device) {
  static thread_local int bound = -1;
  if (bound == device) return 0;
  cudaError_t e = cudaSetDevice(device);
  if (e != cudaSuccess) return (int)e;
  e = cudaFree(nullptr);
  if (e != cudaSuccess) return (int)e;
  bound = device;
  return 0;
}

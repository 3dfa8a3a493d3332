// Cross entropy without any allocation: the per-position scratch lives in a static device array.
//
// Some hosts cannot call cudaMalloc once they are running: a serving process that handed the whole
// GPU to its own arena at start-up, or a latency-critical loop that must not pay the implicit
// device synchronisation of cudaMalloc/cudaFree.  They pass device pointers for the inputs and the
// output and this entry point supplies the intermediate storage itself.
#include "common.h"

#include <string.h>

#include <atomic>

namespace bg {
namespace {

constexpr int64_t kNoAllocMaxPositions = 1 << 20;   // rows x spatial positions per call
constexpr size_t kHeaderBytes = 256;                 // status word, kept apart from the data

// 4 MiB + 256 B on every GPU that loads the library, until the process exits.
static __device__ __align__(256) unsigned char g_ce_scratch[kHeaderBytes + kNoAllocMaxPositions * sizeof(float)];

// The array's name is a host-side stand-in, not a device address: the address each device uses is
// looked up once per device with that device current.  Host threads may race to fill a slot; they all store the
// same address, atomically.
std::atomic<void*> g_scratch_ptr[64];

void set_err(char* err, size_t cap, const char* msg) {
  if (err && cap) {
    strncpy(err, msg, cap - 1);
    err[cap - 1] = 0;
  }
}

}  // namespace
}  // namespace bg

extern "C" int bg_cross_entropy_noalloc(const float* logits, const int64_t* targets, float* out, int64_t rows,
                                        int64_t classes, int64_t inner, int reduction, int64_t ignore_index,
                                        void* stream, char* err, size_t err_capacity) {
  using namespace bg;
  if (!logits || !targets || !out) { set_err(err, err_capacity, "CUDA bridge: cross_entropy_noalloc: null pointer"); return BG_ERR_INVALID; }
  if (rows < 0 || classes <= 0 || inner <= 0) { set_err(err, err_capacity, "CUDA bridge: cross_entropy_noalloc: bad shape"); return BG_ERR_INVALID; }
  if (reduction != 1 && reduction != 2) { set_err(err, err_capacity, "CUDA bridge: cross_entropy_noalloc: reduction must be 1 (mean) or 2 (sum)"); return BG_ERR_INVALID; }
  // rows * inner is compared without being formed: two huge extents must not wrap to a small product
  const int64_t positions = rows > kNoAllocMaxPositions / inner ? kNoAllocMaxPositions + 1 : rows * inner;
  if (positions > kNoAllocMaxPositions) {
    char msg[200];
    snprintf(msg, sizeof(msg), "CUDA bridge: cross_entropy_noalloc: %lld x %lld positions exceed the static scratch of %lld; use run_tensor_plan",
             (long long)rows, (long long)inner, (long long)kNoAllocMaxPositions);
    set_err(err, err_capacity, msg);
    return BG_ERR_UNSUPPORTED;
  }
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess || dev < 0 || dev >= 64) { set_err(err, err_capacity, "CUDA bridge: cross_entropy_noalloc: no current device"); return BG_ERR_CUDA; }
  void* scratch = g_scratch_ptr[dev].load(std::memory_order_acquire);
  if (!scratch) {
    // first call on this device: resolve the device address of the static array
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, g_ce_scratch);
    if (e != cudaSuccess || !p) {
      cudaGetLastError();
      set_err(err, err_capacity, "CUDA bridge: cross_entropy_noalloc: cudaGetSymbolAddress failed");
      return BG_ERR_CUDA;
    }
    g_scratch_ptr[dev].store(p, std::memory_order_release);
    scratch = p;
  }
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  unsigned char* base = reinterpret_cast<unsigned char*>(scratch);
  int* status = reinterpret_cast<int*>(base);
  float* per_pos = reinterpret_cast<float*>(base + kHeaderBytes);
  // the array keeps the previous call's contents: the status word must start at zero, the
  // per-position values are all rewritten before they are read
  e = cudaMemsetAsync(status, 0, sizeof(int), st);
  if (e == cudaSuccess && positions > 0) {
    CeProblem c{};
    c.logits = logits; c.targets = targets; c.per_pos = per_pos;
    c.dtype = BG_F32;
    c.outer = rows; c.C = classes; c.inner = inner; c.ignore_index = ignore_index;
    c.status = status;
    e = launch_ce_rows(c, st);
  }
  if (e == cudaSuccess) e = launch_ce_reduce(per_pos, targets, nullptr, out, BG_F32, positions, reduction, ignore_index, 0.0, st);
  int host_status = 0;
  if (e == cudaSuccess) e = cudaMemcpyAsync(&host_status, status, sizeof(int), cudaMemcpyDeviceToHost, st);
  if (e == cudaSuccess) e = cudaStreamSynchronize(st);
  if (e != cudaSuccess) {
    set_err(err, err_capacity, cudaGetErrorString(e));
    return BG_ERR_CUDA;
  }
  if (host_status != 0) {
    set_err(err, err_capacity, "CUDA bridge: cross_entropy_noalloc: target index outside [0, classes)");
    return host_status;
  }
  return BG_OK;
}

// Host-side runtime of libbgcuda.so: context, handle table, stream-ordered allocator,
// compiled-plan cache.  Internal to the library.
#pragma once

#include "common.h"

namespace bg {

struct HandleRec {
  void* ptr = nullptr;
  int64_t bytes = 0;       // logical bytes (numel * itemsize), what the accounting reports
  int dtype = BG_F32;
  std::vector<int64_t> shape;
};

struct CompiledPlan;

struct ProfileAcc {
  double ms = 0;
  int launches = 0;
};

}  // namespace bg

struct bg_context {
  int device = 0;
  int sm_count = 148;
  cudaStream_t stream = nullptr;
  std::string err;
  std::unordered_map<int64_t, bg::HandleRec> handles;
  int64_t next_handle = 1;
  // byte accounting (logical bytes), mirrors the reference bridge's resource snapshot
  int64_t cur_bytes = 0, peak_bytes = 0, total_alloc = 0, total_rel = 0, plan_peak = 0;
  int64_t launches = 0, cache_hits = 0, cache_misses = 0;
  // options
  bool profiling = false;
  int f64_mode = 2;
  bool fusion = true;
  bool tensor_cores = true;
  bool static_patterns = true;   // use the specialised pattern kernels where an expression matches
  bool gemm_groups = true;       // launch tensor-core GEMMs that share their A operand together
  // device status word written by kernels that can refuse (index range, bounded waits)
  int* d_status = nullptr;
  int* h_status = nullptr;  // pinned
  bool status_pending = false;   // a plan that may have set the word ended without a synchronising check
  int* gemm_counters = nullptr;  // 1024 device ints, zero between launches: tile arrival counters of the split-K small GEMM
  // pinned staging for host <-> device copies
  void* stage = nullptr;
  size_t stage_bytes = 0;
  std::unordered_map<uint64_t, std::shared_ptr<bg::CompiledPlan>> plan_cache;
  std::map<std::string, bg::ProfileAcc> profile;
  std::vector<std::pair<std::string, std::pair<cudaEvent_t, cudaEvent_t>>> pending_events;
  std::string last_trace;
  // "this fp32 buffer holds one repeated value" flags for buffers bound by handle, keyed by device
  // pointer; a flag is 1 when uniform, 0 when not; entries die with their handle
  std::unordered_map<const void*, int*> uniform_flags;
  int* uniform_pool = nullptr;      // 1024 device ints
  std::vector<int> uniform_free;
  // attention mask tile classes + per-row mask bit words for masks bound by handle (their contents cannot
  // change while the handle lives), keyed by device pointer; entries die with their handle
  struct MaskClasses { void* buf; int64_t bytes; int sq, sk, bkv, is_bool; };
  std::unordered_map<const void*, MaskClasses> mask_classes;
  // hi / lo tf32 planes (2 x n floats, hi first) of fp32 / fp64 matrices bound by handle that feed 3xTF32 GEMMs as the
  // B operand (weights): split once, kept until the handle is released
  struct SplitPlanes { float* buf; int64_t n; int dtype; };
  std::unordered_map<const void*, SplitPlanes> split_planes;
  // f16 / bf16 copies of fp32 matrices bound by handle that an autocast graph casts ahead of a GEMM (weights)
  struct CastCopy { void* buf; int64_t bytes; int dtype; };
  std::unordered_map<const void*, CastCopy> cast_copies;
  // Freed device blocks kept for the next allocation of exactly the same (padded) size: repeated plans ask for the
  // same sizes in the same order, so steady state makes no driver allocator call at all.  One stream per context, so
  // reuse is ordered behind the block's last use.  Bounded by block_cache_cap; flushed on allocation failure.
  std::unordered_multimap<size_t, void*> block_cache;
  size_t block_cache_bytes = 0;
  size_t block_cache_cap = (size_t)16 << 30;
  // fault injection on the host (tests): the n-th device allocation from now fails as an exhausted device would
  int64_t fail_alloc_countdown = 0;
};

namespace bg {

int fail(bg_context* ctx, int code, const std::string& msg);
int cuda_fail(bg_context* ctx, cudaError_t e, const char* what);

// Stream-ordered allocation with exact logical accounting.
int dev_alloc(bg_context* ctx, int64_t logical_bytes, void** out);
void dev_free(bg_context* ctx, void* p, int64_t logical_bytes);
bg_handle mint_handle(bg_context* ctx, void* ptr, int64_t bytes, int dtype, const int64_t* shape, int rank);
int h2d(bg_context* ctx, void* dst, const void* src, size_t n);
int d2h(bg_context* ctx, void* dst, const void* src, size_t n);

// Compile (or fetch from the cache) and run a plan.  When `out_host` is non-null the root is
// copied to the host and the stream synchronised; otherwise a handle to the root is minted.
// Device flag telling whether the handle-backed buffer at `ptr` is uniform; *fresh is set when the flag
// was just created and still has to be computed.  Returns nullptr when the pool is exhausted.
int* uniform_flag_for(bg_context* ctx, const void* ptr, bool* fresh);
void uniform_flag_drop(bg_context* ctx, const void* ptr);
// Device buffer holding the tile classes of the handle-backed mask at `ptr` for this geometry; *fresh is set
// when it was just allocated and still has to be computed.  Returns nullptr when the allocation fails.
void* mask_classes_for(bg_context* ctx, const void* ptr, int64_t bytes, int sq, int sk, int bkv, int is_bool, bool* fresh);
void mask_classes_drop(bg_context* ctx, const void* ptr);
// hi / lo planes kept for the handle-backed matrix at `ptr` (hi at the returned pointer, lo n floats later); *fresh is
// set when they were just allocated and still have to be computed.  nullptr when the allocation fails.
float* split_planes_for(bg_context* ctx, const void* ptr, int64_t n, int dtype, bool* fresh);
void split_planes_drop(bg_context* ctx, const void* ptr);
// 16-bit copy kept for the handle-backed fp32 matrix at `ptr`; *fresh is set when it still has to be computed.
void* cast_copy_for(bg_context* ctx, const void* ptr, int64_t bytes, int dtype, bool* fresh);
void cast_copy_drop(bg_context* ctx, const void* ptr);

int take_device_status(bg_context* ctx);
std::string device_status_message(int status_rc);
int run_plan(bg_context* ctx, const bg_plan* plan, const bg_plan_input* inputs, int n_inputs, void* out_host,
             size_t out_nbytes, bg_handle* out_handle);

}  // namespace bg

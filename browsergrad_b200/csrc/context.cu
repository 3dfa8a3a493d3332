// C ABI entry points for lifecycle, buffers, per-op methods and diagnostics.
// The per-op methods (matmul, fused_elementwise, cast, flash_attention) build a small plan and run
// it through the same compiler and kernels as run_tensor_plan, so there is one code path.
#include "runtime.h"

#include <string.h>

namespace bg {

const char* dtype_name(int dt) {
  static const char* names[] = {"float16", "float32", "float64", "int8", "int16", "int32", "int64",
                                "uint8", "uint16", "uint32", "uint64", "bool", "bfloat16"};
  return (dt >= 0 && dt <= BG_BF16) ? names[dt] : "?";
}

const char* op_name(int op) {
  static const char* names[] = {"BUFFER", "LOAD", "CONST", "CAST", "ADD", "MUL", "DIV", "NEG", "EXP", "LOG",
                                "ABS", "SIGN", "SIN", "COS", "ISNAN", "CMP", "WHERE", "MATMUL", "REDUCE",
                                "RESHAPE", "PERMUTE", "BROADCAST_TO", "LAYER_NORM", "CROSS_ENTROPY", "INDEX",
                                "FUSED_ELEMENTWISE", "FUSED_SOFTMAX", "ATTENTION_FORWARD", "TRIL", "TRIU", "FLIP", "CONCAT",
                                "CUMSUM", "SORT_INDICES", "TOPK_INDICES", "SCATTER", "SLICE"};
  return (op >= 0 && op < BG_OP_COUNT) ? names[op] : "?";
}

int fail(bg_context* ctx, int code, const std::string& msg) {
  if (ctx) ctx->err = "CUDA bridge: " + msg;
  return code;
}

int cuda_fail(bg_context* ctx, cudaError_t e, const char* what) {
  std::string m = std::string(what) + " failed: " + cudaGetErrorString(e);
  return fail(ctx, e == cudaErrorMemoryAllocation ? BG_ERR_OOM : BG_ERR_CUDA, m);
}

static size_t padded_size(int64_t logical_bytes) { return ((size_t)(logical_bytes > 0 ? logical_bytes : 1) + 255) & ~(size_t)255; }

static void flush_block_cache(bg_context* ctx) {
  for (auto& kv : ctx->block_cache) cudaFreeAsync(kv.second, ctx->stream);
  ctx->block_cache.clear();
  ctx->block_cache_bytes = 0;
}

int dev_alloc(bg_context* ctx, int64_t logical_bytes, void** out) {
  const size_t padded = padded_size(logical_bytes);
  // test hook (option "fail_allocation_after"): the n-th allocation from now reports what an exhausted device would
  if (ctx->fail_alloc_countdown > 0 && --ctx->fail_alloc_countdown == 0)
    return cuda_fail(ctx, cudaErrorMemoryAllocation, "device allocation");
  auto hit = ctx->block_cache.find(padded);
  if (hit != ctx->block_cache.end()) {
    *out = hit->second;
    ctx->block_cache.erase(hit);
    ctx->block_cache_bytes -= padded;
  } else {
    cudaError_t e = cudaMallocAsync(out, padded, ctx->stream);
    if (e != cudaSuccess && !ctx->block_cache.empty()) {
      // give the kept blocks back to the pool and try once more
      cudaGetLastError();
      flush_block_cache(ctx);
      cudaStreamSynchronize(ctx->stream);
      e = cudaMallocAsync(out, padded, ctx->stream);
    }
    if (e != cudaSuccess) {
      cudaGetLastError();
      return cuda_fail(ctx, e, "device allocation");
    }
  }
  ctx->cur_bytes += logical_bytes;
  ctx->total_alloc += logical_bytes;
  if (ctx->cur_bytes > ctx->peak_bytes) ctx->peak_bytes = ctx->cur_bytes;
  return BG_OK;
}

void dev_free(bg_context* ctx, void* p, int64_t logical_bytes) {
  if (!p) return;
  const size_t padded = padded_size(logical_bytes);
  if (padded >= (64u << 10) && ctx->block_cache_bytes + padded <= ctx->block_cache_cap && ctx->block_cache.size() < 4096) {
    ctx->block_cache.emplace(padded, p);
    ctx->block_cache_bytes += padded;
  } else {
    cudaFreeAsync(p, ctx->stream);
  }
  ctx->cur_bytes -= logical_bytes;
  ctx->total_rel += logical_bytes;
}

bg_handle mint_handle(bg_context* ctx, void* ptr, int64_t bytes, int dtype, const int64_t* shape, int rank) {
  HandleRec r;
  r.ptr = ptr;
  r.bytes = bytes;
  r.dtype = dtype;
  r.shape.assign(shape, shape + rank);
  bg_handle h = ctx->next_handle++;
  ctx->handles.emplace(h, std::move(r));
  return h;
}

// Host <-> device copies go through a pinned staging ring so that pageable caller memory still
// moves at full PCIe rate and the copy engine overlaps the host-side memcpy of the next piece.
constexpr size_t kStagePiece = 32u << 20;

static int ensure_stage(bg_context* ctx) {
  if (ctx->stage) return BG_OK;
  cudaError_t e = cudaHostAlloc(&ctx->stage, 2 * kStagePiece, cudaHostAllocDefault);
  if (e != cudaSuccess) return cuda_fail(ctx, e, "pinned staging allocation");
  ctx->stage_bytes = 2 * kStagePiece;
  return BG_OK;
}

static bool is_pinned(const void* p) {
  cudaPointerAttributes attr;
  cudaError_t e = cudaPointerGetAttributes(&attr, p);
  if (e != cudaSuccess) { cudaGetLastError(); return false; }
  return attr.type == cudaMemoryTypeHost;
}

int h2d(bg_context* ctx, void* dst, const void* src, size_t n) {
  if (n == 0) return BG_OK;
  const bool pinned = is_pinned(src);
  if (n <= (64u << 10) && !pinned) {
    cudaError_t e = cudaMemcpyAsync(dst, src, n, cudaMemcpyHostToDevice, ctx->stream);
    if (e != cudaSuccess) return cuda_fail(ctx, e, "upload copy");
    // pageable source: the runtime has staged it before returning, the caller may reuse its buffer
    return BG_OK;
  }
  if (pinned) {
    // page-locked caller memory: one DMA straight from the caller's buffer
    cudaError_t e = cudaMemcpyAsync(dst, src, n, cudaMemcpyHostToDevice, ctx->stream);
    if (e == cudaSuccess) e = cudaStreamSynchronize(ctx->stream);
    return e == cudaSuccess ? BG_OK : cuda_fail(ctx, e, "upload copy");
  }
  if (int rc = ensure_stage(ctx)) return rc;
  cudaEvent_t ev[2];
  for (auto& x : ev) cudaEventCreateWithFlags(&x, cudaEventDisableTiming);
  bool used[2] = {false, false};
  size_t off = 0;
  int i = 0;
  cudaError_t e = cudaSuccess;
  while (off < n && e == cudaSuccess) {
    size_t piece = n - off < kStagePiece ? n - off : kStagePiece;
    char* st = reinterpret_cast<char*>(ctx->stage) + (size_t)i * kStagePiece;
    if (used[i]) e = cudaEventSynchronize(ev[i]);
    if (e != cudaSuccess) break;
    memcpy(st, reinterpret_cast<const char*>(src) + off, piece);
    e = cudaMemcpyAsync(reinterpret_cast<char*>(dst) + off, st, piece, cudaMemcpyHostToDevice, ctx->stream);
    if (e == cudaSuccess) e = cudaEventRecord(ev[i], ctx->stream);
    used[i] = true;
    off += piece;
    i ^= 1;
  }
  for (int k = 0; k < 2 && e == cudaSuccess; ++k)
    if (used[k]) e = cudaEventSynchronize(ev[k]);
  for (auto& x : ev) cudaEventDestroy(x);
  if (e != cudaSuccess) return cuda_fail(ctx, e, "upload copy");
  return BG_OK;
}

int d2h(bg_context* ctx, void* dst, const void* src, size_t n) {
  if (n == 0) {
    cudaError_t e = cudaStreamSynchronize(ctx->stream);
    return e == cudaSuccess ? BG_OK : cuda_fail(ctx, e, "stream synchronize");
  }
  if (n <= (64u << 10)) {
    cudaError_t e = cudaMemcpyAsync(dst, src, n, cudaMemcpyDeviceToHost, ctx->stream);
    if (e == cudaSuccess) e = cudaStreamSynchronize(ctx->stream);
    return e == cudaSuccess ? BG_OK : cuda_fail(ctx, e, "materialize copy");
  }
  if (is_pinned(dst)) {
    cudaError_t e = cudaMemcpyAsync(dst, src, n, cudaMemcpyDeviceToHost, ctx->stream);
    if (e == cudaSuccess) e = cudaStreamSynchronize(ctx->stream);
    return e == cudaSuccess ? BG_OK : cuda_fail(ctx, e, "materialize copy");
  }
  if (int rc = ensure_stage(ctx)) return rc;
  cudaEvent_t ev[2];
  for (auto& x : ev) cudaEventCreateWithFlags(&x, cudaEventDisableTiming);
  size_t off = 0, done = 0;
  size_t piece_of[2] = {0, 0};
  int issue = 0, drain = 0;
  int in_flight = 0;
  cudaError_t e = cudaSuccess;
  while ((off < n || in_flight > 0) && e == cudaSuccess) {
    if (off < n && in_flight < 2) {
      size_t piece = n - off < kStagePiece ? n - off : kStagePiece;
      char* st = reinterpret_cast<char*>(ctx->stage) + (size_t)issue * kStagePiece;
      e = cudaMemcpyAsync(st, reinterpret_cast<const char*>(src) + off, piece, cudaMemcpyDeviceToHost, ctx->stream);
      if (e == cudaSuccess) e = cudaEventRecord(ev[issue], ctx->stream);
      piece_of[issue] = piece;
      off += piece;
      issue ^= 1;
      ++in_flight;
      continue;
    }
    e = cudaEventSynchronize(ev[drain]);
    if (e != cudaSuccess) break;
    memcpy(reinterpret_cast<char*>(dst) + done, reinterpret_cast<char*>(ctx->stage) + (size_t)drain * kStagePiece,
           piece_of[drain]);
    done += piece_of[drain];
    drain ^= 1;
    --in_flight;
  }
  for (auto& x : ev) cudaEventDestroy(x);
  if (e != cudaSuccess) return cuda_fail(ctx, e, "materialize copy");
  return BG_OK;
}

int* uniform_flag_for(bg_context* ctx, const void* ptr, bool* fresh) {
  *fresh = false;
  auto it = ctx->uniform_flags.find(ptr);
  if (it != ctx->uniform_flags.end()) return it->second;
  if (!ctx->uniform_pool) {
    if (cudaMalloc(&ctx->uniform_pool, 1024 * sizeof(int)) != cudaSuccess) { cudaGetLastError(); return nullptr; }
    for (int i = 1023; i >= 0; --i) ctx->uniform_free.push_back(i);
  }
  if (ctx->uniform_free.empty()) return nullptr;
  int* flag = ctx->uniform_pool + ctx->uniform_free.back();
  ctx->uniform_free.pop_back();
  ctx->uniform_flags[ptr] = flag;
  *fresh = true;
  return flag;
}

void uniform_flag_drop(bg_context* ctx, const void* ptr) {
  auto it = ctx->uniform_flags.find(ptr);
  if (it == ctx->uniform_flags.end()) return;
  ctx->uniform_free.push_back((int)(it->second - ctx->uniform_pool));
  ctx->uniform_flags.erase(it);
}

void* mask_classes_for(bg_context* ctx, const void* ptr, int64_t bytes, int sq, int sk, int bkv, int is_bool, bool* fresh) {
  *fresh = false;
  auto it = ctx->mask_classes.find(ptr);
  if (it != ctx->mask_classes.end()) {
    const auto& m = it->second;
    if (m.bytes == bytes && m.sq == sq && m.sk == sk && m.bkv == bkv && m.is_bool == is_bool) return m.buf;
    dev_free(ctx, m.buf, m.bytes);
    ctx->mask_classes.erase(it);
  }
  if (ctx->mask_classes.size() >= 64) return nullptr;   // callers then fall back to per-run scratch
  void* buf = nullptr;
  if (dev_alloc(ctx, bytes, &buf) != BG_OK) return nullptr;
  ctx->mask_classes[ptr] = {buf, bytes, sq, sk, bkv, is_bool};
  *fresh = true;
  return buf;
}

void mask_classes_drop(bg_context* ctx, const void* ptr) {
  auto it = ctx->mask_classes.find(ptr);
  if (it == ctx->mask_classes.end()) return;
  dev_free(ctx, it->second.buf, it->second.bytes);
  ctx->mask_classes.erase(it);
}

float* split_planes_for(bg_context* ctx, const void* ptr, int64_t n, int dtype, bool* fresh) {
  *fresh = false;
  auto it = ctx->split_planes.find(ptr);
  if (it != ctx->split_planes.end()) {
    if (it->second.n == n && it->second.dtype == dtype) return it->second.buf;
    dev_free(ctx, it->second.buf, 2 * it->second.n * 4);
    ctx->split_planes.erase(it);
  }
  if (ctx->split_planes.size() >= 4096) return nullptr;
  void* buf = nullptr;
  if (dev_alloc(ctx, 2 * n * 4, &buf) != BG_OK) return nullptr;
  ctx->split_planes[ptr] = {reinterpret_cast<float*>(buf), n, dtype};
  *fresh = true;
  return reinterpret_cast<float*>(buf);
}

void split_planes_drop(bg_context* ctx, const void* ptr) {
  auto it = ctx->split_planes.find(ptr);
  if (it == ctx->split_planes.end()) return;
  dev_free(ctx, it->second.buf, 2 * it->second.n * 4);
  ctx->split_planes.erase(it);
}

void* cast_copy_for(bg_context* ctx, const void* ptr, int64_t bytes, int dtype, bool* fresh) {
  *fresh = false;
  auto it = ctx->cast_copies.find(ptr);
  if (it != ctx->cast_copies.end()) {
    if (it->second.bytes == bytes && it->second.dtype == dtype) return it->second.buf;
    dev_free(ctx, it->second.buf, it->second.bytes);
    ctx->cast_copies.erase(it);
  }
  if (ctx->cast_copies.size() >= 4096) return nullptr;
  void* buf = nullptr;
  if (dev_alloc(ctx, bytes, &buf) != BG_OK) return nullptr;
  ctx->cast_copies[ptr] = {buf, bytes, dtype};
  *fresh = true;
  return buf;
}

void cast_copy_drop(bg_context* ctx, const void* ptr) {
  auto it = ctx->cast_copies.find(ptr);
  if (it == ctx->cast_copies.end()) return;
  dev_free(ctx, it->second.buf, it->second.bytes);
  ctx->cast_copies.erase(it);
}

static int64_t numel_of(const int64_t* shape, int rank) {
  int64_t n = 1;
  for (int i = 0; i < rank; ++i) n *= shape[i];
  return n;
}

}  // namespace bg

using namespace bg;

extern "C" {

int bg_abi_version(void) { return BG_ABI_VERSION; }

int bg_create(int device_ordinal, bg_context** out) {
  if (!out) return BG_ERR_INVALID;
  *out = nullptr;
  int n = 0;
  cudaError_t e = cudaGetDeviceCount(&n);
  if (e != cudaSuccess || n == 0) {
    cudaGetLastError();
    return BG_ERR_CUDA;  // no CUDA device: the bridge has no CPU fallback
  }
  if (device_ordinal < 0 || device_ordinal >= n) return BG_ERR_INVALID;
  if (cudaSetDevice(device_ordinal) != cudaSuccess) return BG_ERR_CUDA;
  cudaDeviceProp prop;
  if (cudaGetDeviceProperties(&prop, device_ordinal) != cudaSuccess) return BG_ERR_CUDA;
  if (prop.major != 10) return BG_ERR_UNSUPPORTED;  // kernels are built for sm_100a only
  bg_context* ctx = new bg_context();
  ctx->device = device_ordinal;
  ctx->sm_count = prop.multiProcessorCount;
  if (cudaStreamCreateWithFlags(&ctx->stream, cudaStreamNonBlocking) != cudaSuccess) {
    delete ctx;
    return BG_ERR_CUDA;
  }
  // keep freed blocks in the pool: intermediates of the next plan reuse them without a driver call
  cudaMemPool_t pool;
  if (cudaDeviceGetDefaultMemPool(&pool, device_ordinal) == cudaSuccess) {
    uint64_t thr = UINT64_MAX;
    cudaMemPoolSetAttribute(pool, cudaMemPoolAttrReleaseThreshold, &thr);
  }
  if (cudaMalloc(&ctx->d_status, 256) != cudaSuccess || cudaHostAlloc(&ctx->h_status, 256, cudaHostAllocDefault) != cudaSuccess) {
    delete ctx;
    return BG_ERR_CUDA;
  }
  cudaMemsetAsync(ctx->d_status, 0, 256, ctx->stream);
  if (cudaMalloc(&ctx->gemm_counters, 1024 * sizeof(int)) != cudaSuccess) {
    cudaFree(ctx->d_status);
    cudaFreeHost(ctx->h_status);
    delete ctx;
    return BG_ERR_CUDA;
  }
  cudaMemsetAsync(ctx->gemm_counters, 0, 1024 * sizeof(int), ctx->stream);
  *out = ctx;
  return BG_OK;
}

int bg_destroy(bg_context* ctx) {
  if (!ctx) return BG_OK;
  cudaSetDevice(ctx->device);
  cudaStreamSynchronize(ctx->stream);
  for (auto& kv : ctx->handles) cudaFreeAsync(kv.second.ptr, ctx->stream);
  ctx->handles.clear();
  flush_block_cache(ctx);
  for (auto& kv : ctx->mask_classes) cudaFreeAsync(kv.second.buf, ctx->stream);
  ctx->mask_classes.clear();
  for (auto& kv : ctx->split_planes) cudaFreeAsync(kv.second.buf, ctx->stream);
  ctx->split_planes.clear();
  for (auto& kv : ctx->cast_copies) cudaFreeAsync(kv.second.buf, ctx->stream);
  ctx->cast_copies.clear();
  ctx->plan_cache.clear();
  for (auto& pe : ctx->pending_events) {
    cudaEventDestroy(pe.second.first);
    cudaEventDestroy(pe.second.second);
  }
  cudaStreamSynchronize(ctx->stream);
  if (ctx->uniform_pool) cudaFree(ctx->uniform_pool);
  if (ctx->d_status) cudaFree(ctx->d_status);
  if (ctx->gemm_counters) cudaFree(ctx->gemm_counters);
  if (ctx->h_status) cudaFreeHost(ctx->h_status);
  if (ctx->stage) cudaFreeHost(ctx->stage);
  cudaStreamDestroy(ctx->stream);
  delete ctx;
  return BG_OK;
}

const char* bg_last_error(bg_context* ctx) { return ctx ? ctx->err.c_str() : "CUDA bridge: null context"; }

int bg_set_option(bg_context* ctx, const char* key, int64_t value) {
  if (!ctx || !key) return BG_ERR_INVALID;
  std::string k(key);
  if (k == "profiling") ctx->profiling = value != 0;
  else if (k == "f64_contraction") ctx->f64_mode = (int)value;
  else if (k == "fusion") { ctx->fusion = value != 0; ctx->plan_cache.clear(); }
  else if (k == "tensor_cores") { ctx->tensor_cores = value != 0; ctx->plan_cache.clear(); }
  else if (k == "gemm_cta_pairs") g_tc_pair_mode = (int)value;   // process-wide: a launch policy, not plan state
  else if (k == "gemm_pair_tile_width") {
    if (value != 0 && value != 256 && value != 192 && value != 128) return fail(ctx, BG_ERR_INVALID, "set_option: gemm_pair_tile_width is 0, 256, 192 or 128");
    g_tc_pair_width = (int)value;
  }
  else if (k == "dependent_launch") g_dependent_launch = value != 0;   // process-wide: a launch policy, not plan state
  else if (k == "attention16_kernel") {
    if (value < -1 || value > 15) return fail(ctx, BG_ERR_INVALID, "set_option: attention16_kernel is a bit set in 0..15, or -1 for the default");
    g_attn16_variant = value < 0 ? kAttn16DefaultVariant : (int)value;     // process-wide: a launch policy, not plan state
  }
  else if (k == "attention32_kernel") {
    if (value < -1 || value > 3 || value == 2) return fail(ctx, BG_ERR_INVALID, "set_option: attention32_kernel is 0, 1, 3, or -1 for the default");
    g_attn32_variant = value < 0 ? kAttn32DefaultVariant : (int)value;
  }
  else if (k == "fail_allocation_after") {
    if (value < 0) return fail(ctx, BG_ERR_INVALID, "set_option: fail_allocation_after takes a count (0 = off)");
    ctx->fail_alloc_countdown = value;
  }
  else if (k == "static_patterns") { ctx->static_patterns = value != 0; ctx->plan_cache.clear(); }
  else if (k == "gemm_groups") { ctx->gemm_groups = value != 0; ctx->plan_cache.clear(); }
  else return fail(ctx, BG_ERR_INVALID, "set_option: unknown option '" + k + "'");
  if (k == "f64_contraction") ctx->plan_cache.clear();
  return BG_OK;
}

int bg_upload(bg_context* ctx, const void* data, size_t nbytes, const int64_t* shape, int rank, int dtype,
              bg_handle* out) {
  if (!ctx || !out) return BG_ERR_INVALID;
  if (rank < 0 || rank > BG_MAX_RANK || (rank > 0 && !shape)) return fail(ctx, BG_ERR_INVALID, "upload: bad rank");
  const int es = dtype_size(dtype);
  if (es == 0) return fail(ctx, BG_ERR_INVALID, "upload: unknown dtype");
  for (int i = 0; i < rank; ++i)
    if (shape[i] < 0) return fail(ctx, BG_ERR_INVALID, "upload: negative extent");
  const int64_t bytes = numel_of(shape, rank) * es;
  if ((int64_t)nbytes != bytes)
    return fail(ctx, BG_ERR_INVALID, "upload: byte length " + std::to_string(nbytes) + " does not match shape x " +
                                         dtype_name(dtype) + " = " + std::to_string(bytes));
  if (bytes > 0 && !data) return fail(ctx, BG_ERR_INVALID, "upload: null data");
  cudaSetDevice(ctx->device);
  void* p = nullptr;
  if (int rc = dev_alloc(ctx, bytes, &p)) return rc;
  if (int rc = h2d(ctx, p, data, (size_t)bytes)) {
    dev_free(ctx, p, bytes);
    return rc;
  }
  *out = mint_handle(ctx, p, bytes, dtype, shape, rank);
  return BG_OK;
}

int bg_selftest_wait_timeout(bg_context* ctx, int64_t limit_cycles) {
  if (!ctx) return BG_ERR_INVALID;
  if (limit_cycles < 1000 || limit_cycles > 2000000000ll) return fail(ctx, BG_ERR_INVALID, "selftest_wait_timeout: limit outside [1e3, 2e9] cycles");
  cudaSetDevice(ctx->device);
  cudaError_t e = launch_wait_timeout_selftest(limit_cycles, ctx->d_status, ctx->stream);
  if (e == cudaSuccess) e = cudaMemcpyAsync(ctx->h_status, ctx->d_status, sizeof(int), cudaMemcpyDeviceToHost, ctx->stream);
  if (e == cudaSuccess) e = cudaStreamSynchronize(ctx->stream);
  if (e != cudaSuccess) return cuda_fail(ctx, e, "selftest_wait_timeout");
  const int st = take_device_status(ctx);
  if (st != 0) return fail(ctx, st, device_status_message(st));
  return BG_OK;
}

int bg_alloc(bg_context* ctx, const int64_t* shape, int rank, int dtype, bg_handle* out) {
  if (!ctx || !out) return BG_ERR_INVALID;
  if (rank < 0 || rank > BG_MAX_RANK || (rank > 0 && !shape)) return fail(ctx, BG_ERR_INVALID, "alloc: bad rank");
  const int es = dtype_size(dtype);
  if (es == 0) return fail(ctx, BG_ERR_INVALID, "alloc: unknown dtype");
  for (int i = 0; i < rank; ++i)
    if (shape[i] < 0) return fail(ctx, BG_ERR_INVALID, "alloc: negative extent");
  const int64_t bytes = numel_of(shape, rank) * es;
  cudaSetDevice(ctx->device);
  void* p = nullptr;
  if (int rc = dev_alloc(ctx, bytes, &p)) return rc;
  *out = mint_handle(ctx, p, bytes, dtype, shape, rank);
  return BG_OK;
}

int bg_materialize(bg_context* ctx, bg_handle h, void* out, size_t nbytes) {
  if (!ctx) return BG_ERR_INVALID;
  auto it = ctx->handles.find(h);
  if (it == ctx->handles.end()) return fail(ctx, BG_ERR_UNKNOWN_HANDLE, "materialize: unknown handle " + std::to_string(h));
  if ((int64_t)nbytes != it->second.bytes)
    return fail(ctx, BG_ERR_INVALID, "materialize: byte length " + std::to_string(nbytes) + " does not match the buffer's " +
                                         std::to_string(it->second.bytes));
  if (nbytes > 0 && !out) return fail(ctx, BG_ERR_INVALID, "materialize: null destination");
  cudaSetDevice(ctx->device);
  const int rc = d2h(ctx, out, it->second.ptr, nbytes);
  if (rc == BG_OK && ctx->status_pending) {
    // d2h synchronised the stream: the status copy behind the producing plan has landed
    const int st = take_device_status(ctx);
    if (st != 0) return fail(ctx, st, device_status_message(st) + " (in the plan that produced this buffer or an earlier one)");
  }
  return rc;
}

int bg_release(bg_context* ctx, bg_handle h) {
  if (!ctx) return BG_ERR_INVALID;
  auto it = ctx->handles.find(h);
  if (it == ctx->handles.end()) return BG_OK;  // idempotent, unknown handle is a no-op
  cudaSetDevice(ctx->device);
  uniform_flag_drop(ctx, it->second.ptr);
  mask_classes_drop(ctx, it->second.ptr);
  split_planes_drop(ctx, it->second.ptr);
  cast_copy_drop(ctx, it->second.ptr);
  dev_free(ctx, it->second.ptr, it->second.bytes);
  ctx->handles.erase(it);
  return BG_OK;
}

int bg_handle_nbytes(bg_context* ctx, bg_handle h, int64_t* out) {
  if (!ctx || !out) return BG_ERR_INVALID;
  auto it = ctx->handles.find(h);
  if (it == ctx->handles.end()) return fail(ctx, BG_ERR_UNKNOWN_HANDLE, "unknown handle " + std::to_string(h));
  *out = it->second.bytes;
  return BG_OK;
}

int bg_device_pointer(bg_context* ctx, bg_handle h, void** out) {
  if (!ctx || !out) return BG_ERR_INVALID;
  auto it = ctx->handles.find(h);
  if (it == ctx->handles.end()) return fail(ctx, BG_ERR_UNKNOWN_HANDLE, "unknown handle " + std::to_string(h));
  *out = it->second.ptr;
  return BG_OK;
}

void* bg_stream(bg_context* ctx) { return ctx ? (void*)ctx->stream : nullptr; }

int bg_alive_handle_count(bg_context* ctx, int64_t* out) {
  if (!ctx || !out) return BG_ERR_INVALID;
  *out = (int64_t)ctx->handles.size();
  return BG_OK;
}

int bg_resource_snapshot(bg_context* ctx, bg_resource_stats* out) {
  if (!ctx || !out) return BG_ERR_INVALID;
  out->current_bytes = ctx->cur_bytes;
  out->peak_bytes = ctx->peak_bytes;
  out->total_allocated_bytes = ctx->total_alloc;
  out->total_released_bytes = ctx->total_rel;
  out->alive_handles = (int64_t)ctx->handles.size();
  out->logical_tensor_plan_peak_bytes = ctx->plan_peak;
  out->kernel_launches = ctx->launches;
  out->plan_cache_hits = ctx->cache_hits;
  out->plan_cache_misses = ctx->cache_misses;
  return BG_OK;
}

int bg_flush_profiles(bg_context* ctx, bg_profile_entry* out, int capacity, int* n_out) {
  if (!ctx || !n_out) return BG_ERR_INVALID;
  cudaSetDevice(ctx->device);
  cudaError_t e = cudaStreamSynchronize(ctx->stream);
  if (e != cudaSuccess) return cuda_fail(ctx, e, "flush_profiles synchronize");
  if (ctx->status_pending) {
    const int st = take_device_status(ctx);
    if (st != 0) return fail(ctx, st, device_status_message(st) + " (in an earlier plan)");
  }
  for (auto& pe : ctx->pending_events) {
    float ms = 0.f;
    if (cudaEventElapsedTime(&ms, pe.second.first, pe.second.second) == cudaSuccess) {
      auto& acc = ctx->profile[pe.first];
      acc.ms += ms;
      acc.launches += 1;
    }
    cudaEventDestroy(pe.second.first);
    cudaEventDestroy(pe.second.second);
  }
  ctx->pending_events.clear();
  int n = 0;
  for (auto& kv : ctx->profile) {
    if (out && n < capacity) {
      memset(&out[n], 0, sizeof(bg_profile_entry));
      strncpy(out[n].name, kv.first.c_str(), sizeof(out[n].name) - 1);
      out[n].ms = (float)kv.second.ms;
      out[n].launches = kv.second.launches;
    }
    ++n;
  }
  *n_out = n;
  if (out) ctx->profile.clear();
  return BG_OK;
}

int bg_last_plan_trace(bg_context* ctx, char* out, size_t capacity) {
  if (!ctx || !out || capacity == 0) return BG_ERR_INVALID;
  strncpy(out, ctx->last_trace.c_str(), capacity - 1);
  out[capacity - 1] = 0;
  return BG_OK;
}

// ---- per-op methods, each as a small plan ---------------------------------------------

static void init_step(bg_plan_step& s, int op, int dtype, const int64_t* shape, int rank) {
  memset(&s, 0, sizeof(s));
  s.op = op;
  s.dtype = dtype;
  s.rank = rank;
  for (int i = 0; i < rank; ++i) s.shape[i] = shape[i];
}

static int check_handle(bg_context* ctx, bg_handle h, int64_t want_bytes, const char* what) {
  auto it = ctx->handles.find(h);
  if (it == ctx->handles.end())
    return fail(ctx, BG_ERR_UNKNOWN_HANDLE, std::string(what) + ": unknown handle " + std::to_string(h));
  if (want_bytes >= 0 && it->second.bytes != want_bytes)
    return fail(ctx, BG_ERR_INVALID, std::string(what) + ": buffer holds " + std::to_string(it->second.bytes) +
                                         " bytes, the call implies " + std::to_string(want_bytes));
  return BG_OK;
}

int bg_matmul(bg_context* ctx, bg_handle a, bg_handle b, int64_t m, int64_t k, int64_t n, int dtype, bg_handle* out) {
  if (!ctx || !out) return BG_ERR_INVALID;
  if (m < 0 || k < 0 || n < 0) return fail(ctx, BG_ERR_INVALID, "matmul: negative dimension");
  const int es = dtype_size(dtype);
  if (!es) return fail(ctx, BG_ERR_INVALID, "matmul: unknown dtype");
  if (int rc = check_handle(ctx, a, m * k * es, "matmul lhs")) return rc;
  if (int rc = check_handle(ctx, b, k * n * es, "matmul rhs")) return rc;
  bg_plan_step st[3];
  int64_t sa[2] = {m, k}, sb[2] = {k, n}, sc[2] = {m, n};
  init_step(st[0], BG_OP_BUFFER, dtype, sa, 2);
  init_step(st[1], BG_OP_BUFFER, dtype, sb, 2);
  init_step(st[2], BG_OP_MATMUL, dtype, sc, 2);
  st[2].n_inputs = 2;
  st[2].input_ids[0] = 0;
  st[2].input_ids[1] = 1;
  bg_plan plan{st, 3, 2, nullptr, 0};
  bg_plan_input in[2] = {{0, 0, a, nullptr, 0}, {1, 0, b, nullptr, 0}};
  return run_plan(ctx, &plan, in, 2, nullptr, 0, out);
}

int bg_fused_elementwise(bg_context* ctx, const bg_handle* inputs, int n_inputs, const int32_t* op_triples, int n_ops,
                         const int64_t* shape, int rank, int dtype, bg_handle* out) {
  if (!ctx || !out) return BG_ERR_INVALID;
  // same limits as the reference kernel (fused_elementwise.ts:97-110)
  if (n_inputs < 1 || n_inputs > 8) return fail(ctx, BG_ERR_INVALID, "fused_elementwise: 1..8 inputs required");
  if (n_ops < 1 || n_ops > 32) return fail(ctx, BG_ERR_INVALID, "fused_elementwise: 1..32 ops required");
  if (rank < 0 || rank > BG_MAX_RANK) return fail(ctx, BG_ERR_INVALID, "fused_elementwise: bad rank");
  const int es = dtype_size(dtype);
  if (!es) return fail(ctx, BG_ERR_INVALID, "fused_elementwise: unknown dtype");
  const int64_t bytes = numel_of(shape, rank) * es;
  std::vector<bg_plan_step> st(n_inputs + 1);
  std::vector<bg_plan_input> in(n_inputs);
  for (int i = 0; i < n_inputs; ++i) {
    if (int rc = check_handle(ctx, inputs[i], bytes, "fused_elementwise input")) return rc;
    init_step(st[i], BG_OP_BUFFER, dtype, shape, rank);
    in[i] = {i, 0, inputs[i], nullptr, 0};
  }
  bg_plan_step& f = st[n_inputs];
  init_step(f, BG_OP_FUSED_ELEMENTWISE, dtype, shape, rank);
  f.n_inputs = n_inputs;
  for (int i = 0; i < n_inputs; ++i) f.input_ids[i] = i;
  f.ext_offset = 0;
  f.ext_count = n_ops;
  bg_plan plan{st.data(), n_inputs + 1, n_inputs, op_triples, 3 * n_ops};
  return run_plan(ctx, &plan, in.data(), n_inputs, nullptr, 0, out);
}

int bg_cast(bg_context* ctx, bg_handle h, int src_dtype, int dst_dtype, const int64_t* shape, int rank, bg_handle* out) {
  if (!ctx || !out) return BG_ERR_INVALID;
  if (rank < 0 || rank > BG_MAX_RANK) return fail(ctx, BG_ERR_INVALID, "cast: bad rank");
  if (!dtype_size(src_dtype) || !dtype_size(dst_dtype)) return fail(ctx, BG_ERR_INVALID, "cast: unknown dtype");
  if (int rc = check_handle(ctx, h, numel_of(shape, rank) * dtype_size(src_dtype), "cast")) return rc;
  bg_plan_step st[2];
  init_step(st[0], BG_OP_BUFFER, src_dtype, shape, rank);
  init_step(st[1], BG_OP_CAST, dst_dtype, shape, rank);
  st[1].n_inputs = 1;
  st[1].input_ids[0] = 0;
  bg_plan plan{st, 2, 1, nullptr, 0};
  bg_plan_input in[1] = {{0, 0, h, nullptr, 0}};
  return run_plan(ctx, &plan, in, 1, nullptr, 0, out);
}

int bg_flash_attention(bg_context* ctx, bg_handle q, bg_handle k, bg_handle v, bg_handle mask, const int64_t* mask_shape,
                       int64_t b, int64_t h, int64_t sq, int64_t sk, int64_t d, double scale, int dtype,
                       bg_handle* out) {
  if (!ctx || !out) return BG_ERR_INVALID;
  const int es = dtype_size(dtype);
  if (!es) return fail(ctx, BG_ERR_INVALID, "flash_attention: unknown dtype");
  if (int rc = check_handle(ctx, q, b * h * sq * d * es, "flash_attention q")) return rc;
  if (int rc = check_handle(ctx, k, b * h * sk * d * es, "flash_attention k")) return rc;
  if (int rc = check_handle(ctx, v, b * h * sk * d * es, "flash_attention v")) return rc;
  // q, k, v, [mask] -> PERMUTE(k) -> MATMUL -> MUL(scale) -> [ADD mask] -> FUSED_SOFTMAX -> MATMUL.
  // The plan compiler recognises this shape of graph and runs the fused attention kernel.
  std::vector<bg_plan_step> st;
  std::vector<bg_plan_input> in;
  int64_t sqd[4] = {b, h, sq, d}, skd[4] = {b, h, sk, d}, sdk[4] = {b, h, d, sk}, sss[4] = {b, h, sq, sk};
  bg_plan_step s;
  init_step(s, BG_OP_BUFFER, dtype, sqd, 4); st.push_back(s); in.push_back({0, 0, q, nullptr, 0});
  init_step(s, BG_OP_BUFFER, dtype, skd, 4); st.push_back(s); in.push_back({1, 0, k, nullptr, 0});
  init_step(s, BG_OP_BUFFER, dtype, skd, 4); st.push_back(s); in.push_back({2, 0, v, nullptr, 0});
  int mask_id = -1;
  if (mask != 0) {
    if (!mask_shape) return fail(ctx, BG_ERR_INVALID, "flash_attention: mask shape required");
    if ((mask_shape[0] != 1 && mask_shape[0] != b) || (mask_shape[1] != 1 && mask_shape[1] != h) ||
        mask_shape[2] != sq || mask_shape[3] != sk)
      return fail(ctx, BG_ERR_INVALID, "flash_attention: mask must be [B|1, H|1, Sq, Sk]");
    if (int rc = check_handle(ctx, mask, numel_of(mask_shape, 4) * es, "flash_attention mask")) return rc;
    init_step(s, BG_OP_BUFFER, dtype, mask_shape, 4);
    mask_id = (int)st.size();
    st.push_back(s);
    in.push_back({mask_id, 0, mask, nullptr, 0});
  }
  init_step(s, BG_OP_PERMUTE, dtype, sdk, 4);
  s.n_inputs = 1; s.input_ids[0] = 1; s.iarg[0] = 0; s.iarg[1] = 1; s.iarg[2] = 3; s.iarg[3] = 2;
  const int kt = (int)st.size(); st.push_back(s);
  init_step(s, BG_OP_MATMUL, dtype, sss, 4);
  s.n_inputs = 2; s.input_ids[0] = 0; s.input_ids[1] = kt;
  const int qk = (int)st.size(); st.push_back(s);
  init_step(s, BG_OP_CONST, dtype, nullptr, 0);
  s.farg[0] = (double)(float)scale;
  const int sc = (int)st.size(); st.push_back(s);
  init_step(s, BG_OP_MUL, dtype, sss, 4);
  s.n_inputs = 2; s.input_ids[0] = qk; s.input_ids[1] = sc;
  int cur = (int)st.size(); st.push_back(s);
  if (mask_id >= 0) {
    init_step(s, BG_OP_ADD, dtype, sss, 4);
    s.n_inputs = 2; s.input_ids[0] = cur; s.input_ids[1] = mask_id;
    cur = (int)st.size(); st.push_back(s);
  }
  init_step(s, BG_OP_FUSED_SOFTMAX, dtype, sss, 4);
  s.n_inputs = 1; s.input_ids[0] = cur; s.iarg[0] = 3;
  cur = (int)st.size(); st.push_back(s);
  init_step(s, BG_OP_MATMUL, dtype, sqd, 4);
  s.n_inputs = 2; s.input_ids[0] = cur; s.input_ids[1] = 2;
  cur = (int)st.size(); st.push_back(s);
  bg_plan plan{st.data(), (int)st.size(), cur, nullptr, 0};
  return run_plan(ctx, &plan, in.data(), (int)in.size(), nullptr, 0, out);
}

int bg_run_tensor_plan(bg_context* ctx, const bg_plan* plan, const bg_plan_input* inputs, int n_inputs, void* out_host,
                       size_t out_nbytes) {
  if (!ctx || !plan) return BG_ERR_INVALID;
  if (!out_host && out_nbytes > 0) return fail(ctx, BG_ERR_INVALID, "run_tensor_plan: null destination");
  static char empty;
  return run_plan(ctx, plan, inputs, n_inputs, out_host ? out_host : &empty, out_nbytes, nullptr);
}

int bg_run_tensor_plan_resident(bg_context* ctx, const bg_plan* plan, const bg_plan_input* inputs, int n_inputs,
                                bg_handle* out) {
  if (!ctx || !plan || !out) return BG_ERR_INVALID;
  return run_plan(ctx, plan, inputs, n_inputs, nullptr, 0, out);
}

}  // extern "C"

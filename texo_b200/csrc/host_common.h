// Host-side state shared by the three operators: a per-device context holding the
// grow-only scratch buffer, the device status word and cached device attributes, and the
// driver entry point used to encode TMA tensor maps.
//
// Contract inherited from the reference operators (src/mm_int8.cu:500-509, docs/operators.md
// :9-12 of frezcirno/Texo): work is issued on the legacy default stream of the current
// device, asynchronously, and the scratch is callee-owned, process-static and never freed.
// Unlike the reference, the state is kept per device, so one process may drive several GPUs
// (one after another; calls are still not thread-safe).
#pragma once
#include <cstddef>
#include <cstdint>
#include <cstdio>
#include <cuda.h>
#include <cuda_runtime.h>

namespace texo {

constexpr int MAX_DEVICES = 64;

struct DeviceCtx {
  bool ready = false;
  int device = -1;
  int sm_count = 0;
  int cc_major = 0;
  void* scratch = nullptr;
  size_t scratch_bytes = 0;
  int* status = nullptr;  // 64 ints of device memory; word 0 = first error code
  // Second scratch: split-K workspace of the skinny path.  It is all zero between calls
  // (the kernel that consumes it cleans up after itself); zeroed when (re)allocated.
  void* workspace = nullptr;
  size_t workspace_bytes = 0;
  // Epoch number of the last CTA-pair call (INT8 or W4A8): its epilogues mark finished sum items
  // in the flag array with it (flags are compared, not cleared per call; see next_sums_epoch).
  unsigned sums_epoch = 0;
  void* item_flags = nullptr;  // used by nothing else, so that no other data can pass for an epoch
  size_t item_flag_bytes = 0;
};

inline int& host_status() {
  static int value = 0;
  return value;
}

inline void note_host_error(int code) {
  if (host_status() == 0) host_status() = code;
}

inline DeviceCtx& device_ctx() {
  static DeviceCtx table[MAX_DEVICES];
  int device = 0;
  cudaGetDevice(&device);
  if (device < 0 || device >= MAX_DEVICES) device = 0;
  DeviceCtx& ctx = table[device];
  if (!ctx.ready) {
    ctx.device = device;
    cudaDeviceGetAttribute(&ctx.sm_count, cudaDevAttrMultiProcessorCount, device);
    cudaDeviceGetAttribute(&ctx.cc_major, cudaDevAttrComputeCapabilityMajor, device);
    if (cudaMalloc(&ctx.status, 64 * sizeof(int)) == cudaSuccess)
      cudaMemset(ctx.status, 0, 64 * sizeof(int));
    ctx.ready = true;
  }
  return ctx;
}

// Grow-only scratch (first call / growth allocates; steady state does not).
inline void* device_scratch(DeviceCtx& ctx, size_t bytes) {
  if (bytes > ctx.scratch_bytes) {
    if (ctx.scratch) cudaFree(ctx.scratch);
    ctx.scratch = nullptr;
    ctx.scratch_bytes = 0;
    // Round up so that slowly growing shapes do not reallocate on every call.
    size_t want = (bytes + (size_t(1) << 20) - 1) & ~((size_t(1) << 20) - 1);
    if (cudaMalloc(&ctx.scratch, want) != cudaSuccess) {
      cudaGetLastError();
      std::fprintf(stderr, "texo_b200: scratch allocation of %zu bytes failed\n", want);
      return nullptr;
    }
    ctx.scratch_bytes = want;
  }
  return ctx.scratch;
}

// Grow-only, zero-initialised flag array of the INT8 CTA-pair kernel (see DeviceCtx::sums_epoch).
inline unsigned* device_item_flags(DeviceCtx& ctx, size_t bytes) {
  if (bytes > ctx.item_flag_bytes) {
    if (ctx.item_flags) cudaFree(ctx.item_flags);
    ctx.item_flags = nullptr;
    ctx.item_flag_bytes = 0;
    const size_t want = (bytes + 4095) & ~size_t(4095);
    if (cudaMalloc(&ctx.item_flags, want) != cudaSuccess) {
      cudaGetLastError();
      std::fprintf(stderr, "texo_b200: flag allocation of %zu bytes failed\n", want);
      return nullptr;
    }
    cudaMemsetAsync(ctx.item_flags, 0, want, 0);
    ctx.item_flag_bytes = want;
  }
  return static_cast<unsigned*>(ctx.item_flags);
}

// The epoch number of the next call that publishes sums through the flag array: never zero,
// and when the 32-bit counter wraps the flags are cleared (on the stream, ahead of the kernel)
// so that a flag left behind 2^32 calls ago cannot pass for a fresh one.
inline unsigned next_sums_epoch(DeviceCtx& ctx) {
  if (++ctx.sums_epoch == 0) {
    if (ctx.item_flags) cudaMemsetAsync(ctx.item_flags, 0, ctx.item_flag_bytes, 0);
    ctx.sums_epoch = 1;
  }
  return ctx.sums_epoch;
}

// Grow-only, zero-initialised workspace (see DeviceCtx::workspace).
inline void* device_workspace(DeviceCtx& ctx, size_t bytes) {
  if (bytes > ctx.workspace_bytes) {
    if (ctx.workspace) cudaFree(ctx.workspace);
    ctx.workspace = nullptr;
    ctx.workspace_bytes = 0;
    size_t want = (bytes + (size_t(1) << 20) - 1) & ~((size_t(1) << 20) - 1);
    if (cudaMalloc(&ctx.workspace, want) != cudaSuccess) {
      cudaGetLastError();
      std::fprintf(stderr, "texo_b200: workspace allocation of %zu bytes failed\n", want);
      return nullptr;
    }
    cudaMemsetAsync(ctx.workspace, 0, want, 0);
    ctx.workspace_bytes = want;
  }
  return ctx.workspace;
}

// Reads and clears the status: device word (blocking copy) or, if that is clean, the last
// host-side error.  0 = no error.  Codes are listed in ptx.cuh.
inline int read_and_clear_status() {
  DeviceCtx& ctx = device_ctx();
  int code = 0;
  if (ctx.status) {
    cudaMemcpy(&code, ctx.status, sizeof(int), cudaMemcpyDeviceToHost);
    if (code != 0) {
      cudaMemset(ctx.status, 0, sizeof(int));
      // a kernel that gave up may have left partial sums behind
      if (ctx.workspace) cudaMemset(ctx.workspace, 0, ctx.workspace_bytes);
    }
  }
  if (code == 0) code = host_status();
  host_status() = 0;
  return code;
}

// Launch on the legacy default stream with programmatic stream serialisation: the grid may be
// scheduled while the grid ahead of it drains (its CTAs take SMs as they become free and run
// up to their grid_dependency_wait, ptx.cuh).  Only for kernels that execute that wait before
// touching global memory.
template <typename... Params, typename... Args>
inline cudaError_t launch_overlapping_predecessor(void (*kernel)(Params...), dim3 grid, dim3 block,
                                                  size_t smem_bytes, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem_bytes;
  cfg.stream = 0;
  cudaLaunchAttribute attr;
  attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr.val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = &attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kernel, Params(args)...);
}

// ------------------------------------------------------------ instrumentation
// Cumulative number of kernels this library has launched (all devices).
inline long long& launch_counter() {
  static long long count = 0;
  return count;
}

// Optional CUDA-event bracket around the dominant kernel of each call, for roofline
// reporting: while enabled, up to PROFILE_SLOTS launches are bracketed on the launching
// stream; reading sums the elapsed times (and synchronises).
constexpr int PROFILE_SLOTS = 4096;
struct KernelProfile {
  bool enabled = false;
  int used = 0;
  int created = 0;
  cudaEvent_t start[PROFILE_SLOTS];
  cudaEvent_t stop[PROFILE_SLOTS];
};
inline KernelProfile& kernel_profile() {
  static KernelProfile profile;
  return profile;
}
// Returns the slot to pass to profile_stop, or -1 when not profiling.
inline int profile_start(cudaStream_t stream = 0) {
  KernelProfile& p = kernel_profile();
  if (!p.enabled || p.used >= PROFILE_SLOTS) return -1;
  if (p.used >= p.created) {
    if (cudaEventCreate(&p.start[p.created]) != cudaSuccess ||
        cudaEventCreate(&p.stop[p.created]) != cudaSuccess) {
      cudaGetLastError();
      return -1;
    }
    ++p.created;
  }
  cudaEventRecord(p.start[p.used], stream);
  return p.used++;
}
inline void profile_stop(int slot, cudaStream_t stream = 0) {
  if (slot >= 0) cudaEventRecord(kernel_profile().stop[slot], stream);
}

using TensorMapEncodeFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                       const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                       const cuuint32_t*, CUtensorMapInterleave,
                                       CUtensorMapSwizzle, CUtensorMapL2promotion,
                                       CUtensorMapFloatOOBfill);

inline TensorMapEncodeFn tensor_map_encoder() {
  static TensorMapEncodeFn fn = nullptr;
  static bool tried = false;
  if (!tried) {
    tried = true;
    void* entry = nullptr;
    cudaDriverEntryPointQueryResult result;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &entry, cudaEnableDefault, &result) ==
            cudaSuccess &&
        result == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<TensorMapEncodeFn>(entry);
    else
      cudaGetLastError();
  }
  return fn;
}

// Row-major 2-D tensor [rows, cols] of `elem_bytes` elements; box = box_rows x box_cols.
// Out-of-range parts of a box read as zero.  Returns false if the driver rejects it (base
// not 16-byte aligned, row pitch not a multiple of 16 bytes, ...).
//
// A descriptor is a pure function of these arguments (it holds an address and a shape, not
// data), and inference calls repeat the same handful of (pointer, shape) combinations, so the
// encoded maps are kept in a small per-process cache: a hit replaces the driver call (a
// microsecond or two of host time, a noticeable share of a launch-bound call) by a compare.
// The reference keeps its per-process state the same way (its src/mm_int8.cu:511-527).
struct TensorMapKey {
  const void* base;
  uint64_t rows, cols, pitch;
  uint32_t box_rows, box_cols;
  int type, swizzle;
  bool operator==(const TensorMapKey& o) const {
    return base == o.base && rows == o.rows && cols == o.cols && pitch == o.pitch &&
           box_rows == o.box_rows && box_cols == o.box_cols && type == o.type && swizzle == o.swizzle;
  }
};
constexpr int TENSOR_MAP_CACHE_SLOTS = 32;
struct TensorMapCache {
  TensorMapKey key[TENSOR_MAP_CACHE_SLOTS];
  CUtensorMap map[TENSOR_MAP_CACHE_SLOTS];
  int used = 0, next = 0;
  long long hits = 0, misses = 0;
};
inline TensorMapCache& tensor_map_cache() {
  static TensorMapCache cache;
  return cache;
}

inline bool make_tensor_map_2d(CUtensorMap* map, CUtensorMapDataType type, size_t elem_bytes,
                               const void* base, uint64_t rows, uint64_t cols,
                               uint64_t row_pitch_bytes, uint32_t box_rows, uint32_t box_cols,
                               CUtensorMapSwizzle swizzle) {
  TensorMapCache& cache = tensor_map_cache();
  const TensorMapKey key = {base, rows, cols, row_pitch_bytes, box_rows, box_cols, int(type), int(swizzle)};
  for (int i = 0; i < cache.used; ++i) {
    if (cache.key[i] == key) {
      *map = cache.map[i];
      ++cache.hits;
      return true;
    }
  }
  TensorMapEncodeFn encode = tensor_map_encoder();
  if (!encode) return false;
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {row_pitch_bytes};
  cuuint32_t box[2] = {box_cols, box_rows};
  cuuint32_t elem_strides[2] = {1, 1};
  (void)elem_bytes;
  if (encode(map, type, 2, const_cast<void*>(base), dims, strides, box, elem_strides,
             CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
             CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
    return false;
  ++cache.misses;
  const int slot = cache.used < TENSOR_MAP_CACHE_SLOTS ? cache.used++ : cache.next;
  cache.next = (slot + 1) % TENSOR_MAP_CACHE_SLOTS;
  cache.key[slot] = key;
  cache.map[slot] = *map;
  return true;
}

}  // namespace texo

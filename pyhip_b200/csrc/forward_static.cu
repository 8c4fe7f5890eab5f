// b200moe_forward_static: the whole-layer call for hosts that must not allocate.
//
// Some callers of this library cannot obtain device memory at call time: a serving engine that
// hands every free byte of HBM to its KV-cache pool at start-up (a later cudaMalloc simply fails),
// a plugin running inside someone else's allocator discipline, or a host written in a language
// whose binding exposes no allocator at all.  b200moe_forward asks such a caller for a workspace
// it has no way to produce.  This variant keeps the layer's scratch -- the sort arrays, the
// quantised activation rows, the sorted down-projection rows -- in a fixed array that is part of
// the loaded library image, so the caller passes only inputs and outputs.
//
// Consequences a caller has to know:
//   * the array (kStaticScratchBytes, 48 MiB) is reserved on every GPU that loads the library,
//     for as long as the library stays loaded;
//   * shapes whose workspace layout is larger are refused with an argument error -- this entry
//     point is for decode-sized batches;
//   * all calls on a device share the one array and it keeps whatever the previous call left:
//     the status words are cleared at the start of every call, everything else is rewritten
//     before it is read; two calls whose GPU work overlaps (different streams, no dependency)
//     race on it and must be serialised by the caller;
//   * the first call on each device looks the array's device address up (and the kernels set
//     their shared-memory attributes); make that first call outside any stream capture;
//   * the device that is current when the call is made must be the device `stream` belongs to;
//   * the kernels' error words live inside the array too: b200moe_static_status copies the words the
//     latest call on this device left (the next call clears them).
// Nothing here calls cudaMalloc, cudaFree or any allocating library routine.
#include <mutex>

#include "internal.h"

namespace b200moe {

constexpr int64_t kStaticScratchBytes = B200MOE_STATIC_SCRATCH_BYTES;
constexpr int kMaxDevices = 64;

// Scratch of the no-allocation entry point.  In host code this name is only a handle for
// cudaGetSymbolAddress -- it is NOT a device address and must never be passed to a kernel.
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes + 1024];

static std::mutex g_static_mutex;
static unsigned char* g_static_base[kMaxDevices] = {};   // 1024-byte aligned device address, per device

// Device address of the scratch array on the current device (looked up once per device).
static int static_scratch_base(unsigned char** out) {
  int dev = -1;
  B200_CHECK_CUDA(cudaGetDevice(&dev));
  B200_CHECK_ARG(dev >= 0 && dev < kMaxDevices, "forward_static: device index %d outside [0,%d)", dev, kMaxDevices);
  std::lock_guard<std::mutex> lock(g_static_mutex);
  if (g_static_base[dev] == nullptr) {
    void* ptr = nullptr;
    B200_CHECK_CUDA(cudaGetSymbolAddress(&ptr, g_static_scratch));
    B200_CHECK_ARG(ptr != nullptr, "forward_static: the scratch symbol has no address on device %d", dev);
    const uintptr_t aligned = (reinterpret_cast<uintptr_t>(ptr) + 1023) & ~uintptr_t(1023);
    g_static_base[dev] = reinterpret_cast<unsigned char*>(aligned);
  }
  *out = g_static_base[dev];
  return 0;
}

}  // namespace b200moe

using namespace b200moe;

extern "C" int b200moe_forward_static(const b200moe_shape* shape, const void* x_bf16, const int32_t* topk_ids,
                                      const float* topk_weight, const int32_t* expert_mask, const void* w1_q,
                                      const void* w1_scale_prepared, const void* w2_q,
                                      const void* w2_scale_prepared, void* y_bf16, void* stream) {
  b200moe_workspace ws;
  if (int rc = b200moe_workspace_layout(shape, &ws)) return rc;
  B200_CHECK_ARG(ws.total_bytes <= kStaticScratchBytes,
                 "forward_static: this shape needs %lld bytes of scratch, the built-in array holds %lld "
                 "(use b200moe_forward with a caller-provided workspace)",
                 (long long)ws.total_bytes, (long long)kStaticScratchBytes);
  if (shape->T == 0) return 0;
  unsigned char* base = nullptr;
  if (int rc = static_scratch_base(&base)) return rc;
  // the array still holds the previous call's data: only the status words must start at zero
  B200_CHECK_CUDA(cudaMemsetAsync(base + ws.off_status, 0, 64, (cudaStream_t)stream));
  return b200moe_forward(shape, &ws, base, x_bf16, topk_ids, topk_weight, expert_mask, w1_q, w1_scale_prepared,
                         w2_q, w2_scale_prepared, y_bf16, stream);
}

// Copies the 16 device-side status words of the latest b200moe_forward_static call with this shape on the current
// device into host memory (asynchronously on `stream`: synchronise before reading).  Word 0: non-zero when a
// bounded wait inside a kernel gave up; word 2: non-zero when a block carried an expert id outside the weight image.
extern "C" int b200moe_static_status(const b200moe_shape* shape, int32_t* status_host16, void* stream) {
  b200moe_workspace ws;
  if (int rc = b200moe_workspace_layout(shape, &ws)) return rc;
  B200_CHECK_ARG(status_host16 != nullptr, "static_status: NULL output");
  B200_CHECK_ARG(ws.total_bytes <= kStaticScratchBytes, "static_status: shape is beyond the built-in array");
  unsigned char* base = nullptr;
  if (int rc = static_scratch_base(&base)) return rc;
  B200_CHECK_CUDA(cudaMemcpyAsync(status_host16, base + ws.off_status, 64, cudaMemcpyDeviceToHost, (cudaStream_t)stream));
  return 0;
}

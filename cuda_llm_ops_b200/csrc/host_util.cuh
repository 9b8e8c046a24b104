// Host-side helpers: error bookkeeping, per-device properties, tensor-map encoding.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>

#include <atomic>
#include <mutex>
#include <vector>

#include "common.cuh"

namespace cllo {

static thread_local int t_last_cuda_error = 0;

#define CLLO_CUDA_TRY(expr)                                  \
    do {                                                     \
        cudaError_t _e = (expr);                             \
        if (_e != cudaSuccess) {                             \
            ::cllo::t_last_cuda_error = static_cast<int>(_e); \
            (void)cudaGetLastError();                        \
            return CLLO_E_CUDA;                              \
        }                                                    \
    } while (0)

constexpr int kMaxDevices = 64;

struct DeviceInfo {
    // the *_attr_set flags record that a kernel's launch attributes were set on this device; they are atomics
    // because launchers on different host threads read and set them without taking g_dev_mutex
    bool valid = false;
    int sm_count = 0;
    int cc_major = 0;
    int cc_minor = 0;
    std::atomic<bool> decode_attr_set{false};
    std::atomic<bool> prefill_attr_set{false};
    std::atomic<bool> backward_attr_set{false};
    std::atomic<bool> sgqa_attr_set{false};
    std::atomic<bool> mla_attr_set{false};
    std::atomic<bool> one_tile_attr_set{false};
    void* legacy_ws = nullptr;  // scratch cached by the source-compatibility wrapper only
    size_t legacy_ws_bytes = 0;
    std::vector<void*> retired_ws;  // outgrown scratch buffers, freed by cllo_shutdown()
};

static DeviceInfo g_dev[kMaxDevices];
static std::mutex g_dev_mutex;

// Looks up (and caches) the properties of the current device.
static int current_device_info(DeviceInfo** out, int* dev_out = nullptr) {
    int dev = 0;
    CLLO_CUDA_TRY(cudaGetDevice(&dev));
    if (dev < 0 || dev >= kMaxDevices) return CLLO_E_UNSUPPORTED;
    std::lock_guard<std::mutex> lock(g_dev_mutex);
    DeviceInfo& d = g_dev[dev];
    if (!d.valid) {
        CLLO_CUDA_TRY(cudaDeviceGetAttribute(&d.sm_count, cudaDevAttrMultiProcessorCount, dev));
        CLLO_CUDA_TRY(cudaDeviceGetAttribute(&d.cc_major, cudaDevAttrComputeCapabilityMajor, dev));
        CLLO_CUDA_TRY(cudaDeviceGetAttribute(&d.cc_minor, cudaDevAttrComputeCapabilityMinor, dev));
        d.valid = true;
    }
    *out = &d;
    if (dev_out) *dev_out = dev;
    return CLLO_OK;
}

// cuTensorMapEncodeTiled is a driver entry point; fetch it through the runtime so the library has
// no link-time dependency on libcuda (it must load on machines without a driver).
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static int get_encode_fn(EncodeTiledFn* fn) {
    static EncodeTiledFn cached = nullptr;
    static std::mutex m;
    std::lock_guard<std::mutex> lock(m);
    if (!cached) {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        CLLO_CUDA_TRY(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q));
        if (q != cudaDriverEntryPointSuccess || !p) {
            t_last_cuda_error = static_cast<int>(cudaErrorSymbolNotFound);
            return CLLO_E_CUDA;
        }
        cached = reinterpret_cast<EncodeTiledFn>(p);
    }
    *fn = cached;
    return CLLO_OK;
}

// bf16 tensor map, rank 4, 128-byte swizzle, zero fill outside the tensor.
// dims/strides are listed fastest first; strides (bytes) are given for dims 1..3.
static int encode_bf16_4d(CUtensorMap* map, const void* base, const uint64_t dims[4], const uint64_t strides[3],
                          const uint32_t box[4]) {
    EncodeTiledFn fn;
    int rc = get_encode_fn(&fn);
    if (rc != CLLO_OK) return rc;
    cuuint64_t gdim[4] = {dims[0], dims[1], dims[2], dims[3]};
    cuuint64_t gstr[3] = {strides[0], strides[1], strides[2]};
    cuuint32_t bx[4] = {box[0], box[1], box[2], box[3]};
    cuuint32_t es[4] = {1, 1, 1, 1};
    CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(base), gdim, gstr, bx, es,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        t_last_cuda_error = static_cast<int>(cudaErrorInvalidValue);
        return CLLO_E_CUDA;
    }
    return CLLO_OK;
}

static inline bool aligned_to(const void* p, size_t a) { return (reinterpret_cast<uintptr_t>(p) % a) == 0; }

}  // namespace cllo

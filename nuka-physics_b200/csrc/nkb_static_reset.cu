// Partial reset whose env-id list sits in a fixed device array of this module instead of a heap allocation.
// The kernel is reset_kernel's partial-reset form (nkb_kernels.cu) reading its ids through a pointer argument.
#include <cuda_runtime.h>
#include <mutex>
#include "nkb_launch.h"

namespace nkb {

// Id list of the partial reset in flight: kStaticResetMaxIds words (16 KB) of device memory per device that loads
// the module.  Nothing in it has to start at zero: every call overwrites the first `count` words before its
// kernel reads them, and the kernel reads no further.
static __device__ __align__(256) uint32_t g_static_reset_ids[kStaticResetMaxIds];

__global__ void reset_kernel_static_ids(ResetParams r, const uint32_t* ids) {
    const uint32_t env = ids[blockIdx.x];
    if (env >= r.env_count) return;
    for (uint32_t f = 0u; f < r.field_count; ++f) {
        const ResetField fd = r.fields[f];
        uint32_t* dst = reinterpret_cast<uint32_t*>(fd.dst) + (size_t)env * fd.words;
        const uint32_t* src = reinterpret_cast<const uint32_t*>(fd.src);
        for (uint32_t k = threadIdx.x; k < fd.words; k += blockDim.x) dst[k] = fd.per_env_src ? src[(size_t)env * fd.words + k] : (fd.src != nullptr ? src[k] : fd.fill);
    }
}

namespace {
constexpr int kMaxDevices = 64;
std::mutex g_lock;
uint32_t* g_ids_on_device[kMaxDevices] = {};     // address of g_static_reset_ids per device, resolved on first use
}  // namespace

// Address of the id array on `device`, which must be the current device.  The first call per device asks the
// runtime for it (cudaGetSymbolAddress); later calls return the remembered pointer.
static cudaError_t static_reset_ids(int device, uint32_t** out) {
    if (device < 0 || device >= kMaxDevices) return cudaErrorInvalidDevice;
    std::lock_guard<std::mutex> hold(g_lock);
    if (g_ids_on_device[device] == nullptr) {
        uint32_t* ptr = nullptr;
        const cudaError_t err = cudaGetSymbolAddress((void**)&ptr, g_static_reset_ids);
        if (err != cudaSuccess) return err;
        g_ids_on_device[device] = ptr;
    }
    *out = g_ids_on_device[device];
    return cudaSuccess;
}

cudaError_t launch_reset_static_ids(const ResetParams& r, const uint32_t* host_ids, uint32_t count, int device, cudaStream_t stream,
                                    const uint32_t** device_ids) {
    *device_ids = nullptr;
    if (count == 0u) return cudaSuccess;
    if (count > kStaticResetMaxIds) return cudaErrorInvalidValue;
    uint32_t* ids = nullptr;
    cudaError_t err = static_reset_ids(device, &ids);
    if (err != cudaSuccess) return err;
    err = cudaMemcpyAsync(ids, host_ids, (size_t)count * sizeof(uint32_t), cudaMemcpyHostToDevice, stream);
    if (err != cudaSuccess) return err;
    reset_kernel_static_ids<<<count, 128, 0, stream>>>(r, ids);
    *device_ids = ids;
    return cudaGetLastError();
}

}  // namespace nkb

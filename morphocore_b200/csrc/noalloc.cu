// mc_morpho_backward_noalloc: the dilation / erosion backward pass for hosts that cannot allocate.
//
// Some hosts of this library may not call cudaMalloc at all: an inference or training server that has
// handed every byte of device memory to its own arena at start-up, a plugin that lives inside another
// framework's memory pool, or a latency-critical loop where cudaMalloc's implicit device
// synchronisation is not acceptable. mc_morpho_backward needs scratch memory in one case: a MAX / MIN
// merge whose winner indices were not kept by the forward pass, where the winners are recomputed into a
// caller-provided workspace. For those hosts this file provides the same computation with the scratch
// taken from a fixed array that is part of the library image, so neither the caller nor the library
// allocates anything.
//
// Cost and limits:
//  - the array is MC_NOALLOC_SCRATCH_BYTES (16 MiB) and every GPU that loads the library holds it until
//    the process exits; it bounds the call to B * Co * H * W <= 4 194 304 output pixels, larger calls are
//    rejected with MC_ERR_UNSUPPORTED;
//  - the first call on each device looks the array's device address up (cudaGetSymbolAddress, with that
//    device current). Make that first call outside any stream capture;
//  - every call on a device shares the one array, which still holds the previous call's winners
//    afterwards. Nothing in it has to start at zero, because each call overwrites every entry it later
//    reads, but two calls that overlap on the GPU (different streams, or threads) race on it: serialise
//    them.
#include <mutex>

#include "common.cuh"

namespace
{

constexpr size_t SCRATCH_BYTES = MC_NOALLOC_SCRATCH_BYTES;
constexpr int MAX_DEVICES = 64;

// In host code this name is only a handle for cudaGetSymbolAddress, never a device address.
static __device__ __align__(256) unsigned char g_noalloc_scratch[SCRATCH_BYTES];

std::mutex g_setup_mutex;
void* g_scratch_address[MAX_DEVICES] = {};

/// Device address of the scratch array on the current device, looked up once per device.
int scratch_address(void** out)
{
    int device = -1;
    cudaError_t err = cudaGetDevice(&device);
    if (err != cudaSuccess || device < 0 || device >= MAX_DEVICES)
    {
        mc::set_last_error("cudaGetDevice: %s (device %d)", cudaGetErrorString(err), device);
        return MC_ERR_CUDA;
    }
    std::lock_guard<std::mutex> lock(g_setup_mutex);
    if (g_scratch_address[device] == nullptr)
    {
        void* address = nullptr;
        err = cudaGetSymbolAddress(&address, g_noalloc_scratch);
        if (err != cudaSuccess || address == nullptr)
        {
            mc::set_last_error("cudaGetSymbolAddress(scratch): %s", cudaGetErrorString(err));
            return MC_ERR_CUDA;
        }
        g_scratch_address[device] = address;
    }
    *out = g_scratch_address[device];
    return MC_OK;
}

}  // namespace

extern "C" int mc_morpho_backward_noalloc(const mc_desc* desc, const void* x, const void* w, const void* gy, void* gx, void* gw, void* stream)
{
    // The descriptor is checked before anything is sized from it: a negative extent must read "invalid argument",
    // not a wrapped-around pixel count.
    const int valid = mc::validate(desc, true);
    if (valid != MC_OK) return valid;
    const size_t need = mc_morpho_backward_workspace_bytes(desc, 0);
    if (need > SCRATCH_BYTES)
    {
        mc::set_last_error("mc_morpho_backward_noalloc: B*Co*H*W = %lld output pixels need %zu bytes of winner indices, the built-in scratch "
                           "holds %zu bytes (%zu pixels); use mc_morpho_backward with a workspace",
                           static_cast<long long>(need / sizeof(int32_t)), need, SCRATCH_BYTES, SCRATCH_BYTES / sizeof(int32_t));
        return MC_ERR_UNSUPPORTED;
    }
    void* scratch = nullptr;
    if (need > 0)
    {
        const int rc = scratch_address(&scratch);
        if (rc != MC_OK) return rc;
    }
    // Same validation and kernels as mc_morpho_backward, with the library's own array as the workspace.
    return mc_morpho_backward(desc, x, w, nullptr, gy, gx, gw, scratch, need > 0 ? SCRATCH_BYTES : 0, stream);
}

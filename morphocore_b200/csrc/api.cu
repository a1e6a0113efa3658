// C-ABI entry points: argument validation, dtype dispatch, status strings.
#include <atomic>
#include <cstdarg>
#include <cstdio>

#include "common.cuh"
#include "tma.cuh"

namespace mc
{

static __device__ unsigned int g_device_error = 0;

unsigned int* device_error_counter()
{
    constexpr int MAX_DEVICES = 64;
    static std::atomic<unsigned int*> cache[MAX_DEVICES];
    int device = 0;
    if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= MAX_DEVICES) return nullptr;
    unsigned int* p = cache[device].load(std::memory_order_acquire);
    if (p == nullptr)
    {
        void* address = nullptr;
        if (cudaGetSymbolAddress(&address, g_device_error) != cudaSuccess) return nullptr;
        p = static_cast<unsigned int*>(address);
        cache[device].store(p, std::memory_order_release);
    }
    return p;
}

static std::atomic<uint64_t> g_wait_limit_ns{1000000000ull};  // one second

uint64_t wait_limit_ns() { return g_wait_limit_ns.load(std::memory_order_relaxed); }

/// One CTA that waits, with the bounded wait of the TMA kernels, on an mbarrier that expects 16 bytes which no copy
/// ever delivers: the wait runs out after limit_ns, the CTA counts the time-out and returns. Nothing faults or
/// spins; this is how the time-out path is exercised.
__global__ void wait_timeout_selftest_kernel(unsigned int* errors, uint64_t limit_ns)
{
    __shared__ uint64_t bar;
    if (threadIdx.x == 0)
    {
        mbar_init(&bar, 1);
        mbar_fence_init();
    }
    __syncthreads();
    if (threadIdx.x == 0) mbar_expect_tx(&bar, 16);
    __syncthreads();
    if (!mbar_wait(&bar, 0, limit_ns))
    {
        if (threadIdx.x == 0 && errors != nullptr) atomicAdd(errors, 1u);
        return;
    }
}

static thread_local char g_last_error[512] = "";
static std::atomic<uint64_t> g_launches{0};

void set_last_error(const char* fmt, ...)
{
    va_list args;
    va_start(args, fmt);
    vsnprintf(g_last_error, sizeof(g_last_error), fmt, args);
    va_end(args);
}

void count_launch() { g_launches.fetch_add(1, std::memory_order_relaxed); }

/// Checks shared by every entry point. The limits on taps and channels are those of the packed winner
/// index, (channel << 16) | tap.
int validate(const mc_desc* d, bool morph, bool smooth)
{
    if (d == nullptr) { set_last_error("descriptor is NULL"); return MC_ERR_INVALID_ARGUMENT; }
    if (d->B < 0 || d->Ci <= 0 || d->Co <= 0 || d->H < 0 || d->W < 0 || d->kH <= 0 || d->kW <= 0)
    {
        set_last_error("sizes must be positive (B=%d Ci=%d Co=%d H=%d W=%d kH=%d kW=%d)", d->B, d->Ci, d->Co, d->H, d->W, d->kH, d->kW);
        return MC_ERR_INVALID_ARGUMENT;
    }
    {
        // Element counts must stay far inside 64 bits (the workspace sizes multiply four extents): 2^40 elements is
        // more than any device holds.
        const unsigned __int128 limit = static_cast<unsigned __int128>(1) << 40;
        const unsigned __int128 pixels = static_cast<unsigned __int128>(d->B) * static_cast<unsigned>(d->H) * static_cast<unsigned>(d->W);
        if (pixels * static_cast<unsigned>(d->Ci) > limit || pixels * static_cast<unsigned>(d->Co) > limit)
        {
            set_last_error("tensor of more than 2^40 elements (B=%d Ci=%d Co=%d H=%d W=%d)", d->B, d->Ci, d->Co, d->H, d->W);
            return MC_ERR_INVALID_ARGUMENT;
        }
    }
    if (d->dtype != MC_F32 && d->dtype != MC_F64) { set_last_error("unknown dtype %d", d->dtype); return MC_ERR_INVALID_ARGUMENT; }
    if (d->merge < MC_MERGE_MAX || d->merge > MC_MERGE_IDENTITY) { set_last_error("Unknown merge mode %d", d->merge); return MC_ERR_INVALID_ARGUMENT; }
    if (smooth && d->merge != MC_MERGE_SMOOTH) { set_last_error("mc_smorph_scm_* take merge = MC_MERGE_SMOOTH"); return MC_ERR_INVALID_ARGUMENT; }
    if (!smooth && d->merge == MC_MERGE_SMOOTH)
    {
        set_last_error("the smooth channel merge exists for smorph only and has its own entry points, mc_smorph_scm_*");
        return MC_ERR_UNSUPPORTED;
    }
    if (d->merge == MC_MERGE_IDENTITY && d->Co != d->Ci)
    {
        set_last_error("Identity mode requires weight.shape[0] == input.shape[1]");
        return MC_ERR_INVALID_ARGUMENT;
    }
    if (morph)
    {
        if (d->op != MC_OP_DILATION && d->op != MC_OP_EROSION) { set_last_error("unknown operation %d", d->op); return MC_ERR_INVALID_ARGUMENT; }
        if (d->pad_kind != MC_PAD_FILL && d->pad_kind != MC_PAD_REPLICATE) { set_last_error("Unknown padding kind %d", d->pad_kind); return MC_ERR_INVALID_ARGUMENT; }
        if (d->weight_batch_stride < 0) { set_last_error("negative weight_batch_stride"); return MC_ERR_INVALID_ARGUMENT; }
    }
    else if (d->weight_batch_stride != 0) { set_last_error("smorph takes a shared structuring element"); return MC_ERR_INVALID_ARGUMENT; }
    if (static_cast<int64_t>(d->kH) * d->kW >= (1 << 16) || d->Ci >= (1 << 15))
    {
        set_last_error("Structuring element or channel count too large to save indices");
        return MC_ERR_UNSUPPORTED;
    }
    return MC_OK;
}

static bool empty(const mc_desc* d) { return static_cast<int64_t>(d->B) * d->H * d->W == 0; }

}  // namespace mc

using namespace mc;

#define MC_REQUIRE(ptr)                                                      \
    if ((ptr) == nullptr)                                                    \
    {                                                                        \
        set_last_error(#ptr " is NULL");                                     \
        return MC_ERR_INVALID_ARGUMENT;                                      \
    }

extern "C" {

int mc_morpho_forward(const mc_desc* desc, const void* x, const void* w, void* y, int32_t* idx, void* stream)
{
    const int rc = validate(desc, true);
    if (rc != MC_OK) return rc;
    if (empty(desc)) return MC_OK;
    MC_REQUIRE(x); MC_REQUIRE(w);
    if (y == nullptr && idx == nullptr) { set_last_error("y and idx are both NULL"); return MC_ERR_INVALID_ARGUMENT; }
    if (desc->merge != MC_MERGE_MAX && desc->merge != MC_MERGE_MIN) idx = nullptr;  // only a single winner has an index
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (desc->dtype == MC_F32) return morpho_forward<float>(*desc, static_cast<const float*>(x), static_cast<const float*>(w), static_cast<float*>(y), idx, s);
    return morpho_forward<double>(*desc, static_cast<const double*>(x), static_cast<const double*>(w), static_cast<double*>(y), idx, s);
}

int mc_morpho_pair_forward(const mc_desc* desc, const void* x, const void* w, void* y_dilation, void* y_erosion, void* stream)
{
    const int rc = validate(desc, true);
    if (rc != MC_OK) return rc;
    if (empty(desc)) return MC_OK;
    MC_REQUIRE(x); MC_REQUIRE(w); MC_REQUIRE(y_dilation); MC_REQUIRE(y_erosion);
    if (desc->dtype != MC_F32) return MC_ERR_UNSUPPORTED;
    return morpho_pair_forward(*desc, static_cast<const float*>(x), static_cast<const float*>(w), static_cast<float*>(y_dilation),
                               static_cast<float*>(y_erosion), static_cast<cudaStream_t>(stream));
}

size_t mc_morpho_backward_workspace_bytes(const mc_desc* desc, int have_idx)
{
    if (desc == nullptr || have_idx) return 0;
    if (desc->merge != MC_MERGE_MAX && desc->merge != MC_MERGE_MIN) return 0;
    return sizeof(int32_t) * static_cast<size_t>(desc->B) * desc->Co * desc->H * desc->W;
}

int mc_morpho_backward(const mc_desc* desc, const void* x, const void* w, const int32_t* idx, const void* gy, void* gx, void* gw, void* workspace,
                       size_t workspace_bytes, void* stream)
{
    const int rc = validate(desc, true);
    if (rc != MC_OK) return rc;
    MC_REQUIRE(gw);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (empty(desc))
    {
        const size_t wn = static_cast<size_t>(desc->Co) * (desc->merge == MC_MERGE_IDENTITY ? 1 : desc->Ci) * desc->kH * desc->kW;
        if (cudaMemsetAsync(gw, 0, wn * (desc->dtype == MC_F32 ? 4 : 8), s) != cudaSuccess) { set_last_error("cudaMemsetAsync failed"); return MC_ERR_CUDA; }
        return MC_OK;
    }
    MC_REQUIRE(x); MC_REQUIRE(w); MC_REQUIRE(gy); MC_REQUIRE(gx);
    const size_t need = mc_morpho_backward_workspace_bytes(desc, idx != nullptr);
    if (need > 0 && (workspace == nullptr || workspace_bytes < need))
    {
        set_last_error("workspace of %zu bytes needed, %zu given", need, workspace_bytes);
        return MC_ERR_WORKSPACE;
    }
    if (desc->dtype == MC_F32)
        return morpho_backward<float>(*desc, static_cast<const float*>(x), static_cast<const float*>(w), idx, static_cast<const float*>(gy),
                                      static_cast<float*>(gx), static_cast<float*>(gw), workspace, s);
    return morpho_backward<double>(*desc, static_cast<const double*>(x), static_cast<const double*>(w), idx, static_cast<const double*>(gy),
                                   static_cast<double*>(gx), static_cast<double*>(gw), workspace, s);
}

int mc_smorph_forward(const mc_desc* desc, const void* x, const void* w, const void* alpha_pairs, void* y, void* stream)
{
    const int rc = validate(desc, false);
    if (rc != MC_OK) return rc;
    if (empty(desc)) return MC_OK;
    MC_REQUIRE(x); MC_REQUIRE(w); MC_REQUIRE(alpha_pairs); MC_REQUIRE(y);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (desc->dtype == MC_F32)
        return smorph_forward<float>(*desc, static_cast<const float*>(x), static_cast<const float*>(w), static_cast<const float*>(alpha_pairs),
                                     static_cast<float*>(y), nullptr, s);
    return smorph_forward<double>(*desc, static_cast<const double*>(x), static_cast<const double*>(w), static_cast<const double*>(alpha_pairs),
                                  static_cast<double*>(y), nullptr, s);
}

size_t mc_smorph_backward_workspace_bytes(const mc_desc* desc)
{
    if (desc == nullptr) return 0;
    if (desc->merge != MC_MERGE_MAX && desc->merge != MC_MERGE_MIN) return 0;
    return (desc->dtype == MC_F32 ? 4 : 8) * static_cast<size_t>(desc->B) * desc->Co * desc->H * desc->W;
}

int mc_smorph_backward(const mc_desc* desc, const void* x, const void* w, const void* alpha_pairs, const void* y, const void* gy, void* gx,
                       void* gw, void* galpha_pairs, void* workspace, size_t workspace_bytes, void* stream)
{
    const int rc = validate(desc, false);
    if (rc != MC_OK) return rc;
    MC_REQUIRE(gw); MC_REQUIRE(galpha_pairs);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const size_t esz = desc->dtype == MC_F32 ? 4 : 8;
    if (empty(desc))
    {
        const bool identity = desc->merge == MC_MERGE_IDENTITY;
        const size_t wn = static_cast<size_t>(desc->Co) * (identity ? 1 : desc->Ci) * desc->kH * desc->kW;
        const size_t an = identity ? desc->Co : static_cast<size_t>(desc->Co) * desc->Ci;
        if (cudaMemsetAsync(gw, 0, wn * esz, s) != cudaSuccess || cudaMemsetAsync(galpha_pairs, 0, an * esz, s) != cudaSuccess)
        {
            set_last_error("cudaMemsetAsync failed");
            return MC_ERR_CUDA;
        }
        return MC_OK;
    }
    MC_REQUIRE(x); MC_REQUIRE(w); MC_REQUIRE(alpha_pairs); MC_REQUIRE(y); MC_REQUIRE(gy); MC_REQUIRE(gx);
    const size_t need = mc_smorph_backward_workspace_bytes(desc);
    if (need > 0 && (workspace == nullptr || workspace_bytes < need))
    {
        set_last_error("workspace of %zu bytes needed, %zu given", need, workspace_bytes);
        return MC_ERR_WORKSPACE;
    }
    if (desc->dtype == MC_F32)
        return smorph_backward<float>(*desc, static_cast<const float*>(x), static_cast<const float*>(w), static_cast<const float*>(alpha_pairs),
                                      static_cast<const float*>(y), static_cast<const float*>(gy), static_cast<float*>(gx), static_cast<float*>(gw),
                                      static_cast<float*>(galpha_pairs), workspace, s);
    return smorph_backward<double>(*desc, static_cast<const double*>(x), static_cast<const double*>(w), static_cast<const double*>(alpha_pairs),
                                   static_cast<const double*>(y), static_cast<const double*>(gy), static_cast<double*>(gx), static_cast<double*>(gw),
                                   static_cast<double*>(galpha_pairs), workspace, s);
}

int mc_smorph_scm_forward(const mc_desc* desc, const void* x, const void* w, const void* alpha_pairs, const void* beta, void* y, void* stream)
{
    const int rc = validate(desc, false, true);
    if (rc != MC_OK) return rc;
    if (empty(desc)) return MC_OK;
    MC_REQUIRE(x); MC_REQUIRE(w); MC_REQUIRE(alpha_pairs); MC_REQUIRE(beta); MC_REQUIRE(y);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (desc->dtype == MC_F32)
        return smorph_scm_forward<float>(*desc, static_cast<const float*>(x), static_cast<const float*>(w), static_cast<const float*>(alpha_pairs),
                                         static_cast<const float*>(beta), static_cast<float*>(y), s);
    return smorph_scm_forward<double>(*desc, static_cast<const double*>(x), static_cast<const double*>(w), static_cast<const double*>(alpha_pairs),
                                      static_cast<const double*>(beta), static_cast<double*>(y), s);
}

size_t mc_smorph_scm_backward_workspace_bytes(const mc_desc* desc)
{
    if (desc == nullptr) return 0;
    return 2 * (desc->dtype == MC_F32 ? 4 : 8) * static_cast<size_t>(desc->B) * desc->Co * desc->H * desc->W;
}

int mc_smorph_scm_backward(const mc_desc* desc, const void* x, const void* w, const void* alpha_pairs, const void* beta, const void* y,
                           const void* gy, void* gx, void* gw, void* galpha_pairs, void* gbeta, void* workspace, size_t workspace_bytes,
                           void* stream)
{
    const int rc = validate(desc, false, true);
    if (rc != MC_OK) return rc;
    MC_REQUIRE(gw); MC_REQUIRE(galpha_pairs); MC_REQUIRE(gbeta);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const size_t esz = desc->dtype == MC_F32 ? 4 : 8;
    if (empty(desc))
    {
        const size_t an = static_cast<size_t>(desc->Co) * desc->Ci;
        if (cudaMemsetAsync(gw, 0, an * desc->kH * desc->kW * esz, s) != cudaSuccess || cudaMemsetAsync(galpha_pairs, 0, an * esz, s) != cudaSuccess
            || cudaMemsetAsync(gbeta, 0, desc->Co * esz, s) != cudaSuccess)
        {
            set_last_error("cudaMemsetAsync failed");
            return MC_ERR_CUDA;
        }
        return MC_OK;
    }
    MC_REQUIRE(x); MC_REQUIRE(w); MC_REQUIRE(alpha_pairs); MC_REQUIRE(beta); MC_REQUIRE(y); MC_REQUIRE(gy); MC_REQUIRE(gx);
    const size_t need = mc_smorph_scm_backward_workspace_bytes(desc);
    if (workspace == nullptr || workspace_bytes < need)
    {
        set_last_error("workspace of %zu bytes needed, %zu given", need, workspace_bytes);
        return MC_ERR_WORKSPACE;
    }
    if (desc->dtype == MC_F32)
        return smorph_scm_backward<float>(*desc, static_cast<const float*>(x), static_cast<const float*>(w), static_cast<const float*>(alpha_pairs),
                                          static_cast<const float*>(beta), static_cast<const float*>(y), static_cast<const float*>(gy),
                                          static_cast<float*>(gx), static_cast<float*>(gw), static_cast<float*>(galpha_pairs),
                                          static_cast<float*>(gbeta), workspace, s);
    return smorph_scm_backward<double>(*desc, static_cast<const double*>(x), static_cast<const double*>(w), static_cast<const double*>(alpha_pairs),
                                       static_cast<const double*>(beta), static_cast<const double*>(y), static_cast<const double*>(gy),
                                       static_cast<double*>(gx), static_cast<double*>(gw), static_cast<double*>(galpha_pairs),
                                       static_cast<double*>(gbeta), workspace, s);
}

const char* mc_status_string(int status)
{
    switch (status)
    {
        case MC_OK: return "ok";
        case MC_ERR_INVALID_ARGUMENT: return "invalid argument";
        case MC_ERR_UNSUPPORTED: return "unsupported configuration";
        case MC_ERR_WORKSPACE: return "workspace too small";
        case MC_ERR_CUDA: return "CUDA error";
        default: return "unknown status";
    }
}

const char* mc_last_error(void) { return g_last_error; }

int mc_device_error_count(void)
{
    unsigned int count = 0;
    const cudaError_t err = cudaMemcpyFromSymbol(&count, g_device_error, sizeof(count));
    if (err != cudaSuccess)
    {
        set_last_error("cudaMemcpyFromSymbol: %s", cudaGetErrorString(err));
        return MC_ERR_CUDA;
    }
    return static_cast<int>(count > 0x7fffffffu ? 0x7fffffffu : count);
}

int mc_device_error_reset(void)
{
    const unsigned int zero = 0;
    const cudaError_t err = cudaMemcpyToSymbol(g_device_error, &zero, sizeof(zero));
    if (err != cudaSuccess)
    {
        set_last_error("cudaMemcpyToSymbol: %s", cudaGetErrorString(err));
        return MC_ERR_CUDA;
    }
    return MC_OK;
}

int mc_set_wait_limit_ns(uint64_t limit_ns)
{
    if (limit_ns == 0)
    {
        set_last_error("the wait limit must be positive");
        return MC_ERR_INVALID_ARGUMENT;
    }
    g_wait_limit_ns.store(limit_ns, std::memory_order_relaxed);
    return MC_OK;
}

int mc_selftest_wait_timeout(uint64_t limit_ns, void* stream)
{
    if (limit_ns == 0 || limit_ns > 1000000000ull)
    {
        set_last_error("mc_selftest_wait_timeout: limit of 1 ns .. 1 s expected");
        return MC_ERR_INVALID_ARGUMENT;
    }
    wait_timeout_selftest_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(device_error_counter(), limit_ns);
    return check_launch("wait_timeout_selftest_kernel");
}

uint64_t mc_launch_count(void) { return g_launches.load(std::memory_order_relaxed); }

int mc_version(void) { return 100; }

}  // extern "C"

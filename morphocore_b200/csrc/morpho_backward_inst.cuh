// Instantiates mc::morpho_backward<MC_T>; included by morpho_backward_f32.cu / _f64.cu.
#include <type_traits>

#include "dispatch.cuh"
#include "morpho_backward.cuh"

namespace mc
{

template <>
int morpho_backward<MC_T>(const mc_desc& d, const MC_T* x, const MC_T* w, const int32_t* idx, const MC_T* gy, MC_T* gx, MC_T* gw, void* ws,
                          cudaStream_t stream)
{
    using T = MC_T;
    constexpr int WIDE = sizeof(T) == 4 ? 4 : 2;
    const size_t taps = static_cast<size_t>(d.kH) * d.kW;
    const size_t wnumel = static_cast<size_t>(d.Co) * (d.merge == MC_MERGE_IDENTITY ? 1 : d.Ci) * taps;
    // Both gradients are sums that the kernels below build up with atomic adds: start from zero.
    if (cudaMemsetAsync(gx, 0, sizeof(T) * static_cast<size_t>(d.B) * d.Ci * d.H * d.W, stream) != cudaSuccess
        || cudaMemsetAsync(gw, 0, sizeof(T) * wnumel, stream) != cudaSuccess)
    {
        set_last_error("cudaMemsetAsync: %s", cudaGetErrorString(cudaGetLastError()));
        return MC_ERR_CUDA;
    }
    if (d.merge == MC_MERGE_MAX || d.merge == MC_MERGE_MIN)
    {
        if (idx == nullptr)
        {
            // No saved winners: the forward kernel recomputes them into the workspace.
            const int rc = morpho_forward<T>(d, x, w, nullptr, static_cast<int32_t*>(ws), stream);
            if (rc != MC_OK) return rc;
            idx = static_cast<const int32_t*>(ws);
        }
        return dispatch_kernel_width(d.kH, d.kW, [&](auto kw) { return launch_backward_scatter<T, decltype(kw)::value>(d, idx, gy, gx, gw, stream); });
    }
    const int ob = output_block<T>(d);
    return dispatch_kernel_width(d.kH, d.kW, [&](auto kw) {
        constexpr int KW = decltype(kw)::value;
        if (d.op == MC_OP_DILATION)
            return ob == 1 ? launch_backward_pairs<T, false, KW, 1>(d, x, w, gy, gx, gw, stream)
                           : launch_backward_pairs<T, false, KW, WIDE>(d, x, w, gy, gx, gw, stream);
        return ob == 1 ? launch_backward_pairs<T, true, KW, 1>(d, x, w, gy, gx, gw, stream)
                       : launch_backward_pairs<T, true, KW, WIDE>(d, x, w, gy, gx, gw, stream);
    });
}

}  // namespace mc

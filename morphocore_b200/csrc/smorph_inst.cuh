// Instantiates mc::smorph_forward<MC_T> and mc::smorph_backward<MC_T>; included by smorph_f32.cu / _f64.cu.
#include <type_traits>

#include "dispatch.cuh"
#include "smorph.cuh"

namespace mc
{

template <>
int smorph_forward<MC_T>(const mc_desc& d, const MC_T* x, const MC_T* w, const MC_T* alpha, MC_T* y, MC_T* counts, cudaStream_t stream)
{
    using T = MC_T;
    // Stats mode (counts != nullptr) reads y as the merge target instead of writing it.
    const T* target = counts != nullptr ? y : nullptr;
    const bool wide = d.merge != MC_MERGE_IDENTITY && d.Co >= 2;
    return dispatch_kernel_width(d.kH, d.kW, [&](auto kw) {
        constexpr int KW = decltype(kw)::value;
        // Float, 3 x 3, SUM / MEAN merge: the kernel built around per-pair alphas; it declines (and launches nothing)
        // when the input cannot be staged by TMA.
        if constexpr (std::is_same<T, float>::value && KW == 3)
        {
            if (counts == nullptr && d.Co >= 4 && (d.merge == MC_MERGE_ADD || d.merge == MC_MERGE_AVERAGE))
            {
                const int rc = launch_smorph_forward_lean<3>(d, x, w, alpha, y, stream);
                if (rc != MC_ERR_UNSUPPORTED) return rc;
            }
        }
        // The factorised path has registers to spare: four output channels share every (E, A) buffer.
        if constexpr (can_factorise<T, KW, false>())
        {
            if (counts == nullptr && d.Co >= 4 && (d.merge == MC_MERGE_ADD || d.merge == MC_MERGE_AVERAGE))
                return launch_smorph_forward<T, KW, 4>(d, x, w, alpha, y, target, counts, stream);
        }
        return wide ? launch_smorph_forward<T, KW, 2>(d, x, w, alpha, y, target, counts, stream)
                    : launch_smorph_forward<T, KW, 1>(d, x, w, alpha, y, target, counts, stream);
    });
}

template <>
int smorph_backward<MC_T>(const mc_desc& d, const MC_T* x, const MC_T* w, const MC_T* alpha, const MC_T* y, const MC_T* gy, MC_T* gx, MC_T* gw,
                          MC_T* galpha, void* ws, cudaStream_t stream)
{
    using T = MC_T;
    const size_t taps = static_cast<size_t>(d.kH) * d.kW;
    const bool identity = d.merge == MC_MERGE_IDENTITY;
    const size_t wnumel = static_cast<size_t>(d.Co) * (identity ? 1 : d.Ci) * taps;
    const size_t anumel = identity ? d.Co : static_cast<size_t>(d.Co) * d.Ci;
    if (cudaMemsetAsync(gx, 0, sizeof(T) * static_cast<size_t>(d.B) * d.Ci * d.H * d.W, stream) != cudaSuccess
        || cudaMemsetAsync(gw, 0, sizeof(T) * wnumel, stream) != cudaSuccess
        || cudaMemsetAsync(galpha, 0, sizeof(T) * anumel, stream) != cudaSuccess)
    {
        set_last_error("cudaMemsetAsync: %s", cudaGetErrorString(cudaGetLastError()));
        return MC_ERR_CUDA;
    }
    const T* counts = nullptr;
    if (d.merge == MC_MERGE_MAX || d.merge == MC_MERGE_MIN)
    {
        // Winners per output pixel, from one more pass over every channel.
        const int rc = smorph_forward<T>(d, x, w, alpha, const_cast<T*>(y), static_cast<T*>(ws), stream);
        if (rc != MC_OK) return rc;
        counts = static_cast<const T*>(ws);
    }
    // Square 3, 5 and 7 structuring elements keep grad_input in registers (float only: the double
    // kernels are bound by exp() and keep the smaller code).
    if (sizeof(T) == 4 && d.kH == d.kW)
    {
        if (d.kW == 3) return launch_smorph_backward<T, 3, 3>(d, x, w, alpha, y, counts, gy, gx, gw, galpha, stream);
        if (d.kW == 5) return launch_smorph_backward<T, 5, 5>(d, x, w, alpha, y, counts, gy, gx, gw, galpha, stream);
        if (d.kW == 7) return launch_smorph_backward<T, 7, 7>(d, x, w, alpha, y, counts, gy, gx, gw, galpha, stream);
    }
    return dispatch_kernel_width(d.kH, d.kW, [&](auto kw) {
        constexpr int KW = decltype(kw)::value;
        return launch_smorph_backward<T, 0, KW>(d, x, w, alpha, y, counts, gy, gx, gw, galpha, stream);
    });
}

/// Forward launch of the smooth merge: the merged output, or (soft_ref != nullptr) the per-pixel statistics.
template <typename T>
static int launch_scm_forward(const mc_desc& d, const T* x, const T* w, const T* alpha, const T* beta, T* y, T* soft_ref, T* soft_inv,
                              cudaStream_t stream)
{
    return dispatch_kernel_width(d.kH, d.kW, [&](auto kw) {
        constexpr int KW = decltype(kw)::value;
        return d.Co >= 2 ? launch_smorph_forward<T, KW, 2>(d, x, w, alpha, y, nullptr, nullptr, stream, beta, soft_ref, soft_inv)
                         : launch_smorph_forward<T, KW, 1>(d, x, w, alpha, y, nullptr, nullptr, stream, beta, soft_ref, soft_inv);
    });
}

template <>
int smorph_scm_forward<MC_T>(const mc_desc& d, const MC_T* x, const MC_T* w, const MC_T* alpha, const MC_T* beta, MC_T* y, cudaStream_t stream)
{
    return launch_scm_forward<MC_T>(d, x, w, alpha, beta, y, nullptr, nullptr, stream);
}

template <>
int smorph_scm_backward<MC_T>(const mc_desc& d, const MC_T* x, const MC_T* w, const MC_T* alpha, const MC_T* beta, const MC_T* y, const MC_T* gy,
                              MC_T* gx, MC_T* gw, MC_T* galpha, MC_T* gbeta, void* ws, cudaStream_t stream)
{
    using T = MC_T;
    const size_t taps = static_cast<size_t>(d.kH) * d.kW, pixels = static_cast<size_t>(d.B) * d.Co * d.H * d.W;
    if (cudaMemsetAsync(gx, 0, sizeof(T) * static_cast<size_t>(d.B) * d.Ci * d.H * d.W, stream) != cudaSuccess
        || cudaMemsetAsync(gw, 0, sizeof(T) * d.Co * d.Ci * taps, stream) != cudaSuccess
        || cudaMemsetAsync(galpha, 0, sizeof(T) * d.Co * d.Ci, stream) != cudaSuccess
        || cudaMemsetAsync(gbeta, 0, sizeof(T) * d.Co, stream) != cudaSuccess)
    {
        set_last_error("cudaMemsetAsync: %s", cudaGetErrorString(cudaGetLastError()));
        return MC_ERR_CUDA;
    }
    // One more pass over every channel for the extremum and the sum of the channel weights of each output pixel.
    T* soft_ref = static_cast<T*>(ws);
    T* soft_inv = soft_ref + pixels;
    const int rc = launch_scm_forward<T>(d, x, w, alpha, beta, nullptr, soft_ref, soft_inv, stream);
    if (rc != MC_OK) return rc;
    if (sizeof(T) == 4 && d.kH == d.kW)
    {
        if (d.kW == 3) return launch_smorph_backward<T, 3, 3>(d, x, w, alpha, y, nullptr, gy, gx, gw, galpha, stream, beta, soft_ref, soft_inv, gbeta);
        if (d.kW == 5) return launch_smorph_backward<T, 5, 5>(d, x, w, alpha, y, nullptr, gy, gx, gw, galpha, stream, beta, soft_ref, soft_inv, gbeta);
        if (d.kW == 7) return launch_smorph_backward<T, 7, 7>(d, x, w, alpha, y, nullptr, gy, gx, gw, galpha, stream, beta, soft_ref, soft_inv, gbeta);
    }
    return dispatch_kernel_width(d.kH, d.kW, [&](auto kw) {
        constexpr int KW = decltype(kw)::value;
        return launch_smorph_backward<T, 0, KW>(d, x, w, alpha, y, nullptr, gy, gx, gw, galpha, stream, beta, soft_ref, soft_inv, gbeta);
    });
}

}  // namespace mc

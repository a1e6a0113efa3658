// Instantiates mc::morpho_forward<MC_T>; included by morpho_forward_f32.cu / _f64.cu.
#include <type_traits>

#include "dispatch.cuh"
#include "morpho_forward.cuh"

namespace mc
{

template <>
int morpho_forward<MC_T>(const mc_desc& d, const MC_T* x, const MC_T* w, MC_T* y, int32_t* idx, cudaStream_t stream)
{
    using T = MC_T;
    constexpr int WIDE = sizeof(T) == 4 ? 4 : 2;
    const int ob = output_block<T>(d);
    return dispatch_kernel_width(d.kH, d.kW, [&](auto kw) {
        constexpr int KW = decltype(kw)::value;
        if (d.op == MC_OP_DILATION)
            return ob == 1 ? launch_forward<T, false, KW, 1>(d, x, w, y, idx, stream) : launch_forward<T, false, KW, WIDE>(d, x, w, y, idx, stream);
        return ob == 1 ? launch_forward<T, true, KW, 1>(d, x, w, y, idx, stream) : launch_forward<T, true, KW, WIDE>(d, x, w, y, idx, stream);
    });
}

}  // namespace mc

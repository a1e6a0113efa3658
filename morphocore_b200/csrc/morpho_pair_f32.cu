// The fused dilation + erosion forward pass (float only).
#include <cmath>

#include "dispatch.cuh"
#include "morpho_pair.cuh"

namespace mc
{

int morpho_pair_forward(const mc_desc& d, const float* x, const float* w, float* y_dilation, float* y_erosion, cudaStream_t stream)
{
    if (d.kH != d.kW || (d.kH != 3 && d.kH != 5 && d.kH != 7)) return MC_ERR_UNSUPPORTED;
    if (d.weight_batch_stride != 0) return MC_ERR_UNSUPPORTED;                        // per-sample structuring elements: each pass draws its own
    if (d.pad_kind == MC_PAD_FILL && !std::isfinite(d.fill)) return MC_ERR_UNSUPPORTED;   // the geodesic border differs between the two passes
    const bool single = d.merge == MC_MERGE_IDENTITY || d.Co < 2;
    auto run = [&](auto kw) {
        constexpr int KW = decltype(kw)::value;
        return single ? launch_pair_forward<KW, 1>(d, x, w, y_dilation, y_erosion, stream) : launch_pair_forward<KW, 2>(d, x, w, y_dilation, y_erosion, stream);
    };
    if (d.kH == 3) return run(std::integral_constant<int, 3>{});
    if (d.kH == 5) return run(std::integral_constant<int, 5>{});
    return run(std::integral_constant<int, 7>{});
}

}  // namespace mc

// Runtime shape -> template instantiation switches shared by the per-dtype translation units.
#pragma once
#include "common.cuh"

namespace mc
{

/// Call f(std::integral_constant<int, K>) with the compiled size of a square K x K structuring element
/// (3, 5, 7 or 11), or 0 for any other shape, which takes the any-size path.
template <typename F>
inline int dispatch_kernel_width(int kh, int kw, F f)
{
    switch (kh == kw ? kw : 0)
    {
        case 3: return f(std::integral_constant<int, 3>{});
        case 5: return f(std::integral_constant<int, 5>{});
        case 7: return f(std::integral_constant<int, 7>{});
        case 11: return f(std::integral_constant<int, 11>{});
        default: return f(std::integral_constant<int, 0>{});
    }
}

/// Output channels a thread keeps in registers: sharing the window segments between 4 (float) or 2
/// (double) channels once there are enough of them; identity pairs each channel with itself.
template <typename T>
inline int output_block(const mc_desc& d)
{
    if (d.merge == MC_MERGE_IDENTITY) return 1;
    if (sizeof(T) == 4) return d.Co >= 3 ? 4 : 1;
    return d.Co >= 2 ? 2 : 1;
}

}  // namespace mc

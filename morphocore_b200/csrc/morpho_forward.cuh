// Forward dilation / erosion tile kernel with the fused channel merge.
//
// Replaces the reference's morpho_forward_kernel (morphocore/functional/csrc/cuda/morpho_op_kernels.cuh:339-465)
// with a new design: a CTA owns (batch element, group of OB output channels, 64 x 32 tile); it stages a
// chunk of input-channel windows in shared memory, and every thread keeps an OB x 2 x 4 block of running
// extrema in registers while the taps stream over 128-bit row segments. Two taps cost two adds and ONE
// three-input max/min (an sm_100 instruction), so the inner loop issues 1.5 instructions per tap.
//
// Bit-exactness with the reference CPU path: max/min are exact and order independent, so the per-channel
// extremum equals the reference's strict-compare scan; channels are merged sequentially i = 0..Ci-1 from
// the same initial values with the same std::max / std::min / + semantics
// (csrc/cpp/morpho_merge_policy.hpp:10-86, csrc/cpp/morpho_op_cpu_kernels.hxx:365-395). Erosion stores the
// negated structuring element, x + (-w) being the same IEEE operation as x - w.
#pragma once
#include "common.cuh"
#include "tma.cuh"

namespace mc
{

#ifndef MC_PACKED_ADD
#define MC_PACKED_ADD 1
#endif
/// Use the packed add.f32x2 of sm_100 in the float tap loop.
constexpr bool PACKED_ADD = MC_PACKED_ADD != 0;

template <typename T>
struct ForwardArgs
{
    Geometry g;
    const T* x;
    const T* w;
    T* y;
    int32_t* idx;
    int merge;
    T fill;
    int o_groups;
    int chunk;      // input channels staged per barrier
    bool vec_store; // y rows are 16-byte aligned
    unsigned int* errors;  // counter of timed-out waits
    uint64_t wait_limit_ns; // bound of one wait on a TMA copy
};

template <int OB, typename T>
__device__ __forceinline__ void load_weights(T (&dst)[OB], const T* src)
{
    if constexpr ((OB * sizeof(T)) % 16 == 0)
    {   // callers pass a 16-byte aligned source whenever OB values fill whole vectors
        constexpr int PER = 16 / sizeof(T);
#pragma unroll
        for (int v = 0; v < OB / PER; v++) lds128(&dst[v * PER], src + v * PER);
    }
    else
    {
#pragma unroll
        for (int o = 0; o < OB; o++) dst[o] = src[o];
    }
}

/// Extremum over the structuring element of one staged channel, for the thread's OB x 2 x 4 block. The staged
/// structuring elements hold WS output channels per tap, of which the OB from `wk` on are used.
template <typename T, bool IS_MIN, int KW, int OB, bool PACKED, int WS = OB>
__device__ __forceinline__ void window_extremum(T (&acc)[OB][PATCH_H][PATCH_W], const T* __restrict__ win, const T* __restrict__ wk,
                                                const Geometry& g, int tx, int ty)
{
    if constexpr (KW > 0)
    {
        // Square KW x KW structuring element: kernel rows fully unrolled up to 7 x 7 (constant offsets, no
        // loop-carried register moves).
        constexpr int LEN = segment_len(KW, sizeof(T)), OFF = segment_offset(KW, sizeof(T));
        constexpr int STRIDE = window_stride(KW, sizeof(T));
        const T* base = win + (ty * PATCH_H) * STRIDE + tx * PATCH_W;
#pragma unroll(KW <= 7 ? KW : 1)
        for (int kh = 0; kh < KW; kh++)
        {
            T seg[PATCH_H][LEN];
#pragma unroll
            for (int rr = 0; rr < PATCH_H; rr++) load_segment<LEN>(seg[rr], base + (rr + KW - 1 - kh) * STRIDE);
            const T* wrow = wk + kh * KW * WS;
            if constexpr (sizeof(T) == 4 && PACKED && PACKED_ADD && OB % 2 == 0)
            {
                // Packed adds (add.f32x2) over PAIRS OF OUTPUT CHANNELS: (x, x) + (w[o], w[o + 1]). The structuring elements
                // are staged [tap][channel], so a pair of them is a register pair as loaded; only x has to be doubled, one
                // register move per window element and kernel row, shared by every tap and channel pair that reads it.
                float2 xx[PATCH_H][PATCH_W + KW - 1];
#pragma unroll
                for (int rr = 0; rr < PATCH_H; rr++)
#pragma unroll
                    for (int c = 0; c < PATCH_W + KW - 1; c++) xx[rr][c] = make_float2(seg[rr][OFF + c], seg[rr][OFF + c]);
#pragma unroll
                for (int kw = 0; kw + 1 < KW; kw += 2)
                {
                    T w0[OB], w1[OB];
                    load_weights<OB>(w0, wrow + kw * WS);
                    load_weights<OB>(w1, wrow + (kw + 1) * WS);
#pragma unroll
                    for (int o = 0; o < OB; o += 2)
                    {
                        const float2 wa = make_float2(w0[o], w0[o + 1]), wb = make_float2(w1[o], w1[o + 1]);
#pragma unroll
                        for (int rr = 0; rr < PATCH_H; rr++)
#pragma unroll
                            for (int j = 0; j < PATCH_W; j++)
                            {
                                const float2 va = __fadd2_rn(xx[rr][j + KW - 1 - kw], wa), vb = __fadd2_rn(xx[rr][j + KW - 2 - kw], wb);
                                acc[o][rr][j] = ext3<IS_MIN>(acc[o][rr][j], va.x, vb.x);
                                acc[o + 1][rr][j] = ext3<IS_MIN>(acc[o + 1][rr][j], va.y, vb.y);
                            }
                    }
                }
                if constexpr (KW & 1)
                {
                    T w0[OB];
                    load_weights<OB>(w0, wrow + (KW - 1) * WS);
#pragma unroll
                    for (int o = 0; o < OB; o += 2)
                    {
                        const float2 wa = make_float2(w0[o], w0[o + 1]);
#pragma unroll
                        for (int rr = 0; rr < PATCH_H; rr++)
#pragma unroll
                            for (int j = 0; j < PATCH_W; j++)
                            {
                                const float2 va = __fadd2_rn(xx[rr][j], wa);
                                acc[o][rr][j] = ext2<IS_MIN>(acc[o][rr][j], va.x);
                                acc[o + 1][rr][j] = ext2<IS_MIN>(acc[o + 1][rr][j], va.y);
                            }
                    }
                }
            }
            else if constexpr (sizeof(T) == 4 && PACKED && PACKED_ADD)
            {
                // Packed adds (add.f32x2): two adjacent pixels per instruction. Pixel pairs start at segment
                // element OFF + j + KW-1-kw (j = 0, 2); even starts are register pairs as loaded, odd starts
                // come from a copy of the segment shifted by one element.
                float2 even[PATCH_H][LEN / 2], odd[PATCH_H][LEN / 2];
#pragma unroll
                for (int rr = 0; rr < PATCH_H; rr++)
#pragma unroll
                    for (int i = 0; i < LEN / 2; i++)
                    {
                        even[rr][i] = make_float2(seg[rr][2 * i], seg[rr][2 * i + 1]);
                        odd[rr][i] = make_float2(seg[rr][2 * i + 1], seg[rr][2 * i + 2 < LEN ? 2 * i + 2 : 2 * i + 1]);
                    }
                auto pair_at = [&](int rr, int start) { return (start & 1) ? odd[rr][start >> 1] : even[rr][start >> 1]; };
#pragma unroll
                for (int kw = 0; kw + 1 < KW; kw += 2)
                {
                    T w0[OB], w1[OB];
                    load_weights<OB>(w0, wrow + kw * WS);
                    load_weights<OB>(w1, wrow + (kw + 1) * WS);
#pragma unroll
                    for (int o = 0; o < OB; o++)
                    {
                        const float2 wa = make_float2(w0[o], w0[o]), wb = make_float2(w1[o], w1[o]);
#pragma unroll
                        for (int rr = 0; rr < PATCH_H; rr++)
#pragma unroll
                            for (int j = 0; j < PATCH_W; j += 2)
                            {
                                const float2 va = __fadd2_rn(pair_at(rr, OFF + j + KW - 1 - kw), wa);
                                const float2 vb = __fadd2_rn(pair_at(rr, OFF + j + KW - 2 - kw), wb);
                                acc[o][rr][j] = ext3<IS_MIN>(acc[o][rr][j], va.x, vb.x);
                                acc[o][rr][j + 1] = ext3<IS_MIN>(acc[o][rr][j + 1], va.y, vb.y);
                            }
                    }
                }
                if constexpr (KW & 1)
                {
                    T w0[OB];
                    load_weights<OB>(w0, wrow + (KW - 1) * WS);
#pragma unroll
                    for (int o = 0; o < OB; o++)
                    {
                        const float2 wa = make_float2(w0[o], w0[o]);
#pragma unroll
                        for (int rr = 0; rr < PATCH_H; rr++)
#pragma unroll
                            for (int j = 0; j < PATCH_W; j += 2)
                            {
                                const float2 va = __fadd2_rn(pair_at(rr, OFF + j), wa);
                                acc[o][rr][j] = ext2<IS_MIN>(acc[o][rr][j], va.x);
                                acc[o][rr][j + 1] = ext2<IS_MIN>(acc[o][rr][j + 1], va.y);
                            }
                    }
                }
            }
            else
            {
#pragma unroll
            for (int kw = 0; kw + 1 < KW; kw += 2)
            {
                T w0[OB], w1[OB];
                load_weights<OB>(w0, wrow + kw * WS);
                load_weights<OB>(w1, wrow + (kw + 1) * WS);
#pragma unroll
                for (int o = 0; o < OB; o++)
#pragma unroll
                    for (int rr = 0; rr < PATCH_H; rr++)
#pragma unroll
                        for (int j = 0; j < PATCH_W; j++)
                            acc[o][rr][j] = ext3<IS_MIN>(acc[o][rr][j], seg[rr][OFF + j + KW - 1 - kw] + w0[o], seg[rr][OFF + j + KW - 2 - kw] + w1[o]);
            }
            if constexpr (KW & 1)
            {
                T w0[OB];
                load_weights<OB>(w0, wrow + (KW - 1) * WS);
#pragma unroll
                for (int o = 0; o < OB; o++)
#pragma unroll
                    for (int rr = 0; rr < PATCH_H; rr++)
#pragma unroll
                        for (int j = 0; j < PATCH_W; j++) acc[o][rr][j] = ext2<IS_MIN>(acc[o][rr][j], seg[rr][OFF + j] + w0[o]);
            }
            }
        }
    }
    else
    {
        // Any structuring element size: scalar window reads.
        for (int kh = 0; kh < g.kH; kh++)
        {
            const T* row0 = win + (ty * PATCH_H + g.kH - 1 - kh) * g.win_stride + tx * PATCH_W;
            for (int kw = 0; kw < g.kW; kw++)
            {
                T w0[OB];
                load_weights<OB>(w0, wk + (kh * g.kW + kw) * WS);
#pragma unroll
                for (int rr = 0; rr < PATCH_H; rr++)
#pragma unroll
                    for (int j = 0; j < PATCH_W; j++)
                    {
                        const T xv = row0[rr * g.win_stride + g.seg_off + j + g.kW - 1 - kw];
#pragma unroll
                        for (int o = 0; o < OB; o++) acc[o][rr][j] = ext2<IS_MIN>(acc[o][rr][j], xv + w0[o]);
                    }
            }
        }
    }
}

/// Stage the structuring elements of channels [c0, c0 + cc) for output channels [o0, o0 + OB) as
/// [channel][tap][OB], negated for erosion and zero for output channels past Co.
template <typename T, bool IS_MIN, int OB>
__device__ __forceinline__ void stage_weights(T* __restrict__ sw, const T* __restrict__ w, const Geometry& g, int o0, int c0, int cc)
{
    const int taps = g.taps();
    const int wci = g.identity ? 1 : g.Ci;
    for (int e = threadIdx.x; e < cc * taps * OB; e += THREADS)
    {
        const int o = e % OB, k = (e / OB) % taps, c = e / (OB * taps);
        T v = 0;
        if (o0 + o < g.Co)
        {
            const int wi = g.identity ? 0 : c0 + c;
            v = __ldg(w + (static_cast<int64_t>(o0 + o) * wci + wi) * taps + k);
        }
        sw[e] = IS_MIN ? -v : v;
    }
}

/// Winning channels of the OB output channels of one pixel, packed into 32-bit words: FIELD bits per channel (8 when
/// there are at most 256 input channels, else 16). Replacing one field is a single byte-permute instruction, and a
/// pixel costs one or two registers instead of OB: that is what lets the index-tracking kernel keep the packed adds.
template <int OB, int FIELD> struct PackedWinners
{
    static constexpr int PER = 32 / FIELD, WORDS = (OB + PER - 1) / PER;
    unsigned int word[WORDS];
    __device__ __forceinline__ void clear()
    {
#pragma unroll
        for (int i = 0; i < WORDS; i++) word[i] = 0u;
    }
    /// Field `o` (a compile-time constant after unrolling) := channel.
    __device__ __forceinline__ void set(int o, unsigned int channel)
    {
        const int f = o % PER;
        unsigned int selector;
        if (FIELD == 8) selector = f == 0 ? 0x3214u : (f == 1 ? 0x3240u : (f == 2 ? 0x3410u : 0x4210u));
        else selector = f == 0 ? 0x3254u : 0x5410u;
        word[o / PER] = __byte_perm(word[o / PER], channel, selector);
    }
    __device__ __forceinline__ int get(int o) const { return static_cast<int>((word[o / PER] >> (FIELD * (o % PER))) & ((1u << FIELD) - 1u)); }
};

/// TRACK: 0 = no winner index, 8 / 16 = track the winning channel of MAX / MIN merges in fields of that many bits.
template <typename T, bool IS_MIN, int KW, int OB, int TRACK, bool USE_TMA>
__global__ void __launch_bounds__(THREADS, (sizeof(T) == 8 && (TRACK || OB > 1)) ? 1 : 2)
    morpho_forward_kernel(const ForwardArgs<T> a, const __grid_constant__ CUtensorMap tmap)
{
    extern __shared__ __align__(128) unsigned char smem_raw[];
    const Geometry& g = a.g;
    // Layout: [2 mbarriers][pad to 128][stage 0 windows][stage 1 windows][weights]; a single stage without TMA.
    uint64_t* full = reinterpret_cast<uint64_t*>(smem_raw);
    const int stage_elems = (a.chunk * g.window_elems() * static_cast<int>(sizeof(T)) + 127) / 128 * 128 / static_cast<int>(sizeof(T));
    T* sx0 = reinterpret_cast<T*>(smem_raw + 128);
    T* sw = sx0 + (USE_TMA ? 2 : 1) * stage_elems;

    const int tiles = g.tiles_x * g.tiles_y;
    const int og = blockIdx.x % a.o_groups;
    const int tile = (blockIdx.x / a.o_groups) % tiles;
    const int b = blockIdx.x / (a.o_groups * tiles);
    const int tile_h0 = (tile / g.tiles_x) * TILE_H, tile_w0 = (tile % g.tiles_x) * TILE_W;
    // A tile whose right half is outside the image is split between the warps of each warp row: both take the
    // left block and half of the output channels (thread_patch_split); slots 0 .. o_count - 1 of the register
    // arrays then hold channels o0 + o_base + slot.
    int tx, ty, half;
    bool warp_live, split;
    thread_patch_split(tile_h0, tile_w0, g.H, g.W, OB >= 2, tx, ty, warp_live, split, half);
    const int o_count = split ? OB / 2 : OB, o_base = half * (OB / 2);
    const int o0 = og * OB;
    const int64_t plane = g.plane();
    const T* xb = a.x + static_cast<int64_t>(b) * g.Ci * plane;
    const T* wb = a.w + static_cast<int64_t>(b) * g.weight_batch_stride;

    const int channels = g.identity ? 1 : g.Ci;
    const T op_init = IS_MIN ? Limits<T>::inf() : -Limits<T>::inf();
    const T merge_init = a.merge == MC_MERGE_MAX ? -Limits<T>::max() : (a.merge == MC_MERGE_MIN ? Limits<T>::max() : T(0));

    T merged[OB][PATCH_H][PATCH_W];
    PackedWinners<OB, TRACK ? TRACK : 8> winner[TRACK ? PATCH_H : 1][TRACK ? PATCH_W : 1];
#pragma unroll
    for (int rr = 0; rr < PATCH_H; rr++)
#pragma unroll
        for (int j = 0; j < PATCH_W; j++)
        {
            if constexpr (TRACK != 0) winner[rr][j].clear();
#pragma unroll
            for (int o = 0; o < OB; o++) merged[o][rr][j] = merge_init;
        }

    // TMA: chunk n + 1 is copied into the other stage while chunk n is computed. The copy zero fills
    // outside the image; tiles whose window leaves the image patch those elements for the other border rules.
    const uint32_t stage_bytes = static_cast<uint32_t>(a.chunk) * g.window_elems() * sizeof(T);
    const int first_channel = g.identity ? o0 : 0;
    const bool fix_border = USE_TMA && (g.replicate || a.fill != T(0)) && window_leaves_image(g, tile_h0, tile_w0);
    auto issue = [&](int n) {
        uint64_t* bar = full + (n & 1);
        mbar_expect_tx(bar, stage_bytes);
        tma_load_4d(sx0 + (n & 1) * stage_elems, &tmap, bar, tile_w0 - g.halo_left(), tile_h0 - g.halo_top(), first_channel + n * a.chunk, b);
    };
    if constexpr (USE_TMA)
    {
        if (threadIdx.x == 0)
        {
            mbar_init(full, 1);
            mbar_init(full + 1, 1);
            mbar_fence_init();
        }
        __syncthreads();
        if (threadIdx.x == 0) issue(0);
    }

    int n = 0;
    for (int c0 = 0; c0 < channels; c0 += a.chunk, n++)
    {
        const int cc = min(a.chunk, channels - c0);
        T* sx = sx0 + (USE_TMA ? (n & 1) * stage_elems : 0);
        __syncthreads();
        if constexpr (USE_TMA)
        {
            if (threadIdx.x == 0 && c0 + a.chunk < channels)
            {
                fence_async_smem();
                issue(n + 1);
            }
        }
        else
        {
            for (int c = 0; c < cc; c++)
            {
                const int ci = g.identity ? o0 : c0 + c;
                load_window(sx + c * g.window_elems(), xb + static_cast<int64_t>(ci) * plane, g, tile_h0, tile_w0, a.fill);
            }
        }
        stage_weights<T, IS_MIN, OB>(sw, wb, g, o0, c0, cc);
        if constexpr (USE_TMA)
        {
            if (!mbar_wait(full + (n & 1), (n >> 1) & 1, a.wait_limit_ns))
            {
                if (threadIdx.x == 0 && a.errors != nullptr) atomicAdd(a.errors, 1u);
                return;  // every thread of the CTA waits on the same barrier and gives up together
            }
            if (fix_border) fix_window_border(sx, xb + static_cast<int64_t>(first_channel + c0) * plane, plane, cc, g, tile_h0, tile_w0, a.fill);
        }
        __syncthreads();

        for (int c = 0; c < cc && warp_live; c++)
        {
            T acc[OB][PATCH_H][PATCH_W];
#pragma unroll
            for (int o = 0; o < OB; o++)
#pragma unroll
                for (int rr = 0; rr < PATCH_H; rr++)
#pragma unroll
                    for (int j = 0; j < PATCH_W; j++) acc[o][rr][j] = op_init;

            bool done = false;
            if constexpr (OB >= 2)
            {
                if (split)
                {
                    auto& lower = reinterpret_cast<T (&)[OB / 2][PATCH_H][PATCH_W]>(acc);
                    window_extremum<T, IS_MIN, KW, OB / 2, true, OB>(lower, sx + c * g.window_elems(), sw + c * g.taps() * OB + o_base, g, tx, ty);
                    done = true;
                }
            }
            if (!done) window_extremum<T, IS_MIN, KW, OB, true>(acc, sx + c * g.window_elems(), sw + c * g.taps() * OB, g, tx, ty);

            const int ci = c0 + c;
            // The merge mode is the same for every pixel: one switch around the pixel loops. A channel wins a MAX / MIN
            // merge when it is strictly better than the running value, which starts at the merge's initial value with
            // channel 0 as the winner (the reference's rule, csrc/cpp/morpho_op_cpu_kernels.hxx:358-360, 389-390).
            auto for_values = [&](auto f) {
#pragma unroll
                for (int o = 0; o < OB; o++)
                {
                    if (o >= o_count) break;
#pragma unroll
                    for (int rr = 0; rr < PATCH_H; rr++)
#pragma unroll
                        for (int j = 0; j < PATCH_W; j++) f(merged[o][rr][j], acc[o][rr][j], winner[TRACK ? rr : 0][TRACK ? j : 0], o);
                }
            };
            if (a.merge == MC_MERGE_MAX)
                for_values([&](T& m, T v, auto& win, int o) {
                    if constexpr (TRACK != 0)
                        if (v > m) win.set(o, static_cast<unsigned int>(ci));
                    m = m < v ? v : m;
                });
            else if (a.merge == MC_MERGE_MIN)
                for_values([&](T& m, T v, auto& win, int o) {
                    if constexpr (TRACK != 0)
                        if (v < m) win.set(o, static_cast<unsigned int>(ci));
                    m = v < m ? v : m;
                });
            else if (a.merge == MC_MERGE_IDENTITY) for_values([](T& m, T v, auto&, int) { m = v; });
            else for_values([](T& m, T v, auto&, int) { m = m + v; });
        }
    }

    const T divisor = static_cast<T>(g.Ci);
#pragma unroll
    for (int o = 0; o < OB; o++)
    {
        if (o >= o_count || !warp_live || o0 + o_base + o >= g.Co) continue;
#pragma unroll
        for (int rr = 0; rr < PATCH_H; rr++)
        {
            const int h = tile_h0 + ty * PATCH_H + rr;
            const int w0 = tile_w0 + tx * PATCH_W;
            if (h >= g.H || w0 >= g.W) continue;
            T out[PATCH_W];
#pragma unroll
            for (int j = 0; j < PATCH_W; j++) out[j] = a.merge == MC_MERGE_AVERAGE ? merged[o][rr][j] / divisor : merged[o][rr][j];
            const int64_t row = ((static_cast<int64_t>(b) * g.Co + o0 + o_base + o) * g.H + h) * g.W;
            if (a.y != nullptr)
            {
                if (a.vec_store && w0 + PATCH_W <= g.W)
                {
                    if constexpr (sizeof(T) == 4)
                        *reinterpret_cast<float4*>(a.y + row + w0) = make_float4(out[0], out[1], out[2], out[3]);
                    else
                    {
                        *reinterpret_cast<double2*>(a.y + row + w0) = make_double2(out[0], out[1]);
                        *reinterpret_cast<double2*>(a.y + row + w0 + 2) = make_double2(out[2], out[3]);
                    }
                }
                else
                {
#pragma unroll
                    for (int j = 0; j < PATCH_W; j++)
                        if (w0 + j < g.W) a.y[row + w0 + j] = out[j];
                }
            }
            if constexpr (TRACK != 0)
            {
                // Only the winning channel is known here; the tap search kernels add the tap.
#pragma unroll
                for (int j = 0; j < PATCH_W; j++)
                    if (w0 + j < g.W) a.idx[row + w0 + j] = winner[rr][j].get(o) << 16;
            }
        }
    }
}

/// Second step of the winner index of MAX / MIN merges: one thread per output pixel scans the winning
/// channel alone for its first extremal tap, with the reference's strict comparison from the initial
/// value in kh-major, kw order (index 0 when nothing beats it), and completes idx to (channel << 16) | tap.
/// Running it as its own launch keeps every SM full of independent gathers instead of serialising them at
/// the end of the tile kernel.
template <typename T, bool IS_MIN>
__global__ void __launch_bounds__(THREADS) morpho_find_tap_kernel(const ForwardArgs<T> a, int64_t total)
{
    const Geometry& g = a.g;
    const int64_t plane = g.plane();
    const int taps = g.taps();
    const T op_init = IS_MIN ? Limits<T>::inf() : -Limits<T>::inf();
    for (int64_t at = static_cast<int64_t>(blockIdx.x) * THREADS + threadIdx.x; at < total; at += static_cast<int64_t>(gridDim.x) * THREADS)
    {
        const int w = static_cast<int>(at % g.W), h = static_cast<int>((at / g.W) % g.H);
        const int o = static_cast<int>((at / plane) % g.Co), b = static_cast<int>(at / (plane * g.Co));
        int ch = a.idx[at] >> 16;
        ch = min(max(ch, 0), g.Ci - 1);
        const T* xp = a.x + (static_cast<int64_t>(b) * g.Ci + ch) * plane;
        const T* wk = a.w + static_cast<int64_t>(b) * g.weight_batch_stride + (static_cast<int64_t>(o) * g.Ci + ch) * taps;
        T best = op_init;
        int arg = 0;
        const bool inside = h - (g.kH - 1 - g.pH) >= 0 && h + g.pH < g.H && w - (g.kW - 1 - g.pW) >= 0 && w + g.pW < g.W;
        if (inside)
        {
            for (int kh = 0; kh < g.kH; kh++)
            {
                const T* row = xp + static_cast<int64_t>(h + g.pH - kh) * g.W + w + g.pW;
                for (int kw = 0; kw < g.kW; kw++)
                {
                    const T wv = __ldg(wk + kh * g.kW + kw);
                    const T xv = __ldg(row - kw);
                    const T v = IS_MIN ? xv - wv : xv + wv;
                    if (strictly_better<IS_MIN>(v, best))
                    {
                        best = v;
                        arg = kh * g.kW + kw;
                    }
                }
            }
        }
        else
        {
            for (int kh = 0; kh < g.kH; kh++)
                for (int kw = 0; kw < g.kW; kw++)
                {
                    const T xv = read_border(xp, g, h + g.pH - kh, w + g.pW - kw, a.fill);
                    const T wv = __ldg(wk + kh * g.kW + kw);
                    const T v = IS_MIN ? xv - wv : xv + wv;
                    if (strictly_better<IS_MIN>(v, best))
                    {
                        best = v;
                        arg = kh * g.kW + kw;
                    }
                }
        }
        a.idx[at] = (ch << 16) | arg;
    }
}

/// Tile of the tiled tap search: 16 x 16 output pixels, one per thread.
constexpr int FIND_TILE = 16;

/// The second step of the winner index for the specialised square widths, without gathers from global memory. The
/// one-pixel-per-thread scan above reads 25 (5 x 5) scattered elements of a different channel plane per lane: at 64
/// channels that is an L2 gather of a few hundred bytes per output pixel and takes half as long as the whole
/// forward pass. Here a CTA owns (batch element, 16 x 16 tile), stages the windows of a group of input channels
/// (as many as fit in shared memory; every channel for 64 of them at 5 x 5) and then walks ALL output channels:
/// a thread looks up its pixel's winning channel and scans that channel's window in shared memory, with the
/// output channel's structuring elements staged beside it. The input is read from global memory once per group
/// (plus the halo), the indices once, and every scan is the reference's strict comparison in kh-major, kw order.
template <typename T, bool IS_MIN, int KW>
__global__ void __launch_bounds__(FIND_TILE * FIND_TILE) morpho_find_tap_tiled_kernel(const ForwardArgs<T> a, int group)
{
    static_assert(KW > 0, "specialised widths only");
    constexpr int WIN = FIND_TILE + KW - 1, TAPS = KW * KW, NT = FIND_TILE * FIND_TILE;
    extern __shared__ __align__(16) unsigned char smem_raw[];
    const Geometry& g = a.g;
    T* sx = reinterpret_cast<T*>(smem_raw);            // [group][WIN][WIN]
    T* sw = sx + group * WIN * WIN;                    // [group][TAPS] of the current output channel

    const int tiles_x = (g.W + FIND_TILE - 1) / FIND_TILE;
    const int tile_h0 = (blockIdx.x / tiles_x) * FIND_TILE, tile_w0 = (blockIdx.x % tiles_x) * FIND_TILE;
    const int b = blockIdx.y;
    const int tx = threadIdx.x % FIND_TILE, ty = threadIdx.x / FIND_TILE;
    const int h = tile_h0 + ty, w = tile_w0 + tx;
    const bool live = h < g.H && w < g.W;
    const int64_t plane = g.plane();
    const T op_init = IS_MIN ? Limits<T>::inf() : -Limits<T>::inf();
    const T* wb = a.w + static_cast<int64_t>(b) * g.weight_batch_stride;
    const int row0 = tile_h0 - g.halo_top(), col0 = tile_w0 - halo_left_of(KW);

    for (int c0 = 0; c0 < g.Ci; c0 += group)
    {
        const int cc = min(group, g.Ci - c0);
        __syncthreads();   // the previous group's windows are no longer read
        for (int e = threadIdx.x; e < cc * WIN * WIN; e += NT)
        {
            const int c = e / (WIN * WIN), rest = e - c * (WIN * WIN), r = rest / WIN, col = rest - r * WIN;
            const int iy = row0 + r, ix = col0 + col;
            const bool in = iy >= 0 && iy < g.H && ix >= 0 && ix < g.W;
            const T* src = a.x + (static_cast<int64_t>(b) * g.Ci + c0 + c) * plane;
            if (in || g.replicate) cp_async_element(sx + e, src + static_cast<int64_t>(min(max(iy, 0), g.H - 1)) * g.W + min(max(ix, 0), g.W - 1));
            else sx[e] = a.fill;
        }
        cp_async_wait_all();
        const int64_t at0 = ((static_cast<int64_t>(b) * g.Co) * g.H + h) * g.W + w;
        int next = live ? a.idx[at0] : 0;   // the winner of the next output channel is fetched one iteration ahead
        for (int o = 0; o < g.Co; o++)
        {
            __syncthreads();   // windows landed (first pass); the previous output channel's structuring elements are no longer read
            for (int e = threadIdx.x; e < cc * TAPS; e += NT) sw[e] = __ldg(wb + (static_cast<int64_t>(o) * g.Ci + c0) * TAPS + e);
            const int packed = next;
            if (live && o + 1 < g.Co) next = a.idx[at0 + static_cast<int64_t>(o + 1) * plane];
            __syncthreads();
            if (!live) continue;
            const int64_t at = at0 + static_cast<int64_t>(o) * plane;
            int ch = packed >> 16;
            ch = min(max(ch, 0), g.Ci - 1);
            if (ch < c0 || ch >= c0 + cc) continue;
            const T* win = sx + (ch - c0) * (WIN * WIN) + ty * WIN + tx;
            const T* wk = sw + (ch - c0) * TAPS;
            T best = op_init;
            int arg = 0;
#pragma unroll
            for (int kh = 0; kh < KW; kh++)
#pragma unroll
                for (int kw = 0; kw < KW; kw++)
                {
                    const T xv = win[(KW - 1 - kh) * WIN + KW - 1 - kw], wv = wk[kh * KW + kw];
                    const T v = IS_MIN ? xv - wv : xv + wv;
                    if (strictly_better<IS_MIN>(v, best))
                    {
                        best = v;
                        arg = kh * KW + kw;
                    }
                }
            a.idx[at] = (ch << 16) | arg;
        }
    }
}

template <typename T> struct ForwardPlan
{
    int chunk;
    size_t smem;
};

/// Channels staged per barrier: as many as fit in about 96 KiB (two CTAs per SM), at most 8; `stages`
/// window buffers (2 with TMA double buffering) plus one buffer of structuring elements.
template <typename T>
inline bool plan_forward(const Geometry& g, int ob, int stages, ForwardPlan<T>& plan)
{
    const size_t window = static_cast<size_t>(g.window_elems()) * sizeof(T), weights = static_cast<size_t>(g.taps()) * ob * sizeof(T);
    const size_t per_channel = stages * window + weights;
    const size_t fixed = 128 + stages * 128;
    if (per_channel + fixed > MAX_SHARED_BYTES) return false;
    const int channels = g.identity ? 1 : g.Ci;
    int chunk = static_cast<int>((96 * 1024 - fixed) / per_channel);
    chunk = chunk < 1 ? 1 : (chunk > 8 ? 8 : chunk);
    chunk = chunk > channels ? channels : chunk;
    plan.chunk = chunk;
    plan.smem = fixed + per_channel * chunk;
    return true;
}

template <typename T, bool IS_MIN, int KW, int OB, int TRACK, bool USE_TMA>
int launch_forward_variant(const ForwardArgs<T>& a, const CUtensorMap& tmap, int64_t blocks, size_t smem, cudaStream_t stream)
{
    auto kernel = morpho_forward_kernel<T, IS_MIN, KW, OB, TRACK, USE_TMA>;
    if (!allow_shared(kernel, smem))
    {
        set_last_error("cannot opt in to %zu bytes of shared memory", smem);
        return MC_ERR_UNSUPPORTED;
    }
    kernel<<<static_cast<unsigned>(blocks), THREADS, smem, stream>>>(a, tmap);
    return check_launch("morpho_forward_kernel");
}

template <typename T, bool IS_MIN, int KW, int OB>
int launch_forward(const mc_desc& d, const T* x, const T* w, T* y, int32_t* idx, cudaStream_t stream)
{
    const Geometry g = make_geometry(d, sizeof(T));
    ForwardArgs<T> a;
    a.g = g; a.x = x; a.w = w; a.y = y; a.idx = idx; a.merge = d.merge; a.fill = static_cast<T>(d.fill);
    a.o_groups = (d.Co + OB - 1) / OB;
    a.vec_store = (d.W % 4 == 0) && (reinterpret_cast<uintptr_t>(y) % 16 == 0);
    const int64_t blocks = static_cast<int64_t>(g.tiles_x) * g.tiles_y * a.o_groups * d.B;
    if (blocks > 0x7fffffffLL)
    {
        set_last_error("too many tiles for one launch");
        return MC_ERR_UNSUPPORTED;
    }
    const bool track = idx != nullptr;
    a.errors = device_error_counter();
    a.wait_limit_ns = wait_limit_ns();

    // TMA staging when the tensor can be described by a tensor map (16-byte row pitch and base).
    ForwardPlan<T> plan;
    CUtensorMap tmap{};
    int rc;
    if (plan_forward<T>(g, OB, 2, plan)
        && make_window_tensor_map(&tmap, x, sizeof(T), d.B, d.Ci, d.H, d.W, g.win_stride, g.win_rows, plan.chunk))
    {
        a.chunk = plan.chunk;
        rc = !track ? launch_forward_variant<T, IS_MIN, KW, OB, 0, true>(a, tmap, blocks, plan.smem, stream)
             : (d.Ci <= 256 ? launch_forward_variant<T, IS_MIN, KW, OB, 8, true>(a, tmap, blocks, plan.smem, stream)
                            : launch_forward_variant<T, IS_MIN, KW, OB, 16, true>(a, tmap, blocks, plan.smem, stream));
    }
    else
    {
        if (!plan_forward<T>(g, OB, 1, plan))
        {
            set_last_error("structuring element %dx%d too large for shared memory", d.kH, d.kW);
            return MC_ERR_UNSUPPORTED;
        }
        a.chunk = plan.chunk;
        rc = !track ? launch_forward_variant<T, IS_MIN, KW, OB, 0, false>(a, tmap, blocks, plan.smem, stream)
             : (d.Ci <= 256 ? launch_forward_variant<T, IS_MIN, KW, OB, 8, false>(a, tmap, blocks, plan.smem, stream)
                            : launch_forward_variant<T, IS_MIN, KW, OB, 16, false>(a, tmap, blocks, plan.smem, stream));
    }
    if (rc != MC_OK || !track) return rc;
    if constexpr (KW > 0)
    {
        // Tiled search from shared memory when a useful group of channel windows fits (two CTAs per SM).
        constexpr size_t WINDOW = static_cast<size_t>(FIND_TILE + KW - 1) * (FIND_TILE + KW - 1) * sizeof(T);
        constexpr size_t PER_CHANNEL = WINDOW + static_cast<size_t>(KW) * KW * sizeof(T);
        const int group = static_cast<int>(std::min<size_t>(d.Ci, (110 * 1024) / PER_CHANNEL));
        const int64_t tiles = static_cast<int64_t>((d.W + FIND_TILE - 1) / FIND_TILE) * ((d.H + FIND_TILE - 1) / FIND_TILE);
        auto tiled = morpho_find_tap_tiled_kernel<T, IS_MIN, KW>;
        if (group >= 8 && d.B <= 65535 && tiles <= 0x7fffffffLL && allow_shared(tiled, group * PER_CHANNEL))
        {
            tiled<<<dim3(static_cast<unsigned>(tiles), static_cast<unsigned>(d.B)), FIND_TILE * FIND_TILE, group * PER_CHANNEL, stream>>>(a, group);
            return check_launch("morpho_find_tap_tiled_kernel");
        }
    }
    const int64_t total = static_cast<int64_t>(d.B) * d.Co * d.H * d.W;
    const int64_t finder_blocks = std::min<int64_t>((total + THREADS - 1) / THREADS, 148LL * 64);
    morpho_find_tap_kernel<T, IS_MIN><<<static_cast<unsigned>(finder_blocks), THREADS, 0, stream>>>(a, total);
    return check_launch("morpho_find_tap_kernel");
}

}  // namespace mc

// Dilation AND erosion of one input with one structuring element in a single pass: the two halves of the reference's
// sigma_layer (morphocore/functional/sigma_layer.py:73-83: erosion(x, w) and dilation(x, w) blended by sigmoid(alpha)).
// Erosion receives the flipped structuring element (morphocore/functional/erosion.py:89), so tap k of a pixel yields the
// two candidates x_k + w[k] and x_k - w[K - 1 - k] from the SAME window element: staged as the pair (w[k], -w[K - 1 - k]),
// they are one packed add.f32x2 of (x, x), followed by a three-input max on the first lane and a three-input min on the
// second. The arithmetic is that of the two separate forward kernels, bit for bit; what the fusion saves is the second
// staging of the window and the second set of loads and register moves that bring a window element to the adds.
// float, square 3 x 3 / 5 x 5 / 7 x 7 structuring elements, TMA staging, every merge; no winner index (MAX / MIN merges
// that want one use the separate kernels) and no per-op fill value (the geodesic border differs between the two).
#pragma once

#include "morpho_forward.cuh"

namespace mc
{

struct PairForwardArgs
{
    Geometry g;
    const float* x;
    const float* w;
    float* y_dilation;
    float* y_erosion;
    int merge;
    float fill;
    int o_groups;
    int chunk;               // input channels staged per barrier
    int vec_store;
    unsigned int* errors;    // counter of timed-out waits
    uint64_t wait_limit_ns;  // bound of one wait on a TMA copy
};

/// Stage the structuring elements of channels [c0, c0 + cc) for output channels [o0, o0 + OB) as [channel][tap][OB]
/// pairs (w[k], -w[K - 1 - k]); zero for output channels past Co.
template <int OB>
__device__ __forceinline__ void stage_pair_weights(float2* __restrict__ sw, const float* __restrict__ w, const Geometry& g, int o0, int c0, int cc)
{
    const int taps = g.taps();
    const int wci = g.identity ? 1 : g.Ci;
    for (int e = threadIdx.x; e < cc * taps * OB; e += THREADS)
    {
        const int o = e % OB, k = (e / OB) % taps, c = e / (OB * taps);
        float2 v = make_float2(0.0f, 0.0f);
        if (o0 + o < g.Co)
        {
            const float* base = w + (static_cast<int64_t>(o0 + o) * wci + (g.identity ? 0 : c0 + c)) * taps;
            v = make_float2(__ldg(base + k), -__ldg(base + taps - 1 - k));
        }
        sw[e] = v;
    }
}

/// Both extrema over the structuring element of one staged channel for the thread's OBX x 2 x 4 block: acc.x is the
/// dilation's running maximum, acc.y the erosion's running minimum. WS output channels are staged per tap.
template <int KW, int OBX, int WS>
__device__ __forceinline__ void pair_window_extrema(float2 (&acc)[OBX][PATCH_H][PATCH_W], const float* __restrict__ win, const float2* __restrict__ wk,
                                                    int tx, int ty)
{
    constexpr int LEN = segment_len(KW, 4), OFF = segment_offset(KW, 4), STRIDE = window_stride(KW, 4);
    const float* base = win + (ty * PATCH_H) * STRIDE + tx * PATCH_W;
#pragma unroll
    for (int kh = 0; kh < KW; kh++)
    {
        float seg[PATCH_H][LEN];
#pragma unroll
        for (int rr = 0; rr < PATCH_H; rr++) load_segment<LEN>(seg[rr], base + (rr + KW - 1 - kh) * STRIDE);
        float2 xx[PATCH_H][PATCH_W + KW - 1];
#pragma unroll
        for (int rr = 0; rr < PATCH_H; rr++)
#pragma unroll
            for (int c = 0; c < PATCH_W + KW - 1; c++) xx[rr][c] = make_float2(seg[rr][OFF + c], seg[rr][OFF + c]);
        const float2* wrow = wk + kh * KW * WS;
#pragma unroll
        for (int kw = 0; kw + 1 < KW; kw += 2)
#pragma unroll
            for (int o = 0; o < OBX; o++)
            {
                const float2 wa = wrow[kw * WS + o], wb = wrow[(kw + 1) * WS + o];
#pragma unroll
                for (int rr = 0; rr < PATCH_H; rr++)
#pragma unroll
                    for (int j = 0; j < PATCH_W; j++)
                    {
                        const float2 va = __fadd2_rn(xx[rr][j + KW - 1 - kw], wa), vb = __fadd2_rn(xx[rr][j + KW - 2 - kw], wb);
                        acc[o][rr][j].x = ext3<false>(acc[o][rr][j].x, va.x, vb.x);
                        acc[o][rr][j].y = ext3<true>(acc[o][rr][j].y, va.y, vb.y);
                    }
            }
        if constexpr (KW & 1)
        {
#pragma unroll
            for (int o = 0; o < OBX; o++)
            {
                const float2 wa = wrow[(KW - 1) * WS + o];
#pragma unroll
                for (int rr = 0; rr < PATCH_H; rr++)
#pragma unroll
                    for (int j = 0; j < PATCH_W; j++)
                    {
                        const float2 va = __fadd2_rn(xx[rr][j], wa);
                        acc[o][rr][j].x = ext2<false>(acc[o][rr][j].x, va.x);
                        acc[o][rr][j].y = ext2<true>(acc[o][rr][j].y, va.y);
                    }
            }
        }
    }
}

/// CTA = (batch element, OB output channels, tile), looping over TMA chunks of input channels exactly as
/// morpho_forward_kernel does (two stages, bounded waits, border patching after the zero-filling copy).
template <int KW, int OB>
__global__ void __launch_bounds__(THREADS, 2) morpho_pair_forward_kernel(const PairForwardArgs a, const __grid_constant__ CUtensorMap tmap)
{
    extern __shared__ __align__(128) unsigned char smem_raw[];
    const Geometry& g = a.g;
    uint64_t* full = reinterpret_cast<uint64_t*>(smem_raw);
    const int welems = g.window_elems();
    const int stage_elems = (a.chunk * welems * 4 + 127) / 128 * 128 / 4;
    float* sx0 = reinterpret_cast<float*>(smem_raw + 128);
    float2* sw = reinterpret_cast<float2*>(sx0 + 2 * stage_elems);

    const int tiles = g.tiles_x * g.tiles_y;
    const int og = blockIdx.x % a.o_groups;
    const int tile = (blockIdx.x / a.o_groups) % tiles;
    const int b = blockIdx.x / (a.o_groups * tiles);
    const int tile_h0 = (tile / g.tiles_x) * TILE_H, tile_w0 = (tile % g.tiles_x) * TILE_W;
    int tx, ty, half;
    bool warp_live, split;
    thread_patch_split(tile_h0, tile_w0, g.H, g.W, OB >= 2, tx, ty, warp_live, split, half);
    const int o_count = split ? OB / 2 : OB, o_base = half * (OB / 2);
    const int o0 = og * OB;
    const int64_t plane = g.plane();
    const float* xb = a.x + static_cast<int64_t>(b) * g.Ci * plane;
    const int channels = g.identity ? 1 : g.Ci;
    const float merge_init = a.merge == MC_MERGE_MAX ? -Limits<float>::max() : (a.merge == MC_MERGE_MIN ? Limits<float>::max() : 0.0f);

    float2 merged[OB][PATCH_H][PATCH_W];   // (dilation, erosion)
#pragma unroll
    for (int o = 0; o < OB; o++)
#pragma unroll
        for (int rr = 0; rr < PATCH_H; rr++)
#pragma unroll
            for (int j = 0; j < PATCH_W; j++) merged[o][rr][j] = make_float2(merge_init, merge_init);

    const uint32_t stage_bytes = static_cast<uint32_t>(a.chunk) * welems * 4;
    const int first_channel = g.identity ? o0 : 0;
    const bool fix_border = (g.replicate || a.fill != 0.0f) && window_leaves_image(g, tile_h0, tile_w0);
    auto issue = [&](int n) {
        uint64_t* bar = full + (n & 1);
        mbar_expect_tx(bar, stage_bytes);
        tma_load_4d(sx0 + (n & 1) * stage_elems, &tmap, bar, tile_w0 - g.halo_left(), tile_h0 - g.halo_top(), first_channel + n * a.chunk, b);
    };
    if (threadIdx.x == 0)
    {
        mbar_init(full, 1);
        mbar_init(full + 1, 1);
        mbar_fence_init();
    }
    __syncthreads();
    if (threadIdx.x == 0) issue(0);

    int n = 0;
    for (int c0 = 0; c0 < channels; c0 += a.chunk, n++)
    {
        const int cc = min(a.chunk, channels - c0);
        float* sx = sx0 + (n & 1) * stage_elems;
        __syncthreads();
        if (threadIdx.x == 0 && c0 + a.chunk < channels)
        {
            fence_async_smem();
            issue(n + 1);
        }
        stage_pair_weights<OB>(sw, a.w, g, o0, c0, cc);
        if (!mbar_wait(full + (n & 1), (n >> 1) & 1, a.wait_limit_ns))
        {
            if (threadIdx.x == 0 && a.errors != nullptr) atomicAdd(a.errors, 1u);
            return;  // every thread of the CTA waits on the same barrier and gives up together
        }
        if (fix_border) fix_window_border(sx, xb + static_cast<int64_t>(first_channel + c0) * plane, plane, cc, g, tile_h0, tile_w0, a.fill);
        __syncthreads();

        for (int c = 0; c < cc && warp_live; c++)
        {
            float2 acc[OB][PATCH_H][PATCH_W];
#pragma unroll
            for (int o = 0; o < OB; o++)
#pragma unroll
                for (int rr = 0; rr < PATCH_H; rr++)
#pragma unroll
                    for (int j = 0; j < PATCH_W; j++) acc[o][rr][j] = make_float2(-Limits<float>::inf(), Limits<float>::inf());
            bool done = false;
            if constexpr (OB >= 2)
            {
                if (split)
                {
                    auto& lower = reinterpret_cast<float2 (&)[OB / 2][PATCH_H][PATCH_W]>(acc);
                    pair_window_extrema<KW, OB / 2, OB>(lower, sx + c * welems, sw + c * (KW * KW) * OB + o_base, tx, ty);
                    done = true;
                }
            }
            if (!done) pair_window_extrema<KW, OB, OB>(acc, sx + c * welems, sw + c * (KW * KW) * OB, tx, ty);

#pragma unroll
            for (int o = 0; o < OB; o++)
            {
                if (o >= o_count) break;
#pragma unroll
                for (int rr = 0; rr < PATCH_H; rr++)
#pragma unroll
                    for (int j = 0; j < PATCH_W; j++)
                    {
                        float2& m = merged[o][rr][j];
                        const float2 v = acc[o][rr][j];
                        if (a.merge == MC_MERGE_MAX) m = make_float2(m.x < v.x ? v.x : m.x, m.y < v.y ? v.y : m.y);
                        else if (a.merge == MC_MERGE_MIN) m = make_float2(v.x < m.x ? v.x : m.x, v.y < m.y ? v.y : m.y);
                        else if (a.merge == MC_MERGE_IDENTITY) m = v;
                        else m = make_float2(m.x + v.x, m.y + v.y);
                    }
            }
        }
    }

    const float divisor = static_cast<float>(g.Ci);
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
            float out_d[PATCH_W], out_e[PATCH_W];
#pragma unroll
            for (int j = 0; j < PATCH_W; j++)
            {
                out_d[j] = a.merge == MC_MERGE_AVERAGE ? merged[o][rr][j].x / divisor : merged[o][rr][j].x;
                out_e[j] = a.merge == MC_MERGE_AVERAGE ? merged[o][rr][j].y / divisor : merged[o][rr][j].y;
            }
            const int64_t row = ((static_cast<int64_t>(b) * g.Co + o0 + o_base + o) * g.H + h) * g.W;
            if (a.vec_store && w0 + PATCH_W <= g.W)
            {
                *reinterpret_cast<float4*>(a.y_dilation + row + w0) = make_float4(out_d[0], out_d[1], out_d[2], out_d[3]);
                *reinterpret_cast<float4*>(a.y_erosion + row + w0) = make_float4(out_e[0], out_e[1], out_e[2], out_e[3]);
            }
            else
            {
#pragma unroll
                for (int j = 0; j < PATCH_W; j++)
                    if (w0 + j < g.W)
                    {
                        a.y_dilation[row + w0 + j] = out_d[j];
                        a.y_erosion[row + w0 + j] = out_e[j];
                    }
            }
        }
    }
}

/// Launches the fused pass, or returns MC_ERR_UNSUPPORTED (nothing launched) when the case is not covered: the caller then
/// runs the two separate forward passes.
template <int KW, int OB>
int launch_pair_forward(const mc_desc& d, const float* x, const float* w, float* y_dilation, float* y_erosion, cudaStream_t stream)
{
    PairForwardArgs a;
    a.g = make_geometry(d, sizeof(float));
    a.x = x; a.w = w; a.y_dilation = y_dilation; a.y_erosion = y_erosion; a.merge = d.merge; a.fill = static_cast<float>(d.fill);
    a.o_groups = (d.Co + OB - 1) / OB;
    a.vec_store = (d.W % 4 == 0) && (reinterpret_cast<uintptr_t>(y_dilation) % 16 == 0) && (reinterpret_cast<uintptr_t>(y_erosion) % 16 == 0);
    a.errors = device_error_counter();
    a.wait_limit_ns = wait_limit_ns();
    const int64_t blocks = static_cast<int64_t>(a.g.tiles_x) * a.g.tiles_y * a.o_groups * d.B;
    if (blocks > 0x7fffffffLL) return MC_ERR_UNSUPPORTED;
    // Two window stages per channel plus its pairs of structuring elements; as many channels as fit in about 96 KiB, at most 8.
    const size_t window = static_cast<size_t>(a.g.window_elems()) * sizeof(float), weights = static_cast<size_t>(KW) * KW * OB * sizeof(float2);
    const size_t per_channel = 2 * ((window + 127) / 128 * 128) + weights, fixed = 128 + 2 * 128;
    const int channels = a.g.identity ? 1 : d.Ci;
    int chunk = static_cast<int>((96 * 1024 - fixed) / per_channel);
    chunk = std::max(1, std::min(std::min(chunk, 8), channels));
    const size_t smem = fixed + per_channel * chunk + 256;
    CUtensorMap tmap{};
    if (!make_window_tensor_map(&tmap, x, sizeof(float), d.B, d.Ci, d.H, d.W, a.g.win_stride, a.g.win_rows, chunk)) return MC_ERR_UNSUPPORTED;
    a.chunk = chunk;
    auto kernel = morpho_pair_forward_kernel<KW, OB>;
    if (!allow_shared(kernel, smem)) return MC_ERR_UNSUPPORTED;
    kernel<<<static_cast<unsigned>(blocks), THREADS, smem, stream>>>(a, tmap);
    return check_launch("morpho_pair_forward_kernel");
}

}  // namespace mc

// Backward dilation / erosion kernels.
//
// MAX / MIN merges: one scatter per output pixel from the packed winner index (the reference's
// morpho_backward_indices_kernel, morphocore/functional/csrc/cuda/morpho_op_kernels.cuh:609-676).
// ADD / AVERAGE / IDENTITY merges: every (output, input) channel pair routes the gradient of each pixel
// to its own extremal tap, recomputed here with a tracked strict comparison in the reference's tap order
// (morpho_backward_pairs_kernel, csrc/cuda/morpho_op_kernels.cuh:479-602; CPU semantics
// csrc/cpp/morpho_op_cpu_backward.hxx:94-156). A winning tap that read padding adds to grad_weight but not
// to grad_input (csrc/cpp/morpho_op_cpu_backward.hxx:39-41).
#pragma once
#include "common.cuh"
#include "morpho_forward.cuh"

namespace mc
{

__device__ __forceinline__ void atomic_add(float* p, float v) { atomicAdd(p, v); }
__device__ __forceinline__ void atomic_add(double* p, double v) { atomicAdd(p, v); }

/// Largest power of two number of interleaved bin copies (at most 32) that keeps bins * copies elements
/// within `budget` bytes; 0 when even one copy does not fit.
inline int bin_copies(size_t bins, size_t elem_bytes, size_t budget)
{
    int copies = 32;
    while (copies > 0 && bins * copies * elem_bytes > budget) copies /= 2;
    return copies;
}

template <typename T>
struct IndexBackwardArgs
{
    Geometry g;
    const int32_t* idx;
    const T* gy;
    T* gx;
    T* gw;
    int pixels_per_block;
    int copies;  // interleaved copies of the shared weight-gradient bins, 0 = global atomics
    T sign;      // +1 dilation, -1 erosion
};

/// grid (segments, Co): a CTA owns one output channel, a range of pixels and every batch element, so its
/// Ci * taps weight-gradient bins stay in shared memory until one flush.
template <typename T>
__global__ void __launch_bounds__(THREADS) morpho_backward_index_kernel(const IndexBackwardArgs<T> a)
{
    extern __shared__ __align__(16) unsigned char smem_raw[];
    T* bins = reinterpret_cast<T*>(smem_raw);
    const Geometry& g = a.g;
    const int o = blockIdx.y;
    const int taps = g.taps();
    const int nbins = g.Ci * taps;
    const int64_t plane = g.plane();
    const int lane_copy = a.copies > 0 ? (threadIdx.x & (a.copies - 1)) : 0;

    for (int e = threadIdx.x; e < nbins * a.copies; e += THREADS) bins[e] = T(0);
    __syncthreads();

    const int64_t p_begin = static_cast<int64_t>(blockIdx.x) * a.pixels_per_block;
    const int64_t p_end = min(p_begin + a.pixels_per_block, plane);
    for (int b = 0; b < g.B; b++)
    {
        const int64_t base = (static_cast<int64_t>(b) * g.Co + o) * plane;
        T* gxb = a.gx + static_cast<int64_t>(b) * g.Ci * plane;
        for (int64_t p = p_begin + threadIdx.x; p < p_end; p += THREADS)
        {
            const T grad = __ldg(a.gy + base + p);
            if (grad == T(0)) continue;
            const int32_t packed = __ldg(a.idx + base + p);
            const int ch = packed >> 16, k = packed & 0xFFFF;
            if (ch < 0 || ch >= g.Ci || k >= taps) continue;  // never index out of bounds on a corrupt index
            const int h = static_cast<int>(p / g.W), w = static_cast<int>(p % g.W);
            const int ih = h + g.pH - k / g.kW, iw = w + g.pW - k % g.kW;
            if (ih >= 0 && ih < g.H && iw >= 0 && iw < g.W) atomic_add(gxb + ch * plane + static_cast<int64_t>(ih) * g.W + iw, grad);
            if (a.copies > 0) atomic_add(bins + (ch * taps + k) * a.copies + lane_copy, grad);
            else atomic_add(a.gw + static_cast<int64_t>(o) * nbins + ch * taps + k, a.sign * grad);
        }
    }
    if (a.copies == 0) return;
    __syncthreads();
    for (int e = threadIdx.x; e < nbins; e += THREADS)
    {
        T sum = T(0);
        for (int c = 0; c < a.copies; c++) sum += bins[e * a.copies + c];
        if (sum != T(0)) atomic_add(a.gw + static_cast<int64_t>(o) * nbins + e, a.sign * sum);
    }
}

template <typename T>
int launch_backward_index(const mc_desc& d, const int32_t* idx, const T* gy, T* gx, T* gw, cudaStream_t stream)
{
    IndexBackwardArgs<T> a;
    a.g = make_geometry(d, sizeof(T));
    a.idx = idx; a.gy = gy; a.gx = gx; a.gw = gw;
    a.sign = d.op == MC_OP_DILATION ? T(1) : T(-1);
    const size_t nbins = static_cast<size_t>(d.Ci) * d.kH * d.kW;
    a.copies = bin_copies(nbins, sizeof(T), 64 * 1024);
    const size_t smem = nbins * a.copies * sizeof(T);
    const int64_t plane = a.g.plane();
    int64_t segments = (4 * 148 + d.Co - 1) / d.Co;
    segments = std::min<int64_t>(segments, (plane + THREADS - 1) / THREADS);
    segments = std::max<int64_t>(segments, (plane + 0x3fffffff) / 0x40000000);
    segments = std::max<int64_t>(segments, 1);
    a.pixels_per_block = static_cast<int>((plane + segments - 1) / segments);
    if (d.Co > 65535)
    {
        set_last_error("more than 65535 output channels");
        return MC_ERR_UNSUPPORTED;
    }
    auto kernel = morpho_backward_index_kernel<T>;
    if (!allow_shared(kernel, smem)) { set_last_error("cannot opt in to %zu bytes of shared memory", smem); return MC_ERR_UNSUPPORTED; }
    const dim3 grid(static_cast<unsigned>((plane + a.pixels_per_block - 1) / a.pixels_per_block), static_cast<unsigned>(d.Co));
    kernel<<<grid, THREADS, smem, stream>>>(a);
    return check_launch("morpho_backward_index_kernel");
}

template <typename T>
struct PairsBackwardArgs
{
    Geometry g;
    const T* x;
    const T* w;
    const T* gy;
    T* gx;
    T* gw;
    T fill;
    T scale;   // 1 / Ci for AVERAGE
    T sign;    // +1 dilation, -1 erosion
    int copies;
};

/// A CTA owns (batch element, input channel, tile): it stages the input window once, loops over the
/// output channels in groups of OB, and for every pair finds the extremal tap of its 8 pixels with a
/// tracked strict comparison (kh-major, kw order: the first tap wins ties, index 0 when nothing beats the
/// initial value). Gradients are accumulated in a shared window (grad_input, halo dropped at the flush)
/// and in interleaved shared bins (grad_weight), then flushed with global atomics.
template <typename T, bool IS_MIN, int KW, int OB>
__global__ void __launch_bounds__(THREADS, 2) morpho_backward_pairs_kernel(const PairsBackwardArgs<T> a)
{
    extern __shared__ __align__(16) unsigned char smem_raw[];
    const Geometry& g = a.g;
    const int taps = g.taps();
    T* sx = reinterpret_cast<T*>(smem_raw);
    T* sg = sx + g.window_elems();
    T* sw = sg + g.window_elems();
    T* bins = sw + (taps * OB + 3) / 4 * 4;

    const int tiles = g.tiles_x * g.tiles_y;
    const int ci = blockIdx.x % g.Ci;
    const int tile = (blockIdx.x / g.Ci) % tiles;
    const int b = blockIdx.x / (g.Ci * tiles);
    const int tile_h0 = (tile / g.tiles_x) * TILE_H, tile_w0 = (tile % g.tiles_x) * TILE_W;
    int tx, ty;
    bool warp_live;
    thread_patch(tile_h0, tile_w0, g.H, g.W, tx, ty, warp_live);  // threads of dead warps load zero gradients and skip below
    (void)warp_live;
    const int64_t plane = g.plane();
    const T* wb = a.w + static_cast<int64_t>(b) * g.weight_batch_stride;
    const int wci = g.identity ? 1 : g.Ci;
    const int wi = g.identity ? 0 : ci;
    const int lane_copy = threadIdx.x & (a.copies - 1);
    const T op_init = IS_MIN ? Limits<T>::inf() : -Limits<T>::inf();

    load_window(sx, a.x + (static_cast<int64_t>(b) * g.Ci + ci) * plane, g, tile_h0, tile_w0, a.fill);
    for (int e = threadIdx.x; e < g.window_elems(); e += THREADS) sg[e] = T(0);
    for (int e = threadIdx.x; e < OB * taps * a.copies; e += THREADS) bins[e] = T(0);

    const int o_begin = g.identity ? ci : 0;
    const int o_end = g.identity ? ci + 1 : g.Co;
    for (int o0 = o_begin; o0 < o_end; o0 += OB)
    {
        __syncthreads();
        for (int e = threadIdx.x; e < taps * OB; e += THREADS)
        {
            const int o = e % OB, k = e / OB;
            T v = T(0);
            if (o0 + o < o_end) v = __ldg(wb + (static_cast<int64_t>(o0 + o) * wci + wi) * taps + k);
            sw[e] = IS_MIN ? -v : v;
        }
        __syncthreads();

        T grad[OB][PATCH_H][PATCH_W];
        bool any = false;
#pragma unroll
        for (int o = 0; o < OB; o++)
#pragma unroll
            for (int rr = 0; rr < PATCH_H; rr++)
#pragma unroll
                for (int j = 0; j < PATCH_W; j++)
                {
                    const int h = tile_h0 + ty * PATCH_H + rr, w = tile_w0 + tx * PATCH_W + j;
                    T v = T(0);
                    if (o0 + o < o_end && h < g.H && w < g.W)
                        v = __ldg(a.gy + ((static_cast<int64_t>(b) * g.Co + o0 + o) * g.H + h) * g.W + w) * a.scale;
                    grad[o][rr][j] = v;
                    any |= v != T(0);
                }

        if (any)
        {
            T best[OB][PATCH_H][PATCH_W];
            int arg[OB][PATCH_H][PATCH_W];
#pragma unroll
            for (int o = 0; o < OB; o++)
#pragma unroll
                for (int rr = 0; rr < PATCH_H; rr++)
#pragma unroll
                    for (int j = 0; j < PATCH_W; j++)
                    {
                        best[o][rr][j] = op_init;
                        arg[o][rr][j] = 0;
                    }

            if constexpr (KW > 0)
            {
                constexpr int LEN = segment_len(KW, sizeof(T)), OFF = segment_offset(KW, sizeof(T)), STRIDE = window_stride(KW, sizeof(T));
                for (int kh = 0; kh < KW; kh++)
                {
                    T seg[PATCH_H][LEN];
#pragma unroll
                    for (int rr = 0; rr < PATCH_H; rr++)
                        load_segment<LEN>(seg[rr], sx + (ty * PATCH_H + rr + KW - 1 - kh) * STRIDE + tx * PATCH_W);
#pragma unroll
                    for (int kw = 0; kw < KW; kw++)
                    {
                        T wv[OB];
                        load_weights<OB>(wv, sw + (kh * KW + kw) * OB);
                        const int k = kh * KW + kw;
#pragma unroll
                        for (int o = 0; o < OB; o++)
#pragma unroll
                            for (int rr = 0; rr < PATCH_H; rr++)
#pragma unroll
                                for (int j = 0; j < PATCH_W; j++)
                                {
                                    const T v = seg[rr][OFF + j + KW - 1 - kw] + wv[o];
                                    if (strictly_better<IS_MIN>(v, best[o][rr][j]))
                                    {
                                        best[o][rr][j] = v;
                                        arg[o][rr][j] = k;
                                    }
                                }
                    }
                }
            }
            else
            {
                for (int kh = 0; kh < g.kH; kh++)
                {
                    const T* row0 = sx + (ty * PATCH_H + g.kH - 1 - kh) * g.win_stride + tx * PATCH_W;
                    for (int kw = 0; kw < g.kW; kw++)
                    {
                        T wv[OB];
                        load_weights<OB>(wv, sw + (kh * g.kW + kw) * OB);
                        const int k = kh * g.kW + kw;
#pragma unroll
                        for (int rr = 0; rr < PATCH_H; rr++)
#pragma unroll
                            for (int j = 0; j < PATCH_W; j++)
                            {
                                const T xv = row0[rr * g.win_stride + g.seg_off + j + g.kW - 1 - kw];
#pragma unroll
                                for (int o = 0; o < OB; o++)
                                {
                                    const T v = xv + wv[o];
                                    if (strictly_better<IS_MIN>(v, best[o][rr][j]))
                                    {
                                        best[o][rr][j] = v;
                                        arg[o][rr][j] = k;
                                    }
                                }
                            }
                    }
                }
            }

#pragma unroll
            for (int o = 0; o < OB; o++)
#pragma unroll
                for (int rr = 0; rr < PATCH_H; rr++)
#pragma unroll
                    for (int j = 0; j < PATCH_W; j++)
                    {
                        const T v = grad[o][rr][j];
                        if (v == T(0)) continue;
                        const int k = arg[o][rr][j];
                        const int kh = KW > 0 ? k / KW : k / g.kW, kw = KW > 0 ? k % KW : k % g.kW;
                        atomic_add(sg + (ty * PATCH_H + rr + g.kH - 1 - kh) * g.win_stride + tx * PATCH_W + g.seg_off + j + g.kW - 1 - kw, v);
                        atomic_add(bins + (o * taps + k) * a.copies + lane_copy, v);
                    }
        }
        __syncthreads();
        for (int e = threadIdx.x; e < OB * taps; e += THREADS)
        {
            const int o = e / taps, k = e % taps;
            T sum = T(0);
            for (int c = 0; c < a.copies; c++)
            {
                sum += bins[e * a.copies + c];
                bins[e * a.copies + c] = T(0);
            }
            if (sum != T(0) && o0 + o < o_end) atomic_add(a.gw + (static_cast<int64_t>(o0 + o) * wci + wi) * taps + k, a.sign * sum);
        }
    }
    __syncthreads();

    // Flush the gradient window; elements outside the image are the padding and are dropped.
    T* gxp = a.gx + (static_cast<int64_t>(b) * g.Ci + ci) * plane;
    const int row0 = tile_h0 - g.halo_top(), col0 = tile_w0 - g.halo_left();
    const int used_cols = g.used_cols();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    for (int r = warp; r < g.win_rows; r += THREADS / 32)
    {
        const int iy = row0 + r;
        if (iy < 0 || iy >= g.H) continue;
        for (int c = lane; c < used_cols; c += 32)
        {
            const int ix = col0 + c;
            const T v = sg[r * g.win_stride + c];
            if (ix >= 0 && ix < g.W && v != T(0)) atomic_add(gxp + static_cast<int64_t>(iy) * g.W + ix, v);
        }
    }
}

}  // namespace mc

#include "morpho_backward_rows.cuh"

namespace mc
{

template <typename T, bool IS_MIN, int KW, int OB>
int launch_backward_pairs(const mc_desc& d, const T* x, const T* w, const T* gy, T* gx, T* gw, cudaStream_t stream)
{
    PairsBackwardArgs<T> a;
    a.g = make_geometry(d, sizeof(T));
    a.x = x; a.w = w; a.gy = gy; a.gx = gx; a.gw = gw;
    a.fill = static_cast<T>(d.fill);
    a.scale = d.merge == MC_MERGE_AVERAGE ? T(1.0) / static_cast<T>(d.Ci) : T(1.0);
    a.sign = d.op == MC_OP_DILATION ? T(1) : T(-1);
    const size_t taps = static_cast<size_t>(d.kH) * d.kW;
    const int64_t blocks = static_cast<int64_t>(a.g.tiles_x) * a.g.tiles_y * d.Ci * d.B;
    if (blocks > 0x7fffffffLL) { set_last_error("too many tiles for one launch"); return MC_ERR_UNSUPPORTED; }
    if constexpr (sizeof(T) == 4 && (KW == 3 || KW == 5 || KW == 7))
    {
        const size_t bytes = pairs_rows_smem<KW>(a.g, a.g.identity ? 1 : d.Co);
        if (bytes > 0)
        {
            auto fast = morpho_backward_pairs_rows_kernel<IS_MIN, KW>;
            if (allow_shared(fast, bytes))
            {
                fast<<<static_cast<unsigned>(blocks), THREADS, bytes, stream>>>(a);
                return check_launch("morpho_backward_pairs_rows_kernel");
            }
        }
    }
    const size_t fixed = (2 * static_cast<size_t>(a.g.window_elems()) + (taps * OB + 3) / 4 * 4) * sizeof(T);
    if (fixed + taps * OB * sizeof(T) > MAX_SHARED_BYTES)
    {
        set_last_error("structuring element %dx%d too large for shared memory", d.kH, d.kW);
        return MC_ERR_UNSUPPORTED;
    }
    a.copies = bin_copies(taps * OB, sizeof(T), std::min<size_t>(32 * 1024, MAX_SHARED_BYTES - fixed));
    if (a.copies < 1) a.copies = 1;
    const size_t smem = fixed + taps * OB * a.copies * sizeof(T);
    auto kernel = morpho_backward_pairs_kernel<T, IS_MIN, KW, OB>;
    if (!allow_shared(kernel, smem)) { set_last_error("cannot opt in to %zu bytes of shared memory", smem); return MC_ERR_UNSUPPORTED; }
    kernel<<<static_cast<unsigned>(blocks), THREADS, smem, stream>>>(a);
    return check_launch("morpho_backward_pairs_kernel");
}

}  // namespace mc

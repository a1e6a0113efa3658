// Backward dilation / erosion kernels.
//
// MAX / MIN merges: one scatter per output pixel from the packed winner index (replaces the reference's
// morpho_backward_indices_kernel, morphocore/functional/csrc/cuda/morpho_op_kernels.cuh:609-676).
// ADD / AVERAGE / IDENTITY merges: every (output, input) channel pair routes the gradient of each pixel
// to its own extremal tap, recomputed here with a tracked strict comparison in the reference's tap order
// (morpho_backward_pairs_kernel, csrc/cuda/morpho_op_kernels.cuh:479-602; CPU semantics
// csrc/cpp/morpho_op_cpu_backward.hxx:94-156). A winning tap that read padding adds to grad_weight but not
// to grad_input (csrc/cpp/morpho_op_cpu_backward.hxx:39-41).
#pragma once
#include <type_traits>

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
struct ScatterBackwardArgs
{
    Geometry g;
    const int32_t* idx;
    const T* gy;
    T* gx;
    T* gw;
    int64_t strip;    // pixels of one plane a CTA covers (a multiple of 4 * THREADS)
    int strips;       // CTAs per plane
    int copies;       // interleaved copies of the shared weight-gradient bins (a power of two), 0 = global atomics
    bool vec;         // planes are whole 128-bit vectors and the pointers are aligned: four pixels per load
    T sign;           // +1 dilation, -1 erosion
};

/// Backward of the MAX / MIN merges from the packed winners, (channel << 16) | tap: every output pixel sends its
/// gradient to ONE input pixel and ONE weight bin. HBM-bound work (gy and idx read once, grad_input touched once per
/// output pixel), so the kernel is shaped for memory parallelism:
///   - one CTA per (batch element, output channel, strip of the plane): B * Co * strips CTAs, every SM busy whatever
///     the batch; its Ci * taps weight bins live in shared memory until one flush;
///   - a thread takes four consecutive pixels per step with 128-bit loads of gy and idx, two steps in flight;
///   - the four pixels share one row, so the pixel's (h, w) costs one division per step, and K is a compile-time
///     constant for the specialised widths, so the tap's (kh, kw) costs none.
/// A winning tap that read padding adds to grad_weight but not to grad_input, as in the reference
/// (morphocore/functional/csrc/cpp/morpho_op_cpu_backward.hxx:39-41, 78-84).
template <typename T, int KW>
__global__ void __launch_bounds__(THREADS) morpho_backward_scatter_kernel(const ScatterBackwardArgs<T> a)
{
    extern __shared__ __align__(16) unsigned char smem_raw[];
    T* bins = reinterpret_cast<T*>(smem_raw);
    const Geometry& g = a.g;
    const int kW = KW > 0 ? KW : g.kW;
    const int taps = g.taps();
    const int nbins = g.Ci * taps;
    const int64_t plane = g.plane();
    const int strip_id = blockIdx.x % a.strips;
    const int64_t bo = blockIdx.x / a.strips;          // b * Co + o
    const int o = static_cast<int>(bo % g.Co);
    const int lane_copy = a.copies > 0 ? (threadIdx.x & (a.copies - 1)) : 0;

    for (int e = threadIdx.x; e < nbins * a.copies; e += THREADS) bins[e] = T(0);
    __syncthreads();

    const T* gyp = a.gy + bo * plane;
    const int32_t* ip = a.idx + bo * plane;
    T* gxb = a.gx + (bo / g.Co) * g.Ci * plane;
    T* gwo = a.gw + static_cast<int64_t>(o) * nbins;
    const int64_t p_begin = strip_id * a.strip, p_end = min(p_begin + a.strip, plane);

    auto route = [&](T grad, int32_t packed, int h, int w) {
        if (grad == T(0)) return;
        const int ch = packed >> 16, k = packed & 0xFFFF;
        if (ch < 0 || ch >= g.Ci || k >= taps) return;   // a corrupt index is dropped, never dereferenced
        const int kh = k / kW, kw = k - kh * kW;
        const int ih = h + g.pH - kh, iw = w + g.pW - kw;
        if (ih >= 0 && ih < g.H && iw >= 0 && iw < g.W) atomic_add(gxb + ch * plane + static_cast<int64_t>(ih) * g.W + iw, grad);
        if (a.copies > 0) atomic_add(bins + (ch * taps + k) * a.copies + lane_copy, grad);
        else atomic_add(gwo + ch * taps + k, a.sign * grad);
    };

    if (a.vec)
    {
        constexpr int STEP = 4 * THREADS;
        auto load = [&](int64_t p, T (&gv)[4], int4& iv) {
            if (p < p_end)
            {
                if constexpr (sizeof(T) == 4)
                {
                    const float4 q = __ldg(reinterpret_cast<const float4*>(gyp + p));
                    gv[0] = q.x; gv[1] = q.y; gv[2] = q.z; gv[3] = q.w;
                }
                else
                {
                    const double2 q0 = __ldg(reinterpret_cast<const double2*>(gyp + p)), q1 = __ldg(reinterpret_cast<const double2*>(gyp + p + 2));
                    gv[0] = q0.x; gv[1] = q0.y; gv[2] = q1.x; gv[3] = q1.y;
                }
                iv = __ldg(reinterpret_cast<const int4*>(ip + p));
            }
            else
            {
                gv[0] = gv[1] = gv[2] = gv[3] = T(0);
                iv = make_int4(0, 0, 0, 0);
            }
        };
        for (int64_t p = p_begin + 4 * threadIdx.x; p < p_end; p += 2 * STEP)
        {
            T g0[4], g1[4];
            int4 i0, i1;
            load(p, g0, i0);
            load(p + STEP, g1, i1);
            {
                const int h = static_cast<int>(p / g.W), w = static_cast<int>(p - static_cast<int64_t>(h) * g.W);
                route(g0[0], i0.x, h, w); route(g0[1], i0.y, h, w + 1); route(g0[2], i0.z, h, w + 2); route(g0[3], i0.w, h, w + 3);
            }
            if (p + STEP < p_end)
            {
                const int64_t q = p + STEP;
                const int h = static_cast<int>(q / g.W), w = static_cast<int>(q - static_cast<int64_t>(h) * g.W);
                route(g1[0], i1.x, h, w); route(g1[1], i1.y, h, w + 1); route(g1[2], i1.z, h, w + 2); route(g1[3], i1.w, h, w + 3);
            }
        }
    }
    else
    {
        for (int64_t p = p_begin + threadIdx.x; p < p_end; p += THREADS)
        {
            const int h = static_cast<int>(p / g.W);
            route(__ldg(gyp + p), __ldg(ip + p), h, static_cast<int>(p - static_cast<int64_t>(h) * g.W));
        }
    }
    if (a.copies == 0) return;
    __syncthreads();
    for (int e = threadIdx.x; e < nbins; e += THREADS)
    {
        T sum = T(0);
        for (int c = 0; c < a.copies; c++) sum += bins[e * a.copies + c];
        if (sum != T(0)) atomic_add(gwo + e, a.sign * sum);
    }
}

template <typename T, int KW>
int launch_backward_scatter(const mc_desc& d, const int32_t* idx, const T* gy, T* gx, T* gw, cudaStream_t stream)
{
    ScatterBackwardArgs<T> a;
    a.g = make_geometry(d, sizeof(T));
    a.idx = idx; a.gy = gy; a.gx = gx; a.gw = gw;
    a.sign = d.op == MC_OP_DILATION ? T(1) : T(-1);
    const size_t nbins = static_cast<size_t>(d.Ci) * d.kH * d.kW;
    a.copies = bin_copies(nbins, sizeof(T), 48 * 1024);
    const size_t smem = nbins * a.copies * sizeof(T);
    const int64_t plane = a.g.plane();
    a.vec = d.W % 4 == 0 && reinterpret_cast<uintptr_t>(gy) % 16 == 0 && reinterpret_cast<uintptr_t>(idx) % 16 == 0;
    // Enough CTAs to fill the device several times over, but strips long enough that the flush of the bins
    // (Ci * taps global atomics per CTA) stays small beside the strip's own scatter.
    constexpr int64_t QUANTUM = 4 * THREADS;
    const int64_t pairs = static_cast<int64_t>(d.B) * d.Co;
    int64_t strips = (148 * 8 + pairs - 1) / pairs;
    const int64_t min_strip = std::max<int64_t>(QUANTUM, (static_cast<int64_t>(nbins) * 8 + QUANTUM - 1) / QUANTUM * QUANTUM);
    strips = std::min<int64_t>(strips, (plane + min_strip - 1) / min_strip);
    strips = std::max<int64_t>(strips, 1);
    a.strip = ((plane + strips - 1) / strips + QUANTUM - 1) / QUANTUM * QUANTUM;
    a.strips = static_cast<int>((plane + a.strip - 1) / a.strip);
    const int64_t blocks = pairs * a.strips;
    if (blocks > 0x7fffffffLL) { set_last_error("too many strips for one launch"); return MC_ERR_UNSUPPORTED; }
    auto kernel = morpho_backward_scatter_kernel<T, KW>;
    if (!allow_shared(kernel, smem)) { set_last_error("cannot opt in to %zu bytes of shared memory", smem); return MC_ERR_UNSUPPORTED; }
    kernel<<<static_cast<unsigned>(blocks), THREADS, smem, stream>>>(a);
    return check_launch("morpho_backward_scatter_kernel");
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
    int channels_per_cta;   // identity kernel: channels of one tile a CTA walks
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

/// Column of a window row -> element offset inside the stored row. With SWIZZLE the 16-byte vectors (two doubles) of a
/// row are permuted: vector n is stored at n ^ ((n >> 3) & 1), i.e. the two vectors of every other 32-byte pair swap
/// places. Lanes 0..7 of a quarter warp read vectors 2 tx + i; after the swap lanes 0..3 and lanes 4..7 land in bank
/// groups of different parity, so the eight lanes cover all eight bank groups and the load is conflict free.
template <bool SWIZZLE> struct SwizzledRow
{
    __device__ __forceinline__ static int at(int c)
    {
        if constexpr (SWIZZLE) return c ^ ((c >> 3) & 2);   // doubles: vector index c >> 1, its bit 3 is bit 4 of c; flip bit 1 of c
        else return c;
    }
};

/// Channels of one tile a CTA of the identity kernel walks. The kernel can pipeline several (the window of the next
/// channel is copied while the current one computes), but on B200 one channel per CTA measured fastest on the fp64
/// 11 x 11 case (5.35 ms against 5.7 - 5.9 ms for 2, 4 and 8): two co-resident CTAs already overlap each other's
/// staging, and more CTAs balance the SMs better.
constexpr int IDENTITY_CHANNELS_PER_CTA = 1;

/// Backward of the IDENTITY merge for the specialised square widths (any dtype): each channel is paired with itself,
/// so a (batch element, channel, tile) triple is one pair and every output pixel emits exactly one gradient.
/// Replaces the reference's morpho_backward_pairs_kernel for this case
/// (morphocore/functional/csrc/cuda/morpho_op_kernels.cuh:479-602) with a shape of its own:
///   - the window and the structuring element travel into shared memory by cp.async, every copy of a thread in flight
///     at once; a CTA may walk several channels of its tile (IDENTITY_CHANNELS_PER_CTA), the next channel's copies
///     landing in the other of two buffers while the current channel computes;
///   - the extremum pass is the forward kernel's inner loop (add, compare, select per tap: nothing is tracked per
///     tap); per kernel ROW the row extremum is compared once with the running best and the first improving row
///     is kept (rows ascend, so ties go to the lower kh); every window row is loaded into registers once and serves
///     both patch rows;
///   - a second pass scans that one row, from the last column down, for the lowest kw whose candidate equals the
///     best: together the first tap in kh-major, kw order that attains the extremum, the reference's winner
///     (csrc/cpp/morpho_op_cpu_kernels.hxx:212-252); index 0 when nothing beats the initial value;
///   - grad_input: one global atomic per output pixel straight to its target (no shared gradient window to zero,
///     fill and flush: with one pair it would be traversed for 2048 contributions);
///   - grad_weight: interleaved shared bins, flushed after each channel.
template <typename T, bool IS_MIN, int KW>
__global__ void __launch_bounds__(THREADS, 2) morpho_backward_identity_kernel(const PairsBackwardArgs<T> a)
{
    static_assert(KW > 0, "specialised widths only");
    constexpr int TAPS = KW * KW, TAPS_PAD = (TAPS + 3) / 4 * 4;
    constexpr int LEN = segment_len(KW, sizeof(T)), OFF = segment_offset(KW, sizeof(T)), STRIDE = window_stride(KW, sizeof(T));
    constexpr int PER = 16 / sizeof(T), VECS = LEN / PER;
    constexpr int WINDOW = (TILE_H + KW - 1) * STRIDE;
    using Row = SwizzledRow<sizeof(T) == 8>;
    extern __shared__ __align__(16) unsigned char smem_raw[];
    const Geometry& g = a.g;
    T* sx0 = reinterpret_cast<T*>(smem_raw);     // two windows
    T* sw0 = sx0 + 2 * WINDOW;                   // two structuring elements [KW][KW]
    T* bins = sw0 + 2 * TAPS_PAD;                // [TAPS][copies]

    const int tiles = g.tiles_x * g.tiles_y;
    const int groups = (g.Ci + a.channels_per_cta - 1) / a.channels_per_cta;
    const int c_begin = (blockIdx.x % groups) * a.channels_per_cta;
    const int c_count = min(a.channels_per_cta, g.Ci - c_begin);
    const int tile = (blockIdx.x / groups) % tiles;
    const int b = blockIdx.x / (groups * tiles);
    const int tile_h0 = (tile / g.tiles_x) * TILE_H, tile_w0 = (tile % g.tiles_x) * TILE_W;
    int tx, ty;
    bool warp_live;
    thread_patch(tile_h0, tile_w0, g.H, g.W, tx, ty, warp_live);
    const int64_t plane = g.plane();
    const int lane_copy = threadIdx.x & (a.copies - 1);
    const T op_init = IS_MIN ? Limits<T>::inf() : -Limits<T>::inf();
    const int h0 = tile_h0 + ty * PATCH_H, w0 = tile_w0 + tx * PATCH_W, y0 = ty * PATCH_H;
    const T* wbase = a.w + static_cast<int64_t>(b) * g.weight_batch_stride;

    // Element offsets of the thread's segment vectors inside a (swizzled) window row: constant over rows and channels.
    int vec_at[VECS];
#pragma unroll
    for (int i = 0; i < VECS; i++) vec_at[i] = Row::at(tx * PATCH_W + i * PER);

    auto stage = [&](int n) {
        const int c = c_begin + n;
        stage_window_async<STRIDE>(sx0 + (n & 1) * WINDOW, a.x + (static_cast<int64_t>(b) * g.Ci + c) * plane, g, tile_h0, tile_w0, a.fill,
                                   [](int col) { return Row::at(col); });
        for (int e = threadIdx.x; e < TAPS; e += THREADS) cp_async_element(sw0 + (n & 1) * TAPS_PAD + e, wbase + static_cast<int64_t>(c) * TAPS + e);
        asm volatile("cp.async.commit_group;" ::: "memory");
    };

    for (int e = threadIdx.x; e < TAPS * a.copies; e += THREADS) bins[e] = T(0);
    stage(0);
    for (int n = 0; n < c_count; n++)
    {
        const int ci = c_begin + n;
        const T* sx = sx0 + (n & 1) * WINDOW;
        const T* sw = sw0 + (n & 1) * TAPS_PAD;   // as stored by the caller: erosion subtracts it below

        // Is any of the thread's eight output gradients non-zero? (They are read again, from cache, when they are
        // routed: holding them through the extremum pass would cost sixteen registers in double.)
        const T* gyp = a.gy + ((static_cast<int64_t>(b) * g.Co + ci) * g.H + h0) * g.W + w0;
        bool any = false;
#pragma unroll
        for (int rr = 0; rr < PATCH_H; rr++)
#pragma unroll
            for (int j = 0; j < PATCH_W; j++)
                if (h0 + rr < g.H && w0 + j < g.W) any |= __ldg(gyp + static_cast<int64_t>(rr) * g.W + j) != T(0);
        if (n + 1 < c_count)
        {
            stage(n + 1);   // the other buffer: its last readers passed the barrier that ended channel n - 1
            asm volatile("cp.async.wait_group 1;" ::: "memory");
        }
        else asm volatile("cp.async.wait_group 0;" ::: "memory");
        __syncthreads();

        if (warp_live && __any_sync(0xffffffffu, any))
        {
            auto load_row = [&](T (&seg)[LEN], int window_row) {
                const T* row = sx + window_row * STRIDE;
#pragma unroll
                for (int i = 0; i < VECS; i++) lds128(&seg[i * PER], row + vec_at[i]);
            };
            T best[PATCH_H][PATCH_W];
            int row[PATCH_H][PATCH_W];
#pragma unroll
            for (int rr = 0; rr < PATCH_H; rr++)
#pragma unroll
                for (int j = 0; j < PATCH_W; j++)
                {
                    best[rr][j] = op_init;
                    row[rr][j] = 0;
                }
            // Kernel row kh reads window row y + KW-1-kh for the patch row y: the lower patch row's window row at kh is
            // the upper patch row's at kh + 1, so every window row is loaded once and the two segment buffers swap roles.
            static_assert(PATCH_H == 2, "two segment buffers, one per patch row");
            auto row_pass = [&](int kh, const T (&upper)[LEN], const T (&lower)[LEN]) {
                // Taps outermost: one structuring-element value in registers at a time, eight independent chains.
                T rb[PATCH_H][PATCH_W];
#pragma unroll
                for (int rr = 0; rr < PATCH_H; rr++)
#pragma unroll
                    for (int j = 0; j < PATCH_W; j++) rb[rr][j] = op_init;
#pragma unroll
                for (int kw = 0; kw < KW; kw++)
                {
                    const T wv = IS_MIN ? -sw[kh * KW + kw] : sw[kh * KW + kw];
#pragma unroll
                    for (int rr = 0; rr < PATCH_H; rr++)
#pragma unroll
                        for (int j = 0; j < PATCH_W; j++) rb[rr][j] = ext2<IS_MIN>(rb[rr][j], (rr == 0 ? upper : lower)[OFF + j + KW - 1 - kw] + wv);
                }
#pragma unroll
                for (int rr = 0; rr < PATCH_H; rr++)
#pragma unroll
                    for (int j = 0; j < PATCH_W; j++)
                        if (strictly_better<IS_MIN>(rb[rr][j], best[rr][j]))
                        {
                            best[rr][j] = rb[rr][j];
                            row[rr][j] = kh;
                        }
            };
            T seg_a[LEN], seg_b[LEN];
            load_row(seg_b, y0 + KW);   // window row of patch row 1 at kh = 0
#pragma unroll(KW <= 7 ? (KW + 1) / 2 : 1)
            for (int kh = 0; kh < KW; kh += 2)
            {
                load_row(seg_a, y0 + KW - 1 - kh);
                row_pass(kh, seg_a, seg_b);
                if (kh + 1 < KW)
                {
                    load_row(seg_b, y0 + KW - 2 - kh);
                    row_pass(kh + 1, seg_b, seg_a);
                }
            }

            T* gxp = a.gx + (static_cast<int64_t>(b) * g.Ci + ci) * plane;
#pragma unroll
            for (int rr = 0; rr < PATCH_H; rr++)
#pragma unroll
                for (int j = 0; j < PATCH_W; j++)
                {
                    if (h0 + rr >= g.H || w0 + j >= g.W) continue;
                    const T v = __ldg(gyp + static_cast<int64_t>(rr) * g.W + j) * a.scale;
                    if (v == T(0)) continue;
                    int kh = 0, kw = 0;
                    const T target = best[rr][j];
                    if (target != op_init)    // something beat the initial value (never true for NaN)
                    {
                        kh = row[rr][j];
                        kw = KW - 1;
                        const T* xr = sx + (y0 + rr + KW - 1 - kh) * STRIDE;
                        const int c0 = tx * PATCH_W + OFF + j;
                        const T* wr = sw + kh * KW;
#pragma unroll
                        for (int q = KW - 2; q >= 0; q--)
                            if (xr[Row::at(c0 + KW - 1 - q)] + (IS_MIN ? -wr[q] : wr[q]) == target) kw = q;
                    }
                    const int ih = h0 + rr + g.pH - kh, iw = w0 + j + g.pW - kw;
                    if (ih >= 0 && ih < g.H && iw >= 0 && iw < g.W) atomic_add(gxp + static_cast<int64_t>(ih) * g.W + iw, v);
                    atomic_add(bins + (kh * KW + kw) * a.copies + lane_copy, v);
                }
        }
        __syncthreads();   // every warp is done with this channel's buffers and bins
        for (int e = threadIdx.x; e < TAPS; e += THREADS)
        {
            T sum = T(0);
            for (int c = 0; c < a.copies; c++)
            {
                sum += bins[e * a.copies + c];
                bins[e * a.copies + c] = T(0);
            }
            if (sum != T(0)) atomic_add(a.gw + static_cast<int64_t>(ci) * TAPS + e, a.sign * sum);
        }
        // the next channel's first bin update comes after its own barrier above
    }
}

}  // namespace mc

#include "morpho_backward_rows.cuh"
#include "morpho_backward_regs.cuh"

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
    if constexpr (sizeof(T) == 4 && (KW == 3 || KW == 5))
    {
        const size_t bytes = pairs_regs_smem<KW>(a.g, a.g.identity ? 1 : d.Co);
        if (bytes > 0)
        {
            auto fast = morpho_backward_pairs_regs_kernel<IS_MIN, KW>;
            if (allow_shared(fast, bytes))
            {
                fast<<<static_cast<unsigned>(blocks), THREADS, bytes, stream>>>(a);
                return check_launch("morpho_backward_pairs_regs_kernel");
            }
        }
    }
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
    if constexpr (KW > 0)
    {
        if (a.g.identity)
        {
            a.copies = bin_copies(taps, sizeof(T), 8 * 1024);
            const size_t bytes = (2 * static_cast<size_t>(a.g.window_elems()) + 2 * ((taps + 3) / 4 * 4) + taps * a.copies) * sizeof(T);
            a.channels_per_cta = IDENTITY_CHANNELS_PER_CTA;
            const int64_t groups = (d.Ci + a.channels_per_cta - 1) / a.channels_per_cta;
            const int64_t id_blocks = static_cast<int64_t>(a.g.tiles_x) * a.g.tiles_y * groups * d.B;
            auto kernel = morpho_backward_identity_kernel<T, IS_MIN, KW>;
            if (a.copies >= 1 && bytes <= 100 * 1024 && allow_shared(kernel, bytes))
            {
                kernel<<<static_cast<unsigned>(id_blocks), THREADS, bytes, stream>>>(a);
                return check_launch("morpho_backward_identity_kernel");
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

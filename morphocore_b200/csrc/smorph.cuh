// Smorph (alpha-softmax soft extremum) tile kernels, forward and backward.
//
// For an output pixel and a channel pair (o, i), over the taps k that read a pixel inside the image
// (the border is excluded, not padded):
//     v_k = x_k + w_k,  ref = max_k v_k if alpha >= 0 else min_k v_k,
//     e_k = exp(alpha (v_k - ref)),  S = sum e_k,  out = (sum e_k v_k) / S
// (reference: morphocore/functional/csrc/cpp/smorph_cpu_kernels.hxx:14-24, 76-147; CUDA kernels
// csrc/cuda/smorph_kernels.cuh:80-175, 307-407, 418-571). The kernels work on u = s v with s = sign(alpha),
// so both cases are a max: u_k = s x_k + (s w_k) is one fused multiply-add with the sign folded into
// the staged structuring element, and alpha (v_k - ref) = |alpha| (u_k - ref_u) <= 0.
// Out-of-image window elements are staged as NaN: max ignores them in the first pass, and the second
// pass turns them into e = 0.
#pragma once
#include "common.cuh"
#include "morpho_backward.cuh"

namespace mc
{

constexpr float LOG2E_F = 1.4426950408889634f;

/// exp of a non-positive argument given as (difference, scale): float uses the hardware 2^x with the
/// scale pre-multiplied by log2(e); double uses exp().
__device__ __forceinline__ float soft_exp(float d, float scale2)
{
    float t = d * scale2, e;
    t = fmaxf(t, -Limits<float>::inf());  // NaN (excluded tap) -> -inf -> e = 0
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e) : "f"(t));
    return e;
}
__device__ __forceinline__ double soft_exp(double d, double scale)
{
    const double t = fmax(d * scale, -Limits<double>::inf());
    return exp(t);
}
__device__ __forceinline__ float exp_scale(float abs_alpha) { return abs_alpha * LOG2E_F; }
__device__ __forceinline__ double exp_scale(double abs_alpha) { return abs_alpha; }

/// Visit every tap of the thread's 2 x 4 patch: f(k, rr, j, x) with k = kh * kW + kw.
template <int KW, typename T, typename F>
__device__ __forceinline__ void for_each_tap(const T* __restrict__ win, const Geometry& g, int tx, int ty, F f)
{
    if constexpr (KW > 0)
    {
        constexpr int LEN = segment_len(KW, sizeof(T));
        for (int kh = 0; kh < g.kH; kh++)
        {
            T seg[PATCH_H][LEN];
#pragma unroll
            for (int rr = 0; rr < PATCH_H; rr++)
                load_segment<LEN>(seg[rr], win + (ty * PATCH_H + rr + g.kH - 1 - kh) * g.win_stride + tx * PATCH_W);
#pragma unroll
            for (int kw = 0; kw < KW; kw++)
#pragma unroll
                for (int rr = 0; rr < PATCH_H; rr++)
#pragma unroll
                    for (int j = 0; j < PATCH_W; j++) f(kh * KW + kw, rr, j, seg[rr][j + KW - 1 - kw]);
        }
    }
    else
    {
        for (int kh = 0; kh < g.kH; kh++)
        {
            const T* row0 = win + (ty * PATCH_H + g.kH - 1 - kh) * g.win_stride + tx * PATCH_W;
            for (int kw = 0; kw < g.kW; kw++)
#pragma unroll
                for (int rr = 0; rr < PATCH_H; rr++)
#pragma unroll
                    for (int j = 0; j < PATCH_W; j++) f(kh * g.kW + kw, rr, j, row0[rr * g.win_stride + j + g.kW - 1 - kw]);
        }
    }
}

/// Soft extremum of one staged pair for the thread's patch, in the u domain: ref_u, S and out_u.
template <int KW, typename T>
__device__ __forceinline__ void smorph_pair(const T* __restrict__ win, const T* __restrict__ swk, int wstride, T s, T scale, const Geometry& g,
                                            int tx, int ty, T (&ref)[PATCH_H][PATCH_W], T (&sum)[PATCH_H][PATCH_W], T (&out)[PATCH_H][PATCH_W])
{
#pragma unroll
    for (int rr = 0; rr < PATCH_H; rr++)
#pragma unroll
        for (int j = 0; j < PATCH_W; j++) ref[rr][j] = -Limits<T>::inf();
    for_each_tap<KW>(win, g, tx, ty, [&](int k, int rr, int j, T xv) { ref[rr][j] = ext2<false>(ref[rr][j], fma(s, xv, swk[k * wstride])); });

    T weighted[PATCH_H][PATCH_W];
#pragma unroll
    for (int rr = 0; rr < PATCH_H; rr++)
#pragma unroll
        for (int j = 0; j < PATCH_W; j++)
        {
            sum[rr][j] = T(0);
            weighted[rr][j] = T(0);
        }
    for_each_tap<KW>(win, g, tx, ty, [&](int k, int rr, int j, T xv) {
        const T u = fma(s, xv, swk[k * wstride]);
        const T e = soft_exp(u - ref[rr][j], scale);
        const T us = ext2<false>(u, -Limits<T>::max());  // NaN -> finite, so that 0 * us stays 0
        sum[rr][j] += e;
        weighted[rr][j] = fma(e, us, weighted[rr][j]);
    });
#pragma unroll
    for (int rr = 0; rr < PATCH_H; rr++)
#pragma unroll
        for (int j = 0; j < PATCH_W; j++) out[rr][j] = weighted[rr][j] * (T(1) / sum[rr][j]);
}

template <typename T>
struct SmorphForwardArgs
{
    Geometry g;
    const T* x;
    const T* w;
    const T* alpha;   // one per pair
    T* y;             // output (normal mode)
    const T* target;  // forward output, stats mode
    T* counts;        // stats mode: channels within 1e-6 of the target, per output pixel
    int merge;
    int o_groups;
    int chunk;
};

/// CTA = (batch element, group of OB output channels, tile), looping over chunks of input channels.
/// STATS: instead of the merged output, count for MAX / MIN merges the channels whose soft extremum is
/// within 1e-6 of the merged value, which share the gradient (csrc/cpp/smorph_cpu_kernels.hxx:397-398, 507-519).
template <typename T, int KW, int OB, bool STATS>
__global__ void __launch_bounds__(THREADS, sizeof(T) == 8 ? 1 : 2) smorph_forward_kernel(const SmorphForwardArgs<T> a)
{
    extern __shared__ __align__(16) unsigned char smem_raw[];
    const Geometry& g = a.g;
    const int taps = g.taps();
    T* sx = reinterpret_cast<T*>(smem_raw);
    T* sw = sx + a.chunk * g.window_elems();     // [chunk][taps][OB], sign folded
    T* sa = sw + a.chunk * taps * OB;            // [chunk][OB][2]: sign, exp scale

    const int tiles = g.tiles_x * g.tiles_y;
    const int og = blockIdx.x % a.o_groups;
    const int tile = (blockIdx.x / a.o_groups) % tiles;
    const int b = blockIdx.x / (a.o_groups * tiles);
    const int tile_h0 = (tile / g.tiles_x) * TILE_H, tile_w0 = (tile % g.tiles_x) * TILE_W;
    const int tx = threadIdx.x % (TILE_W / PATCH_W), ty = threadIdx.x / (TILE_W / PATCH_W);
    const int o0 = og * OB;
    const int64_t plane = g.plane();
    const T* xb = a.x + static_cast<int64_t>(b) * g.Ci * plane;
    const int channels = g.identity ? 1 : g.Ci;
    const int wci = g.identity ? 1 : g.Ci;
    const T nan = __longlong_as_double(0x7ff8000000000000LL);

    T merged[OB][PATCH_H][PATCH_W];
    T target[OB][PATCH_H][PATCH_W];
#pragma unroll
    for (int o = 0; o < OB; o++)
#pragma unroll
        for (int rr = 0; rr < PATCH_H; rr++)
#pragma unroll
            for (int j = 0; j < PATCH_W; j++)
            {
                merged[o][rr][j] = STATS ? T(0) : (a.merge == MC_MERGE_MAX ? -Limits<T>::max() : (a.merge == MC_MERGE_MIN ? Limits<T>::max() : T(0)));
                if constexpr (STATS)
                {
                    const int h = tile_h0 + ty * PATCH_H + rr, w = tile_w0 + tx * PATCH_W + j;
                    target[o][rr][j] = (o0 + o < g.Co && h < g.H && w < g.W)
                                           ? __ldg(a.target + ((static_cast<int64_t>(b) * g.Co + o0 + o) * g.H + h) * g.W + w) : T(0);
                }
            }

    for (int c0 = 0; c0 < channels; c0 += a.chunk)
    {
        const int cc = min(a.chunk, channels - c0);
        __syncthreads();
        for (int c = 0; c < cc; c++)
        {
            const int ci = g.identity ? o0 : c0 + c;
            load_window(sx + c * g.window_elems(), xb + static_cast<int64_t>(ci) * plane, g, tile_h0, tile_w0, nan);
        }
        for (int e = threadIdx.x; e < cc * OB; e += THREADS)
        {
            const int o = e % OB, c = e / OB;
            T al = T(0);
            if (o0 + o < g.Co) al = __ldg(a.alpha + (g.identity ? o0 + o : static_cast<int64_t>(o0 + o) * g.Ci + c0 + c));
            sa[e * 2] = al >= T(0) ? T(1) : T(-1);
            sa[e * 2 + 1] = exp_scale(al >= T(0) ? al : -al);
        }
        for (int e = threadIdx.x; e < cc * taps * OB; e += THREADS)
        {
            const int o = e % OB, k = (e / OB) % taps, c = e / (OB * taps);
            T v = T(0), al = T(0);
            if (o0 + o < g.Co)
            {
                const int wi = g.identity ? 0 : c0 + c;
                v = __ldg(a.w + (static_cast<int64_t>(o0 + o) * wci + wi) * taps + k);
                al = __ldg(a.alpha + (g.identity ? o0 + o : static_cast<int64_t>(o0 + o) * g.Ci + c0 + c));
            }
            sw[e] = al >= T(0) ? v : -v;
        }
        __syncthreads();

        for (int c = 0; c < cc; c++)
        {
#pragma unroll
            for (int o = 0; o < OB; o++)
            {
                const T s = sa[(c * OB + o) * 2], scale = sa[(c * OB + o) * 2 + 1];
                T ref[PATCH_H][PATCH_W], sum[PATCH_H][PATCH_W], out[PATCH_H][PATCH_W];
                smorph_pair<KW>(sx + c * g.window_elems(), sw + c * taps * OB + o, OB, s, scale, g, tx, ty, ref, sum, out);
#pragma unroll
                for (int rr = 0; rr < PATCH_H; rr++)
#pragma unroll
                    for (int j = 0; j < PATCH_W; j++)
                    {
                        const T v = s * out[rr][j];
                        T& m = merged[o][rr][j];
                        if constexpr (STATS)
                        {
                            const T dist = v - target[o][rr][j];
                            if (dist < T(1e-6) && dist > -T(1e-6)) m += T(1);
                        }
                        else if (a.merge == MC_MERGE_MAX) m = m < v ? v : m;
                        else if (a.merge == MC_MERGE_MIN) m = v < m ? v : m;
                        else if (a.merge == MC_MERGE_IDENTITY) m = v;
                        else m = m + v;
                    }
            }
        }
    }

    const T divisor = static_cast<T>(g.Ci);
    T* dst = STATS ? a.counts : a.y;
#pragma unroll
    for (int o = 0; o < OB; o++)
#pragma unroll
        for (int rr = 0; rr < PATCH_H; rr++)
#pragma unroll
            for (int j = 0; j < PATCH_W; j++)
            {
                const int h = tile_h0 + ty * PATCH_H + rr, w = tile_w0 + tx * PATCH_W + j;
                if (o0 + o >= g.Co || h >= g.H || w >= g.W) continue;
                const T v = (!STATS && a.merge == MC_MERGE_AVERAGE) ? merged[o][rr][j] / divisor : merged[o][rr][j];
                dst[((static_cast<int64_t>(b) * g.Co + o0 + o) * g.H + h) * g.W + w] = v;
            }
}

template <typename T, int KW, int OB>
int launch_smorph_forward(const mc_desc& d, const T* x, const T* w, const T* alpha, T* y, const T* target, T* counts, cudaStream_t stream)
{
    SmorphForwardArgs<T> a;
    a.g = make_geometry(d, sizeof(T));
    a.g.replicate = false;  // out-of-image taps are excluded, never read
    a.x = x; a.w = w; a.alpha = alpha; a.y = y; a.target = target; a.counts = counts; a.merge = d.merge;
    a.o_groups = (d.Co + OB - 1) / OB;
    const size_t per_channel = (static_cast<size_t>(a.g.window_elems()) + static_cast<size_t>(a.g.taps()) * OB + 2 * OB) * sizeof(T);
    if (per_channel > MAX_SHARED_BYTES)
    {
        set_last_error("structuring element %dx%d too large for shared memory", d.kH, d.kW);
        return MC_ERR_UNSUPPORTED;
    }
    const int channels = a.g.identity ? 1 : d.Ci;
    int chunk = static_cast<int>((96 * 1024) / per_channel);
    chunk = chunk < 1 ? 1 : (chunk > 8 ? 8 : chunk);
    a.chunk = chunk > channels ? channels : chunk;
    const size_t smem = per_channel * a.chunk;
    const int64_t blocks = static_cast<int64_t>(a.g.tiles_x) * a.g.tiles_y * a.o_groups * d.B;
    if (blocks > 0x7fffffffLL) { set_last_error("too many tiles for one launch"); return MC_ERR_UNSUPPORTED; }
    auto kernel = counts != nullptr ? smorph_forward_kernel<T, KW, OB, true> : smorph_forward_kernel<T, KW, OB, false>;
    if (!allow_shared(kernel, smem)) { set_last_error("cannot opt in to %zu bytes of shared memory", smem); return MC_ERR_UNSUPPORTED; }
    kernel<<<static_cast<unsigned>(blocks), THREADS, smem, stream>>>(a);
    return check_launch("smorph_forward_kernel");
}

template <typename T>
struct SmorphBackwardArgs
{
    Geometry g;
    const T* x;
    const T* w;
    const T* alpha;
    const T* y;       // forward output: merge target of MAX / MIN
    const T* counts;  // winners per output pixel, MAX / MIN
    const T* gy;
    T* gx;
    T* gw;
    T* galpha;
    int merge;
    T scale;  // 1 / Ci for AVERAGE
};

template <typename T>
__device__ __forceinline__ T warp_sum(T v)
{
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
    return v;
}

/// CTA = (batch element, input channel, tile), looping over the output channels. Per pair the forward
/// state (ref, S, out) is recomputed, then every tap k of every pixel contributes
///     c_k = p_k g + alpha p_k g (v_k - out),   p_k g = e_k (g / S)
/// to grad_input (at the pixel the tap read, accumulated in a shared gradient window) and to grad_weight
/// (summed over the warp, then per-warp private bins), and p_k g (v_k - ref)(v_k - out) to grad_alpha
/// (csrc/cpp/smorph_cpu_kernels.hxx:149-206). In the u domain alpha (v_k - out) = |alpha| (u_k - out_u) and
/// (v_k - ref)(v_k - out) = (u_k - ref_u)(u_k - out_u).
template <typename T, int KW>
__global__ void __launch_bounds__(THREADS, sizeof(T) == 8 ? 1 : 2) smorph_backward_kernel(const SmorphBackwardArgs<T> a)
{
    extern __shared__ __align__(16) unsigned char smem_raw[];
    constexpr int WARPS = THREADS / 32;
    const Geometry& g = a.g;
    const int taps = g.taps();
    T* sx = reinterpret_cast<T*>(smem_raw);
    T* sg = sx + g.window_elems();
    T* sw = sg + g.window_elems();        // [taps], sign folded
    T* wbins = sw + (taps + 3) / 4 * 4;   // [WARPS][taps]
    T* abins = wbins + WARPS * taps;      // [WARPS]

    const int tiles = g.tiles_x * g.tiles_y;
    const int ci = blockIdx.x % g.Ci;
    const int tile = (blockIdx.x / g.Ci) % tiles;
    const int b = blockIdx.x / (g.Ci * tiles);
    const int tile_h0 = (tile / g.tiles_x) * TILE_H, tile_w0 = (tile % g.tiles_x) * TILE_W;
    const int tx = threadIdx.x % (TILE_W / PATCH_W), ty = threadIdx.x / (TILE_W / PATCH_W);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int64_t plane = g.plane();
    const int wci = g.identity ? 1 : g.Ci;
    const int wi = g.identity ? 0 : ci;
    const bool winner_takes_all = a.merge == MC_MERGE_MAX || a.merge == MC_MERGE_MIN;
    const T nan = __longlong_as_double(0x7ff8000000000000LL);

    load_window(sx, a.x + (static_cast<int64_t>(b) * g.Ci + ci) * plane, g, tile_h0, tile_w0, nan);
    for (int e = threadIdx.x; e < g.window_elems(); e += THREADS) sg[e] = T(0);

    const int o_begin = g.identity ? ci : 0;
    const int o_end = g.identity ? ci + 1 : g.Co;
    for (int o = o_begin; o < o_end; o++)
    {
        const int pair = g.identity ? o : o * g.Ci + ci;
        const T al = __ldg(a.alpha + pair);
        const T s = al >= T(0) ? T(1) : T(-1);
        const T abs_alpha = al >= T(0) ? al : -al;
        const T scale = exp_scale(abs_alpha);
        __syncthreads();
        for (int k = threadIdx.x; k < taps; k += THREADS)
        {
            const T v = __ldg(a.w + (static_cast<int64_t>(o) * wci + wi) * taps + k);
            sw[k] = s * v;
        }
        for (int e = threadIdx.x; e < WARPS * taps + WARPS; e += THREADS) wbins[e] = T(0);
        __syncthreads();

        T ref[PATCH_H][PATCH_W], sum[PATCH_H][PATCH_W], out[PATCH_H][PATCH_W];
        smorph_pair<KW>(sx, sw, 1, s, scale, g, tx, ty, ref, sum, out);

        // scaled = g / S for the pixels of the image; pixels of a partial tile that lie outside it are
        // dead: their forward state may be inf or NaN and must not reach any sum.
        T scaled[PATCH_H][PATCH_W];
        bool live[PATCH_H][PATCH_W];
#pragma unroll
        for (int rr = 0; rr < PATCH_H; rr++)
#pragma unroll
            for (int j = 0; j < PATCH_W; j++)
            {
                const int h = tile_h0 + ty * PATCH_H + rr, w = tile_w0 + tx * PATCH_W + j;
                live[rr][j] = h < g.H && w < g.W;
                T grad = T(0);
                if (live[rr][j])
                {
                    const int64_t at = ((static_cast<int64_t>(b) * g.Co + o) * g.H + h) * g.W + w;
                    grad = __ldg(a.gy + at) * a.scale;
                    if (winner_takes_all)
                    {
                        const T winners = __ldg(a.counts + at);
                        grad = grad / (winners > T(0) ? winners : T(1));
                        const T dist = s * out[rr][j] - __ldg(a.y + at);
                        if (!(dist < T(1e-6) && dist > -T(1e-6))) grad = T(0);
                    }
                }
                scaled[rr][j] = live[rr][j] ? grad * (T(1) / sum[rr][j]) : T(0);
            }

        T alpha_sum = T(0);
        T tap_sum = T(0);
        int current = -1;
        // Taps are visited in order, 8 pixels per tap: when the tap index changes, the finished tap's
        // sum is reduced over the warp and stored by lane 0 in the warp's private bin.
        auto flush_tap = [&](int k) {
            const T total = warp_sum(tap_sum);
            if (lane == 0) wbins[warp * taps + k] = total;
            tap_sum = T(0);
        };
        for_each_tap<KW>(sx, g, tx, ty, [&](int k, int rr, int j, T xv) {
            if (k != current)
            {
                if (current >= 0) flush_tap(current);
                current = k;
            }
            const T u = fma(s, xv, sw[k]);
            const bool valid = u == u && live[rr][j];  // the tap reads a pixel of the image, for a pixel of the image
            const T d = valid ? u - ref[rr][j] : T(0);
            const T e = valid ? soft_exp(d, scale) : T(0);
            const T pg = e * scaled[rr][j];
            const T centered = valid ? u - out[rr][j] : T(0);
            const T c = fma(abs_alpha * pg, centered, pg);
            if (c != T(0))
            {
                const int kh = k / g.kW, kw = k % g.kW;
                atomic_add(sg + (ty * PATCH_H + rr + g.kH - 1 - kh) * g.win_stride + tx * PATCH_W + j + g.kW - 1 - kw, c);
            }
            tap_sum += c;
            alpha_sum = fma(pg * d, centered, alpha_sum);
        });
        flush_tap(current);
        alpha_sum = warp_sum(alpha_sum);
        if (lane == 0) abins[warp] = alpha_sum;
        __syncthreads();
        for (int k = threadIdx.x; k < taps; k += THREADS)
        {
            T total = T(0);
#pragma unroll
            for (int wp = 0; wp < WARPS; wp++) total += wbins[wp * taps + k];
            if (total != T(0)) atomic_add(a.gw + (static_cast<int64_t>(o) * wci + wi) * taps + k, total);
        }
        if (threadIdx.x == 0)
        {
            T total = T(0);
#pragma unroll
            for (int wp = 0; wp < WARPS; wp++) total += abins[wp];
            if (total != T(0)) atomic_add(a.galpha + pair, total);
        }
    }
    __syncthreads();

    T* gxp = a.gx + (static_cast<int64_t>(b) * g.Ci + ci) * plane;
    const int row0 = tile_h0 - g.halo_top(), col0 = tile_w0 - g.halo_left();
    const int used_cols = TILE_W + g.kW - 1;
    for (int r = warp; r < g.win_rows; r += WARPS)
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

template <typename T, int KW>
int launch_smorph_backward(const mc_desc& d, const T* x, const T* w, const T* alpha, const T* y, const T* counts, const T* gy, T* gx, T* gw,
                           T* galpha, cudaStream_t stream)
{
    SmorphBackwardArgs<T> a;
    a.g = make_geometry(d, sizeof(T));
    a.g.replicate = false;  // out-of-image taps are excluded, never read
    a.x = x; a.w = w; a.alpha = alpha; a.y = y; a.counts = counts; a.gy = gy; a.gx = gx; a.gw = gw; a.galpha = galpha;
    a.merge = d.merge;
    a.scale = d.merge == MC_MERGE_AVERAGE ? T(1.0) / static_cast<T>(d.Ci) : T(1.0);
    const size_t taps = static_cast<size_t>(d.kH) * d.kW;
    const size_t smem = (2 * static_cast<size_t>(a.g.window_elems()) + (taps + 3) / 4 * 4 + (THREADS / 32) * (taps + 1)) * sizeof(T);
    if (smem > MAX_SHARED_BYTES)
    {
        set_last_error("structuring element %dx%d too large for shared memory", d.kH, d.kW);
        return MC_ERR_UNSUPPORTED;
    }
    const int64_t blocks = static_cast<int64_t>(a.g.tiles_x) * a.g.tiles_y * d.Ci * d.B;
    if (blocks > 0x7fffffffLL) { set_last_error("too many tiles for one launch"); return MC_ERR_UNSUPPORTED; }
    auto kernel = smorph_backward_kernel<T, KW>;
    if (!allow_shared(kernel, smem)) { set_last_error("cannot opt in to %zu bytes of shared memory", smem); return MC_ERR_UNSUPPORTED; }
    kernel<<<static_cast<unsigned>(blocks), THREADS, smem, stream>>>(a);
    return check_launch("smorph_backward_kernel");
}

}  // namespace mc

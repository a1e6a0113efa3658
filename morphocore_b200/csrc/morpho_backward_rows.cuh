// Backward of the ADD / AVERAGE / IDENTITY merges for float and square 3 / 5 / 7 structuring elements:
// a cheaper search for the extremal tap than a tracked comparison, and no atomics on grad_weight.
// Included by morpho_backward.cuh.
#pragma once

namespace mc
{

///  - Tap search: a first pass takes the extremum of every kernel row with the 3-input max and keeps the
///    FIRST row that strictly improves on the running best (rows ascend, so ties go to the lower kh); a
///    second pass scans that one row, from the last column down, for the lowest kw whose value equals the
///    best. Result: the first tap in kh-major, kw order that attains the extremum, the reference's winner
///    (morphocore/functional/csrc/cpp/morpho_op_cpu_kernels.hxx:212-252), at about 2 instructions per tap
///    instead of the 4 of a tracked comparison. When nothing beats the initial value the index stays 0, as
///    in the reference.
///  - grad_weight: every warp owns bins [tap][32 lanes] (lane l uses column (l + tap) % 32, so the later
///    column sums are conflict free); a lane only ever touches its own column, a plain read-modify-write.
///    After each output channel the warp sums its columns (one lane per tap) and adds the totals to the
///    CTA's [channel][tap] table, 25 shared atomics per warp and channel; the table is flushed once per CTA.
///  - grad_input: one shared atomic per (pair, pixel) into the gradient window, as in the general kernel.
template <bool IS_MIN, int KW>
__global__ void __launch_bounds__(THREADS, 2) morpho_backward_pairs_rows_kernel(const PairsBackwardArgs<float> a)
{
    using T = float;
    constexpr int OB = 4, WARPS = THREADS / 32, TAPS = KW * KW;
    constexpr int LEN = segment_len(KW, sizeof(T)), OFF = segment_offset(KW, sizeof(T)), STRIDE = window_stride(KW, sizeof(T));
    extern __shared__ __align__(16) unsigned char smem_raw[];
    const Geometry& g = a.g;
    T* sx = reinterpret_cast<T*>(smem_raw);
    T* sg = sx + g.window_elems();
    T* sw = sg + g.window_elems();                   // [TAPS][OB] of the current group, negated for erosion
    T* bins = sw + TAPS * OB;                        // [WARPS][TAPS][32]
    T* totals = bins + WARPS * TAPS * 32;            // [channels rounded up to OB][TAPS]

    const int tiles = g.tiles_x * g.tiles_y;
    const int ci = blockIdx.x % g.Ci;
    const int tile = (blockIdx.x / g.Ci) % tiles;
    const int b = blockIdx.x / (g.Ci * tiles);
    const int tile_h0 = (tile / g.tiles_x) * TILE_H, tile_w0 = (tile % g.tiles_x) * TILE_W;
    int tx, ty;
    bool warp_live;
    thread_patch(tile_h0, tile_w0, g.H, g.W, tx, ty, warp_live);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int64_t plane = g.plane();
    const T* wb = a.w + static_cast<int64_t>(b) * g.weight_batch_stride;
    const int wci = g.identity ? 1 : g.Ci;
    const int wi = g.identity ? 0 : ci;
    const T op_init = IS_MIN ? Limits<T>::inf() : -Limits<T>::inf();
    const int o_begin = g.identity ? ci : 0;
    const int o_end = g.identity ? ci + 1 : g.Co;
    const int o_span = (o_end - o_begin + OB - 1) / OB * OB;

    load_window(sx, a.x + (static_cast<int64_t>(b) * g.Ci + ci) * plane, g, tile_h0, tile_w0, a.fill);
    for (int e = threadIdx.x; e < g.window_elems(); e += THREADS) sg[e] = T(0);
    for (int e = threadIdx.x; e < WARPS * TAPS * 32; e += THREADS) bins[e] = T(0);
    for (int e = threadIdx.x; e < o_span * TAPS; e += THREADS) totals[e] = T(0);
    T* my_bins = bins + warp * TAPS * 32;
    const T* base = sx + (ty * PATCH_H) * STRIDE + tx * PATCH_W;

    for (int o0 = o_begin; o0 < o_end; o0 += OB)
    {
        __syncthreads();
        for (int e = threadIdx.x; e < TAPS * OB; e += THREADS)
        {
            const int o = e % OB, k = e / OB;
            T v = T(0);
            if (o0 + o < o_end) v = __ldg(wb + (static_cast<int64_t>(o0 + o) * wci + wi) * TAPS + k);
            sw[e] = IS_MIN ? -v : v;
        }
        __syncthreads();
        if (!warp_live) continue;

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
        if (!__any_sync(0xffffffffu, any)) continue;

        // Pass 1: best value and the first kernel row that attains it.
        T best[OB][PATCH_H][PATCH_W];
        unsigned int row[PATCH_H][PATCH_W];   // byte o: the first kernel row that attains best[o] (one register for the four channels)
        static_assert(OB <= 4 && KW < 256, "one byte per channel");
#pragma unroll
        for (int rr = 0; rr < PATCH_H; rr++)
#pragma unroll
            for (int j = 0; j < PATCH_W; j++)
            {
                row[rr][j] = 0u;
#pragma unroll
                for (int o = 0; o < OB; o++) best[o][rr][j] = op_init;
            }
#pragma unroll
        for (int kh = 0; kh < KW; kh++)
        {
            T seg[PATCH_H][LEN];
#pragma unroll
            for (int rr = 0; rr < PATCH_H; rr++) load_segment<LEN>(seg[rr], base + (rr + KW - 1 - kh) * STRIDE);
            T wv[KW][OB];
#pragma unroll
            for (int kw = 0; kw < KW; kw++) load_weights<OB>(wv[kw], sw + (kh * KW + kw) * OB);
#pragma unroll
            for (int o = 0; o < OB; o++)
#pragma unroll
                for (int rr = 0; rr < PATCH_H; rr++)
#pragma unroll
                    for (int j = 0; j < PATCH_W; j++)
                    {
                        T rb = seg[rr][OFF + j + KW - 1] + wv[0][o];
#pragma unroll
                        for (int kw = 1; kw + 1 < KW; kw += 2)
                            rb = ext3<IS_MIN>(rb, seg[rr][OFF + j + KW - 1 - kw] + wv[kw][o], seg[rr][OFF + j + KW - 2 - kw] + wv[kw + 1][o]);
                        if (strictly_better<IS_MIN>(rb, best[o][rr][j]))
                        {
                            best[o][rr][j] = rb;
                            row[rr][j] = (row[rr][j] & ~(0xffu << (8 * o))) | (static_cast<unsigned int>(kh) << (8 * o));
                        }
                    }
        }

        // Pass 2 and scatter, one (pair, pixel) at a time, channel by channel.
#pragma unroll
        for (int o = 0; o < OB; o++)
        {
#pragma unroll
            for (int rr = 0; rr < PATCH_H; rr++)
#pragma unroll
                for (int j = 0; j < PATCH_W; j++)
                {
                    const T v = grad[o][rr][j];
                    if (v == T(0)) continue;
                    int kh = static_cast<int>((row[rr][j] >> (8 * o)) & 0xffu), kw = 0;
                    const T target = best[o][rr][j];
                    if (target != op_init)
                    {
                        const T* xr = base + (rr + KW - 1 - kh) * STRIDE + OFF + j;
                        const T* wr = sw + kh * KW * OB + o;
#pragma unroll
                        for (int q = KW - 1; q >= 0; q--)
                            if (xr[KW - 1 - q] + wr[q * OB] == target) kw = q;
                    }
                    else kh = 0;
                    const int k = kh * KW + kw;
                    atomic_add(sg + (ty * PATCH_H + rr + KW - 1 - kh) * STRIDE + tx * PATCH_W + OFF + j + KW - 1 - kw, v);
                    my_bins[k * 32 + ((lane + k) & 31)] += v;
                }
            // Column sums of the warp's bins: a lane adds the 32 partial sums of one tap, conflict free thanks
            // to the skew, clears them for the next channel and adds the warp's total to the CTA's table.
            __syncwarp();
            for (int k = lane; k < TAPS; k += 32)
            {
                T sum = T(0);
#pragma unroll 8
                for (int c = 0; c < 32; c++)
                {
                    const int col = (c + k) & 31;
                    sum += my_bins[k * 32 + col];
                    my_bins[k * 32 + col] = T(0);
                }
                if (sum != T(0)) atomic_add(totals + (o0 - o_begin + o) * TAPS + k, sum);
            }
            __syncwarp();
        }
    }
    __syncthreads();

    for (int e = threadIdx.x; e < (o_end - o_begin) * TAPS; e += THREADS)
    {
        const T sum = totals[e];
        const int o = o_begin + e / TAPS, k = e % TAPS;
        if (sum != T(0)) atomic_add(a.gw + (static_cast<int64_t>(o) * wci + wi) * TAPS + k, a.sign * sum);
    }

    T* gxp = a.gx + (static_cast<int64_t>(b) * g.Ci + ci) * plane;
    const int row0 = tile_h0 - g.halo_top(), col0 = tile_w0 - g.halo_left();
    const int used_cols = g.used_cols();
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

/// Shared memory of the kernel above, or 0 when the channel count makes it too large for two CTAs per SM.
template <int KW>
inline size_t pairs_rows_smem(const Geometry& g, int channels)
{
    constexpr int OB = 4, WARPS = THREADS / 32, TAPS = KW * KW;
    const size_t o_span = (static_cast<size_t>(channels) + OB - 1) / OB * OB;
    const size_t bytes = (2 * static_cast<size_t>(g.window_elems()) + TAPS * OB + WARPS * TAPS * 32 + o_span * TAPS) * sizeof(float);
    return bytes <= 110 * 1024 ? bytes : 0;
}

}  // namespace mc

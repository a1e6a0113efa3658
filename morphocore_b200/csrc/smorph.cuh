// Smorph (alpha-softmax soft extremum) tile kernels, forward and backward.
//
// For an output pixel and a channel pair (o, i), over the taps k that read a pixel inside the image
// (the border is excluded, not padded):
//     v_k = x_k + w_k,  ref = max_k v_k if alpha >= 0 else min_k v_k,
//     e_k = exp(alpha (v_k - ref)),  S = sum e_k,  out = (sum e_k v_k) / S
// (reference: morphocore/functional/csrc/cpp/smorph_cpu_kernels.hxx:14-24, 76-147; CUDA kernels
// csrc/cuda/smorph_kernels.cuh:80-175, 307-407, 418-571). The kernels work on u = s v with s = sign(alpha),
// so both cases are a max and alpha (v_k - ref) = |alpha| (u_k - ref_u) <= 0; u_k = s x_k + (s w_k) is one fused
// multiply-add with the sign folded into the staged structuring element. Window elements outside the
// image hold -1e30 in the window read by pairs with alpha >= 0 and +1e30 in the one read by pairs with
// alpha < 0, so u = -1e30 there: it never wins the maximum and its exponential is exactly zero (the
// exponent scale is clamped to 1e-20 from below so that this also holds for alpha = 0). Excluded taps
// therefore cost no instruction.
#pragma once
#include <type_traits>

#include "common.cuh"
#include "morpho_backward.cuh"
#include "tma.cuh"

namespace mc
{

constexpr float LOG2E_F = 1.4426950408889634f;

/// exp of a non-positive argument given as (difference, scale): float uses the hardware 2^x with the
/// scale pre-multiplied by log2(e); double uses exp().
__device__ __forceinline__ float soft_exp(float d, float scale2)
{
    float e;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e) : "f"(d * scale2));
    return e;
}
__device__ __forceinline__ double soft_exp(double d, double scale) { return exp(d * scale); }
__device__ __forceinline__ float exp_scale(float abs_alpha) { return fmaxf(abs_alpha * LOG2E_F, Limits<float>::tiny()); }
__device__ __forceinline__ double exp_scale(double abs_alpha) { return fmax(abs_alpha, Limits<double>::tiny()); }

/// 1 / x for x >= 1 (a sum of exponentials whose largest term is 1); float: hardware reciprocal, 1 ulp.
__device__ __forceinline__ float soft_rcp(float x)
{
    float r;
    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(x));
    return r;
}
__device__ __forceinline__ double soft_rcp(double x) { return 1.0 / x; }

/// Visit every tap of the thread's 2 x 4 patch: f(kh, kw, rr, j, x). KW > 0 reads whole row segments with
/// 128-bit loads and unrolls the kernel row; KH > 0 also unrolls the kernel rows, so that every index the
/// callback receives is a compile-time constant.
template <int KH, int KW, typename T, typename F>
__device__ __forceinline__ void for_each_tap(const T* __restrict__ win, const Geometry& g, int tx, int ty, F f)
{
    if constexpr (KW > 0)
    {
        // KW > 0 means a square KW x KW structuring element.
        constexpr int LEN = segment_len(KW, sizeof(T)), OFF = segment_offset(KW, sizeof(T)), STRIDE = window_stride(KW, sizeof(T));
        auto row = [&](int kh, int top) {
            T seg[PATCH_H][LEN];
#pragma unroll
            for (int rr = 0; rr < PATCH_H; rr++)
                load_segment<LEN>(seg[rr], win + (ty * PATCH_H + rr + top - kh) * STRIDE + tx * PATCH_W);
#pragma unroll
            for (int kw = 0; kw < KW; kw++)
#pragma unroll
                for (int rr = 0; rr < PATCH_H; rr++)
#pragma unroll
                    for (int j = 0; j < PATCH_W; j++) f(kh, kw, rr, j, seg[rr][OFF + j + KW - 1 - kw]);
        };
        if constexpr (KH > 0)
        {
#pragma unroll
            for (int kh = 0; kh < KH; kh++) row(kh, KH - 1);
        }
        else
        {
#pragma unroll 1
            for (int kh = 0; kh < KW; kh++) row(kh, KW - 1);
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
                    for (int j = 0; j < PATCH_W; j++) f(kh, kw, rr, j, row0[rr * g.win_stride + g.seg_off + j + g.kW - 1 - kw]);
        }
    }
}

/// Soft extremum of one staged pair for the thread's patch, in the u domain: ref_u, 1 / S and out_u.
/// `win` is the window of x for the sign s and `swk` the structuring element s w (element k at swk[k * wstride]).
template <int KH, int KW, typename T>
__device__ __forceinline__ void smorph_pair(const T* __restrict__ win, const T* __restrict__ swk, int wstride, T s, T scale, const Geometry& g, int tx,
                                            int ty, T (&ref)[PATCH_H][PATCH_W], T (&inv_sum)[PATCH_H][PATCH_W], T (&out)[PATCH_H][PATCH_W])
{
    const int kwr = KW > 0 ? KW : g.kW;
#pragma unroll
    for (int rr = 0; rr < PATCH_H; rr++)
#pragma unroll
        for (int j = 0; j < PATCH_W; j++) ref[rr][j] = -Limits<T>::inf();
    for_each_tap<KH, KW>(win, g, tx, ty, [&](int kh, int kw, int rr, int j, T xv) {
        ref[rr][j] = ext2<false>(ref[rr][j], fma(s, xv, swk[(kh * kwr + kw) * wstride]));
    });

    // d_k = (s x - ref) + s w_k: for the taps that carry the weight s x is close to ref, so the first difference is exact
    // and the sum rounds at the size of d_k, not at the size of u_k. A pixel all of whose taps are excluded (far outside
    // the image, partial tiles) keeps ref above the excluded values, so that its exponentials are 0 rather than 2^(scale w).
    T sum[PATCH_H][PATCH_W], weighted[PATCH_H][PATCH_W], minus_ref[PATCH_H][PATCH_W];
#pragma unroll
    for (int rr = 0; rr < PATCH_H; rr++)
#pragma unroll
        for (int j = 0; j < PATCH_W; j++)
        {
            sum[rr][j] = T(0);
            weighted[rr][j] = T(0);
            ref[rr][j] = ext2<false>(ref[rr][j], -Limits<T>::big() / T(16));
            minus_ref[rr][j] = -ref[rr][j];
        }
    for_each_tap<KH, KW>(win, g, tx, ty, [&](int kh, int kw, int rr, int j, T xv) {
        const T d = fma(s, xv, minus_ref[rr][j]) + swk[(kh * kwr + kw) * wstride];
        const T e = soft_exp(d, scale);
        sum[rr][j] += e;
        weighted[rr][j] = fma(e, d, weighted[rr][j]);   // relative to ref: the taps that carry the weight have small d
    });
#pragma unroll
    for (int rr = 0; rr < PATCH_H; rr++)
#pragma unroll
        for (int j = 0; j < PATCH_W; j++)
        {
            inv_sum[rr][j] = sum[rr][j] > T(0) ? soft_rcp(sum[rr][j]) : T(0);
            out[rr][j] = fma(weighted[rr][j], inv_sum[rr][j], ref[rr][j]);
        }
}

template <typename T>
__device__ __forceinline__ T warp_sum(T v)
{
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
    return v;
}

// ---------------------------------------------------------------------------------------------------
// 3 x 3 structuring elements: everything about one pair and one 4-pixel row of the patch lives in
// registers. The 9 values u_k of each pixel are formed once and serve the maximum, the exponentials and,
// in the backward pass (which also keeps the 9 exponentials), the gradients: 7 to 8 issued instructions
// per tap forward, of which one ex2, so the forward pass runs at the rate of the special-function unit.
// ---------------------------------------------------------------------------------------------------

/// u_k = s x + (s w) for the 4 pixels of patch row rr, k = kh * 3 + kw.
template <typename T>
__device__ __forceinline__ void smorph3_values(const T* __restrict__ win, const T* __restrict__ swk, int wstride, T s, const Geometry& g, int tx,
                                               int ty, int rr, T (&u)[9][PATCH_W])
{
    constexpr int LEN = segment_len(3, sizeof(T)), OFF = segment_offset(3, sizeof(T)), STRIDE = window_stride(3, sizeof(T));
#pragma unroll
    for (int kh = 0; kh < 3; kh++)
    {
        T seg[LEN];
        load_segment<LEN>(seg, win + (ty * PATCH_H + rr + 2 - kh) * STRIDE + tx * PATCH_W);
#pragma unroll
        for (int kw = 0; kw < 3; kw++)
        {
            const T wv = swk[(kh * 3 + kw) * wstride];
#pragma unroll
            for (int j = 0; j < PATCH_W; j++) u[kh * 3 + kw][j] = fma(s, seg[OFF + j + 2 - kw], wv);
        }
    }
}

/// From the u_k of 4 pixels: ref = max_k u_k, then IN PLACE d_k = u_k - ref, and e_k = exp(|alpha| d_k),
/// 1 / S and out_d = sum_k e_k d_k / S, the soft extremum relative to ref (out_u = ref + out_d).
template <typename T>
__device__ __forceinline__ void smorph3_softmax(T (&d)[9][PATCH_W], T scale, T (&ref)[PATCH_W], T (&e)[9][PATCH_W], T (&inv_sum)[PATCH_W],
                                                T (&out_d)[PATCH_W])
{
#pragma unroll
    for (int j = 0; j < PATCH_W; j++)
    {
        T m = ext3<false>(d[0][j], d[1][j], d[2][j]);
        m = ext3<false>(m, d[3][j], d[4][j]);
        m = ext3<false>(m, d[5][j], d[6][j]);
        ref[j] = ext3<false>(m, d[7][j], d[8][j]);
        T sum = T(0), weighted = T(0);
#pragma unroll
        for (int k = 0; k < 9; k++)
        {
            d[k][j] -= ref[j];
            e[k][j] = soft_exp(d[k][j], scale);
            sum += e[k][j];
            weighted = fma(e[k][j], d[k][j], weighted);
        }
        inv_sum[j] = soft_rcp(sum);
        out_d[j] = weighted * inv_sum[j];
    }
}

/// Rows of the per-warp scratch used to add 10 per-lane values over the warp (33 floats per row: the odd
/// stride keeps both the writes and the strip reads free of bank conflicts).
constexpr int RED_ROWS = 10, RED_STRIDE = 33;

/// Backward of one 3 x 3 pair for the thread's patch, see smorph_pair_backward. With d_k = u_k - ref,
/// out_d = out_u - ref = W / S, W = sum_k e_k d_k, M = sum_k e_k d_k^2 and G = g / S:
///     c_k = G e_k (1 + |alpha| (d_k - out_d)) = (G (1 - |alpha| out_d)) e_k + (G |alpha|) (e_k d_k),
///     d out / d alpha = sum_k p_k d_k (d_k - out_d) = (M - out_d W) / S,
/// so the exponential pass also forms e_k d_k and M, and each tap then costs one multiply and one fused
/// multiply-add for c_k; the alpha gradient is per pixel, not per tap. The 9 tap sums and the alpha sum of
/// the 32 lanes are added through the warp's scratch `red`: every lane stores its 10 values, three lanes
/// per row add a strip of 11 columns each, two shuffles join the strips.
template <typename T>
__device__ __forceinline__ void smorph3_pair_backward(const T* __restrict__ win, const T* __restrict__ swk, T* __restrict__ wbin, T* __restrict__ abin,
                                                      T* __restrict__ red, T s, T abs_alpha, T scale, const T (&grad)[PATCH_H][PATCH_W],
                                                      const Geometry& g, int tx, int ty, int lane, T (&gxr)[PATCH_H + 2][PATCH_W + 2])
{
    T tap_sum[9];
#pragma unroll
    for (int k = 0; k < 9; k++) tap_sum[k] = T(0);
    T alpha_sum = T(0);
#pragma unroll
    for (int rr = 0; rr < PATCH_H; rr++)
    {
        T ed[9][PATCH_W], e[9][PATCH_W];
        smorph3_values(win, swk, 1, s, g, tx, ty, rr, ed);   // u_k for now
#pragma unroll
        for (int j = 0; j < PATCH_W; j++)
        {
            T m = ext3<false>(ed[0][j], ed[1][j], ed[2][j]);
            m = ext3<false>(m, ed[3][j], ed[4][j]);
            m = ext3<false>(m, ed[5][j], ed[6][j]);
            const T ref = ext3<false>(m, ed[7][j], ed[8][j]);
            T sum = T(0), weighted = T(0), second = T(0);
#pragma unroll
            for (int k = 0; k < 9; k++)
            {
                const T d = ed[k][j] - ref;
                e[k][j] = soft_exp(d, scale);
                sum += e[k][j];
                ed[k][j] = e[k][j] * d;
                weighted += ed[k][j];
                second = fma(ed[k][j], d, second);
            }
            const T inv_sum = soft_rcp(sum);
            const T out_d = weighted * inv_sum;
            const T scaled = grad[rr][j] * inv_sum;
            const T ge = scaled * fma(-abs_alpha, out_d, T(1)), ged = scaled * abs_alpha;
            alpha_sum = fma(scaled, fma(-out_d, weighted, second), alpha_sum);
#pragma unroll
            for (int k = 0; k < 9; k++)
            {
                const T c = fma(ged, ed[k][j], ge * e[k][j]);
                gxr[rr + 2 - k / 3][j + 2 - k % 3] += c;
                tap_sum[k] += c;
            }
        }
    }
    __syncwarp();
#pragma unroll
    for (int k = 0; k < 9; k++) red[k * RED_STRIDE + lane] = tap_sum[k];
    red[9 * RED_STRIDE + lane] = alpha_sum;
    __syncwarp();
    T part = T(0);
    if (lane < 3 * RED_ROWS)
    {
        const T* strip = red + (lane / 3) * RED_STRIDE + (lane % 3) * 11;
        const int n = (lane % 3) == 2 ? 10 : 11;
#pragma unroll
        for (int c = 0; c < 11; c++)
            if (c < n) part += strip[c];
    }
    part += __shfl_down_sync(0xffffffffu, part, 1) + __shfl_down_sync(0xffffffffu, part, 2);
    if (lane < 3 * RED_ROWS && lane % 3 == 0)
    {
        if (lane < 27) wbin[lane / 3] = part;
        else *abin = part;
    }
}


// ---------------------------------------------------------------------------------------------------
// Factorised forward (float, square structuring elements up to 7 x 7, merges that need no winner test).
// exp(|alpha| (u_k - ref)) with u_k = s x_q + s w_k splits into a factor of the pixel and a factor of the tap:
//     e_k ~ E_q Ew_k,   E_q = 2^(a2 (s x_q - Mx)),   Ew_k = 2^(a2 (s w_k - Mw)),   a2 = |alpha| log2(e),
// and any common scale cancels in out_u = sum e_k u_k / sum e_k. With A_q = E_q (s x_q - Mx) and
// Bw_k = Ew_k (s w_k - Mw):
//     S = sum_k E_q Ew_k,   N = sum_k (A_q Ew_k + E_q Bw_k),   out_u = Mx + Mw + N / S,
// three fused multiply-adds per tap and no exponential, no maximum. Each warp keeps (E, A) of its own
// 32 x 8 pixel block plus halo in a private buffer, refreshed when the channel, the sign or |alpha| of
// the pair changes (pairs that share |alpha| share the buffer), with Mx the largest s x in that block, so
// E <= 1. The split is exact in real arithmetic; in float it needs 2^(-a2 (range of x in the block + range
// of w)) to stay a normal number, so a pair whose a2 * range exceeds FACTOR_RANGE (or whose block holds
// no image pixel, or NaN) takes the stable max-subtracting path instead. All terms of N have one sign, so
// the quotient loses no digits.
// ---------------------------------------------------------------------------------------------------

#ifndef MC_PACKED_FMA
#define MC_PACKED_FMA 1
#endif

// 2^-96 leaves 30 binades above the smallest normal float for the products with (s x - Mx) and (s w - Mw); the
// reciprocal of the smallest possible S, 2^96, is far from overflow.
constexpr float FACTOR_RANGE = 96.0f;
// The backward pass multiplies the relative error of the exponentials by |alpha| times the gradient, and s x - Mx rounds
// at the size of the range: beyond FACTOR_PRECISE binades its tables and its statistics carry the rounding errors of
// their differences into the exponents (factor_fill, smorph_stats_factored), which lets it use the forward limit.
constexpr float FACTOR_RANGE_BACKWARD = 96.0f;
constexpr float FACTOR_PRECISE = 8.0f;

template <int KW>
struct FactorLayout
{
    static constexpr int LEN = segment_len(KW, 4), OFF = segment_offset(KW, 4), STRIDE = window_stride(KW, 4);
    static constexpr int WS = 32 - PATCH_W + LEN;   // columns of the x window a warp's 8 x 4 threads can read
    static constexpr int ROWS = 8 + KW - 1;
    static constexpr int VECS = WS / 4;             // 128-bit vectors of x per row
    // The (E, A) block is stored in 16-byte chunks of two pixels. Thread column t (0..7) reads the LEN / 2
    // chunks from 2 t on. In one plain row the 8 lanes of a quarter warp, 32 bytes apart, would hit every bank
    // twice, so a row holds two copies: chunks [0, HALF) for t < 4 and, an odd number of chunks further,
    // chunks [8, 8 + HALF) for t >= 4. The two groups of lanes then cover all 32 banks, and every load is the
    // lane's base plus a compile-time offset.
    static constexpr int HALF = 6 + LEN / 2;
    static constexpr int SECOND = HALF % 2 == 0 ? HALF + 1 : HALF;   // chunk at which the second copy starts
    static constexpr int ROW_CHUNKS = SECOND + HALF;
    static constexpr int BYTES = ROWS * ROW_CHUNKS * 16;
    static_assert(WS % 4 == 0 && HALF % 2 == 0 && 2 * (8 + HALF) >= WS, "the two copies cover the row");
};

/// Signed integers that sort like the floats they are made from (and back).
__device__ __forceinline__ int to_ordered(float v)
{
    const int i = __float_as_int(v);
    return i ^ ((i >> 31) & 0x7fffffff);
}
__device__ __forceinline__ float from_ordered(int i) { return __int_as_float(i ^ ((i >> 31) & 0x7fffffff)); }

/// 2^(d * scale) with the product formed exactly: d * scale = hi + lo, hi the nearest integer, lo the remainder taken by
/// one fused multiply-add, so the result does not inherit the rounding of a product of magnitude up to FACTOR_RANGE
/// (half an ulp of 100 is a relative error of 2.6e-6 in the exponential, which the backward pass multiplies by |alpha|).
/// Excluded window elements (d = -1e30) give 0.
/// `tail` is a small correction of d (the rounding error of the difference that gave d): 2^((d + tail) * scale).
__device__ __forceinline__ float exp2_product(float d, float scale, float tail = 0.0f)
{
    const float product = d * scale;
    const float hi = rintf(fmaxf(product, -160.0f));
    float e_hi, e_lo;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e_hi) : "f"(hi));
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e_lo) : "f"(fmaf(tail, scale, fmaf(d, scale, -hi))));
    return product > -160.0f ? e_hi * e_lo : 0.0f;
}

/// a + b = sum + error exactly (Knuth's two-sum; the build keeps float arithmetic as written).
__device__ __forceinline__ void two_sum(float a, float b, float& sum, float& error)
{
    sum = a + b;
    const float bb = sum - a;
    error = (a - (sum - bb)) + (b - bb);
}

/// Smallest and largest in-image x of the warp's block (window elements outside the image hold +-1e30 and are
/// masked out; a block that lies inside the image, `inside`, has none and skips the masks).
/// Lanes 0 .. 3 VECS - 1 each own one vector column of every third row.
template <int KW>
__device__ __forceinline__ void factor_range(const float* __restrict__ origin, int lane, float& lo, float& hi, bool inside = false)
{
    using L = FactorLayout<KW>;
    static_assert(3 * L::VECS <= 32, "three rows per sweep");
    lo = Limits<float>::inf();
    hi = -Limits<float>::inf();
    const int r0 = lane / L::VECS, c = lane - r0 * L::VECS;
    if (r0 < 3 && inside)
        for (int r = r0; r < L::ROWS; r += 3)
        {
            const float4 v = *reinterpret_cast<const float4*>(origin + r * L::STRIDE + 4 * c);
            lo = fminf(fminf(lo, v.x), fminf(v.y, fminf(v.z, v.w)));
            hi = fmaxf(fmaxf(hi, v.x), fmaxf(v.y, fmaxf(v.z, v.w)));
        }
    else if (r0 < 3)
        for (int r = r0; r < L::ROWS; r += 3)
        {
            const float4 v = *reinterpret_cast<const float4*>(origin + r * L::STRIDE + 4 * c);
            const float e[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
            for (int i = 0; i < 4; i++)
            {
                lo = fminf(lo, e[i] > -1e29f ? e[i] : Limits<float>::inf());
                hi = fmaxf(hi, e[i] < 1e29f ? e[i] : -Limits<float>::inf());
            }
        }
    // Warp minimum and maximum with the integer warp-reduce instruction on an order-preserving image of the floats.
    lo = from_ordered(__reduce_min_sync(0xffffffffu, to_ordered(lo)));
    hi = from_ordered(__reduce_max_sync(0xffffffffu, to_ordered(hi)));
}

/// (E, A) of the warp's block for sign s, scale a2 and centre Mx.
/// `precise` (warp uniform; backward pass only, ALLOW_PRECISE) forms the exponentials with exp2_product: worth its few
/// extra instructions once the exponents are large.
template <int KW, bool ALLOW_PRECISE = false>
__device__ __forceinline__ void factor_fill(const float* __restrict__ origin, float4* __restrict__ ea, float s, float scale, float centre, int lane,
                                            bool precise = false)
{
    using L = FactorLayout<KW>;
    __syncwarp();   // every lane is done with the previous contents
    const int r0 = lane / L::VECS, c = lane - r0 * L::VECS;
    if (r0 < 3)
        for (int r = r0; r < L::ROWS; r += 3)
        {
            const float4 v = *reinterpret_cast<const float4*>(origin + r * L::STRIDE + 4 * c);
            const float x0 = fmaf(s, v.x, -centre), x1 = fmaf(s, v.y, -centre), x2 = fmaf(s, v.z, -centre), x3 = fmaf(s, v.w, -centre);
            float e0, e1, e2, e3;
            if (ALLOW_PRECISE && precise)
            {
                // s x - centre rounds at the size of the range: its rounding error goes into the exponent too.
                float t0, t1, t2, t3, h;
                two_sum(s * v.x, -centre, h, t0);
                two_sum(s * v.y, -centre, h, t1);
                two_sum(s * v.z, -centre, h, t2);
                two_sum(s * v.w, -centre, h, t3);
                e0 = exp2_product(x0, scale, t0); e1 = exp2_product(x1, scale, t1); e2 = exp2_product(x2, scale, t2); e3 = exp2_product(x3, scale, t3);
            }
            else
            {
                e0 = soft_exp(x0, scale); e1 = soft_exp(x1, scale); e2 = soft_exp(x2, scale); e3 = soft_exp(x3, scale);
            }
            const float4 first = make_float4(e0, e0 * x0, e1, e1 * x1), second = make_float4(e2, e2 * x2, e3, e3 * x3);
            float4* row = ea + r * L::ROW_CHUNKS;
            if (2 * c < L::HALF)   // HALF is even: both chunks of the vector fall on the same side
            {
                row[2 * c] = first;
                row[2 * c + 1] = second;
            }
            if (2 * c >= 8)
            {
                row[L::SECOND + 2 * c - 8] = first;
                row[L::SECOND + 2 * c - 7] = second;
            }
        }
    __syncwarp();
}

/// S and N of one pair for the thread's patch: acc = (S, sum A Ew), rest = sum E Bw, N = acc.y + rest.
/// `eb` holds (Ew_k, Bw_k) of the pair, element k at eb[k * wstride]. Every row of the (E, A) block is loaded
/// once and serves the kernel rows of both patch rows that read it.
/// `shift` (backward pass) moves the centre of the linear factor for this thread: A' = A - shift E = E (s x - Mx - shift),
/// so that N becomes sum_k e_k (d_k - shift). With shift near the soft extremum of the thread's pixels the sum is small
/// and its rounding error, which the backward pass multiplies by |alpha|, shrinks with it.
template <int KW, bool RECENTRE = false>
__device__ __forceinline__ void factor_pair(const float4* __restrict__ ea, const float2* __restrict__ eb, int wstride, int lane,
                                            float2 (&acc)[PATCH_H][PATCH_W], float (&rest)[PATCH_H][PATCH_W], float shift = 0.0f)
{
    using L = FactorLayout<KW>;
    static_assert(PATCH_H == 2, "the row schedule below is written for two patch rows");
    const int t = lane & 7;
    const float4* base = ea + ((lane >> 3) * PATCH_H) * L::ROW_CHUNKS + (t < 4 ? 2 * t : L::SECOND + 2 * t - 8);
#pragma unroll
    for (int rr = 0; rr < PATCH_H; rr++)
#pragma unroll
        for (int j = 0; j < PATCH_W; j++)
        {
            acc[rr][j] = make_float2(0.0f, 0.0f);
            rest[rr][j] = 0.0f;
        }
    // Block row r (relative to the thread's first patch row) is read by patch row rr through kernel row kh = rr + KW - 1 - r.
    auto row = [&](int r, bool first, bool second) {
        float2 seg[L::LEN];
        const float4* src = base + r * L::ROW_CHUNKS;
#pragma unroll
        for (int v = 0; v < L::LEN / 2; v++)
        {
            const float4 t = src[v];
            seg[2 * v] = make_float2(t.x, RECENTRE ? fmaf(-shift, t.x, t.y) : t.y);
            seg[2 * v + 1] = make_float2(t.z, RECENTRE ? fmaf(-shift, t.z, t.w) : t.w);
        }
        auto apply = [&](int rr, int kh) {
#pragma unroll
            for (int kw = 0; kw < KW; kw++)
            {
                const float2 t = eb[(kh * KW + kw) * wstride];
                const float2 ew2 = make_float2(t.x, t.x);
#pragma unroll
                for (int j = 0; j < PATCH_W; j++)
                {
                    const float2 q = seg[L::OFF + j + KW - 1 - kw];
#if MC_PACKED_FMA
                    acc[rr][j] = __ffma2_rn(q, ew2, acc[rr][j]);
#else
                    acc[rr][j].x = fmaf(q.x, ew2.x, acc[rr][j].x);
                    acc[rr][j].y = fmaf(q.y, ew2.y, acc[rr][j].y);
#endif
                    rest[rr][j] = fmaf(q.x, t.y, rest[rr][j]);
                }
            }
        };
        if (first) apply(0, KW - 1 - r);
        if (second) apply(1, KW - r);
    };
    row(0, true, false);
    if constexpr (KW == 3)
    {
#pragma unroll
        for (int r = 1; r < KW; r++) row(r, true, true);
    }
    else
    {
#pragma unroll 1
        for (int r = 1; r < KW; r++) row(r, true, true);
    }
    row(KW, false, true);
}

template <typename T, int KW, bool STATS>
__host__ __device__ constexpr bool can_factorise() { return sizeof(T) == 4 && !STATS && KW >= 3 && KW <= 7; }

/// 2^x, hardware approximation (flushes denormal results to zero).
__device__ __forceinline__ float ex2_approx(float x)
{
    float e;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e) : "f"(x));
    return e;
}

/// Register window of grad_input of the 3 x 3 float kernels: (PATCH_H + 2) rows of three column pairs, so that the
/// contributions of the taps with an even column offset are one packed add per pair of pixels.
using GradWindow3 = float2[PATCH_H + 2][(PATCH_W + 2) / 2];
__device__ __forceinline__ float& window_at(GradWindow3& w, int r, int c) { return (c & 1) ? w[r][c >> 1].y : w[r][c >> 1].x; }

/// float version of smorph3_pair_backward on pairs of horizontally adjacent pixels: apart from the values
/// u_k, the maximum, the exponentials and the register window of grad_input, every step is a packed
/// two-lane instruction (add.f32x2, mul.f32x2, fma.rn.f32x2), half the issue slots of the scalar form.
__device__ __forceinline__ void smorph3_pair_backward(const float* __restrict__ win, const float* __restrict__ swk, float* __restrict__ wbin,
                                                      float* __restrict__ abin, float* __restrict__ red, float s, float abs_alpha, float scale,
                                                      const float (&grad)[PATCH_H][PATCH_W], const Geometry& g, int tx, int ty, int lane,
                                                      GradWindow3& gxr)
{
    constexpr int OFF = segment_offset(3, 4), STRIDE = window_stride(3, 4);
    float2 tap_sum[9];
#pragma unroll
    for (int k = 0; k < 9; k++) tap_sum[k] = make_float2(0.0f, 0.0f);
    float2 alpha_sum = make_float2(0.0f, 0.0f);
    const float2 scale2 = make_float2(scale, scale), alpha2 = make_float2(abs_alpha, abs_alpha), minus_alpha2 = make_float2(-abs_alpha, -abs_alpha);
    const float2 one2 = make_float2(1.0f, 1.0f);
#pragma unroll
    for (int rr = 0; rr < PATCH_H; rr++)
#pragma unroll
        for (int jp = 0; jp < PATCH_W / 2; jp++)
        {
            // The two pixels read segment columns first .. first + 3: two aligned 128-bit loads per window row.
            const int first = OFF + 2 * jp, quad = first / 4, base = first - 4 * quad;
            float2 d[9], e[9];
#pragma unroll
            for (int kh = 0; kh < 3; kh++)
            {
                float seg[8];
                const float* row = win + (ty * PATCH_H + rr + 2 - kh) * STRIDE + tx * PATCH_W + 4 * quad;
                lds128(seg, row);
                lds128(seg + 4, row + 4);
#pragma unroll
                for (int kw = 0; kw < 3; kw++)
                {
                    const float wv = swk[kh * 3 + kw];
                    d[kh * 3 + kw] = make_float2(fmaf(s, seg[base + 2 - kw], wv), fmaf(s, seg[base + 3 - kw], wv));   // u_k for now
                }
            }
            float mx = ext3<false>(d[0].x, d[1].x, d[2].x), my = ext3<false>(d[0].y, d[1].y, d[2].y);
            mx = ext3<false>(mx, d[3].x, d[4].x); my = ext3<false>(my, d[3].y, d[4].y);
            mx = ext3<false>(mx, d[5].x, d[6].x); my = ext3<false>(my, d[5].y, d[6].y);
            mx = ext3<false>(mx, d[7].x, d[8].x); my = ext3<false>(my, d[7].y, d[8].y);
            const float2 minus_ref = make_float2(-mx, -my);
            float2 sum = make_float2(0.0f, 0.0f), weighted = sum, second = sum;
#pragma unroll
            for (int k = 0; k < 9; k++)
            {
                const float2 dk = __fadd2_rn(d[k], minus_ref);
                const float2 t = __fmul2_rn(dk, scale2);
                e[k] = make_float2(ex2_approx(t.x), ex2_approx(t.y));
                sum = __fadd2_rn(sum, e[k]);
                d[k] = __fmul2_rn(e[k], dk);   // e_k d_k from here on: exactly zero for excluded taps, whose d_k is -1e30
                weighted = __fadd2_rn(weighted, d[k]);
                second = __ffma2_rn(d[k], dk, second);
            }
            const float2 inv_sum = make_float2(soft_rcp(sum.x), soft_rcp(sum.y));
            const float2 out_d = __fmul2_rn(weighted, inv_sum);
            const float2 scaled = __fmul2_rn(make_float2(grad[rr][2 * jp], grad[rr][2 * jp + 1]), inv_sum);
            const float2 ge = __fmul2_rn(scaled, __ffma2_rn(minus_alpha2, out_d, one2)), ged = __fmul2_rn(scaled, alpha2);
            const float2 minus_out_d = make_float2(-out_d.x, -out_d.y);
            alpha_sum = __ffma2_rn(scaled, __ffma2_rn(minus_out_d, weighted, second), alpha_sum);
#pragma unroll
            for (int k = 0; k < 9; k++)
            {
                const float2 c = __ffma2_rn(ged, d[k], __fmul2_rn(ge, e[k]));
                window_at(gxr, rr + 2 - k / 3, 2 * jp + 2 - k % 3) += c.x;
                window_at(gxr, rr + 2 - k / 3, 2 * jp + 3 - k % 3) += c.y;
                tap_sum[k] = __fadd2_rn(tap_sum[k], c);
            }
        }
    __syncwarp();
#pragma unroll
    for (int k = 0; k < 9; k++) red[k * RED_STRIDE + lane] = tap_sum[k].x + tap_sum[k].y;
    red[9 * RED_STRIDE + lane] = alpha_sum.x + alpha_sum.y;
    __syncwarp();
    float part = 0.0f;
    if (lane < 3 * RED_ROWS)
    {
        const float* strip = red + (lane / 3) * RED_STRIDE + (lane % 3) * 11;
        const int n = (lane % 3) == 2 ? 10 : 11;
#pragma unroll
        for (int c = 0; c < 11; c++)
            if (c < n) part += strip[c];
    }
    part += __shfl_down_sync(0xffffffffu, part, 1) + __shfl_down_sync(0xffffffffu, part, 2);
    if (lane < 3 * RED_ROWS && lane % 3 == 0)
    {
        if (lane < 27) wbin[lane / 3] = part;
        else *abin = part;
    }
}

/// Floats per pair in the table of smorph3_pair_backward_bounded: nine duplicated shifted weights, a pad, and at
/// BOUNDED_PARAMS the pair's (s scale, |alpha| / scale, 1 / scale^2, widest range of x for which the form is used).
constexpr int BOUNDED_ROW = 24, BOUNDED_PARAMS = 20;
/// Range of exponent scales for which smorph3_pair_backward_bounded works in scaled units.
constexpr float BOUNDED_SCALE_MIN = 1e-6f, BOUNDED_SCALE_MAX = 1e6f;

/// smorph3_pair_backward (float) without the maximum, in units of the exponent. The exponentials are taken relative to
/// centre_x + bound_w, where centre_x is the MIDDLE of the range of s x that the thread's pixels can read and bound_w the
/// largest s w_k, and the caller has checked that scale * (widest such range in the warp + range of w) is at most
/// BOUND_RANGE: every exponent then lies within BOUND_RANGE / 2 of zero (plus the range of w below), so no exponential,
/// sum, reciprocal or product of two of them leaves the normal floats. The maximum pass goes. The exponent itself,
///     t_k = scale (u_k - centre_x - bound_w) = (scale s x - scale centre_x) + scale (s w_k - bound_w),
/// takes the place of d_k: one fma per window element and one packed add per tap, the second term read ready-made
/// (duplicated, for the packed add) from `shifted`, which the chunk's preparation fills. The sums S, sum e t and
/// sum e t^2 are scale and scale^2 times those of the unscaled form; the middle of the range keeps |t_k| as small as a
/// per-thread reference can (the difference sum e t^2 - out_t sum e t of grad_alpha cancels at the size of t^2), and a
/// common rounding error of the reference shifts every t_k of a pixel alike and cancels in all three results:
///     c_k = (g / S) e_k (1 + kappa (t_k - out_t)),   kappa = |alpha| / scale,   out_t = sum e t / S
///     grad_alpha += (g / S) (sum e t^2 - out_t sum e t) / scale^2.
__device__ __forceinline__ void smorph3_pair_backward_bounded(const float* __restrict__ win, const float4* __restrict__ shifted4,
                                                              float* __restrict__ wbin, float* __restrict__ abin, float* __restrict__ red,
                                                              float4 params, float centre_x, const float* __restrict__ slot, float grad_scale,
                                                              int tx, int ty, int lane, GradWindow3& gxr)
{
    constexpr int OFF = segment_offset(3, 4), STRIDE = window_stride(3, 4);
    float2 tap_sum[9];
    const uint32_t shifted = static_cast<uint32_t>(__cvta_generic_to_shared(shifted4));
#pragma unroll
    for (int k = 0; k < 9; k++) tap_sum[k] = make_float2(0.0f, 0.0f);
    const float slope = params.x, minus_bound = -(fabsf(slope) * centre_x);
    const float2 kappa2 = make_float2(params.y, params.y);
    float2 alpha_sum = make_float2(0.0f, 0.0f);
#pragma unroll
    for (int rr = 0; rr < PATCH_H; rr++)
#pragma unroll
        for (int jp = 0; jp < PATCH_W / 2; jp++)
        {
            const int first = OFF + 2 * jp, quad = first / 4, base = first - 4 * quad;
            float2 d[9], e[9];
#pragma unroll
            for (int kh = 0; kh < 3; kh++)
            {
                float seg[8];
                const float* row = win + (ty * PATCH_H + rr + 2 - kh) * STRIDE + tx * PATCH_W + 4 * quad;
                lds128(seg, row);
                lds128(seg + 4, row + 4);
                float centred[4];
#pragma unroll
                for (int i = 0; i < 4; i++) centred[i] = fmaf(slope, seg[base + i], minus_bound);
#pragma unroll
                for (int kw = 0; kw < 3; kw++) {
                    float2 sh;
                    asm volatile("ld.shared.v2.f32 {%0, %1}, [%2];" : "=f"(sh.x), "=f"(sh.y) : "r"(shifted + 8u * (kh * 3 + kw)));
                    d[kh * 3 + kw] = __fadd2_rn(make_float2(centred[2 - kw], centred[3 - kw]), sh);
                }
            }
            float2 sum = make_float2(0.0f, 0.0f), weighted = sum, second = sum;
#pragma unroll
            for (int k = 0; k < 9; k++)
            {
                const float2 t = d[k];
                e[k] = make_float2(ex2_approx(t.x), ex2_approx(t.y));
                sum = __fadd2_rn(sum, e[k]);
                d[k] = __fmul2_rn(e[k], t);   // e_k t_k from here on: exactly zero for excluded taps, whose t_k is hugely negative
                weighted = __fadd2_rn(weighted, d[k]);
                second = __ffma2_rn(d[k], t, second);
            }
            // A pixel far outside the image (partial tiles) has no tap at all: S = 0 and its gradient is zero; the floor
            // keeps 1 / S finite, so that its products are exact zeros.
            const float2 inv_sum = make_float2(soft_rcp(fmaxf(sum.x, 1e-30f)), soft_rcp(fmaxf(sum.y, 1e-30f)));
            const float2 out_t = __fmul2_rn(weighted, inv_sum);
            // The two gradients come from the thread's slot only now: eight registers less across the tap loops.
            const float2 raw = *reinterpret_cast<const float2*>(slot + rr * PATCH_W + 2 * jp);
            const float2 scaled = __fmul2_rn(make_float2(raw.x * grad_scale, raw.y * grad_scale), inv_sum);
            const float2 ged = __fmul2_rn(scaled, kappa2);
            const float2 minus_out_t = make_float2(-out_t.x, -out_t.y);
            const float2 ge = __ffma2_rn(ged, minus_out_t, scaled);
            alpha_sum = __ffma2_rn(scaled, __ffma2_rn(minus_out_t, weighted, second), alpha_sum);
#pragma unroll
            for (int k = 0; k < 9; k++)
            {
                const float2 c = __ffma2_rn(ged, d[k], __fmul2_rn(ge, e[k]));
                const int r = rr + 2 - k / 3, kw = k % 3;
                if (kw == 1)
                {
                    gxr[r][jp].y += c.x;
                    gxr[r][jp + 1].x += c.y;
                }
                else
                {
                    float2& into = gxr[r][kw == 0 ? jp + 1 : jp];
                    into = __fadd2_rn(into, c);
                }
                tap_sum[k] = __fadd2_rn(tap_sum[k], c);
            }
        }
    __syncwarp();
#pragma unroll
    for (int k = 0; k < 9; k++) red[k * RED_STRIDE + lane] = tap_sum[k].x + tap_sum[k].y;
    red[9 * RED_STRIDE + lane] = (alpha_sum.x + alpha_sum.y) * params.z;
    __syncwarp();
    float part = 0.0f;
    if (lane < 3 * RED_ROWS)
    {
        // Three lanes per row, eleven columns each: the last strip ends on the row's pad column, which the kernel keeps zero.
        const float* strip = red + (lane / 3) * RED_STRIDE + (lane % 3) * 11;
#pragma unroll
        for (int c = 0; c < 11; c++) part += strip[c];
    }
    part += __shfl_down_sync(0xffffffffu, part, 1) + __shfl_down_sync(0xffffffffu, part, 2);
    if (lane < 3 * RED_ROWS && lane % 3 == 0)
    {
        if (lane < 27) wbin[lane / 3] = part;
        else *abin = part;
    }
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
    const T* beta;    // smooth merge: one value per output channel
    T* soft_ref;      // smooth merge, backward's statistics pass: extremum of the channel outputs per output pixel (instead of y)
    T* soft_inv;      // and 1 / sum_i q_i
    int merge;
    int o_groups;
    int chunk;
    int factorise;    // use the factorised path where it is safe (merges without winner test)
    unsigned int* errors;  // counter of timed-out waits
    uint64_t wait_limit_ns; // bound of one wait on a TMA copy
};

/// CTA = (batch element, group of OB output channels, tile), looping over chunks of input channels; with
/// USE_TMA the windows of chunk n + 1 are copied by TMA while chunk n is computed, see morpho_forward_kernel.
/// STATS: instead of the merged output, count for MAX / MIN merges the channels whose soft extremum is
/// within 1e-6 of the merged value, which share the gradient (csrc/cpp/smorph_cpu_kernels.hxx:397-398, 507-519).
/// MODE 2 (smooth merge, Smorph SCM; csrc/cpp/smorph_cpu_kernels.hxx:231-266): the channel outputs c_i of an output
/// pixel are merged by a second soft extremum with the output channel's beta, final = sum_i q_i c_i / sum_i q_i,
/// q_i = exp(beta (c_i - ref)), ref = max_i c_i (beta >= 0) or min_i c_i. The channels stream through the CTA, so the
/// sums are kept relative to the running extremum and rescaled when it moves. The kernel writes the merged value,
/// or, for the backward pass, ref and 1 / sum_i q_i.
template <typename T, int KW, int OB, int MODE, bool USE_TMA>
__global__ void __launch_bounds__(THREADS, sizeof(T) == 8 ? 1 : 2)
    smorph_forward_kernel(const SmorphForwardArgs<T> a, const __grid_constant__ CUtensorMap tmap)
{
    constexpr bool STATS = MODE == 1, SOFT = MODE == 2;
    extern __shared__ __align__(128) unsigned char smem_raw[];
    const Geometry& g = a.g;
    const int taps = g.taps();
    const int welems = g.window_elems();
    // Layout: [2 mbarriers][pad to 128][stage 0][stage 1 (TMA only)][weights][signs and scales]; a stage is
    // [slot][chunk][window]: slot 0 read by pairs of the CTA's first sign, slot 1 by the other sign if any.
    uint64_t* full = reinterpret_cast<uint64_t*>(smem_raw);
    const int slot_elems = (a.chunk * welems * static_cast<int>(sizeof(T)) + 127) / 128 * 128 / static_cast<int>(sizeof(T));
    T* sx0 = reinterpret_cast<T*>(smem_raw + 128);
    T* sw = sx0 + (USE_TMA ? 2 : 1) * 2 * slot_elems;   // [2 chunk][taps][OB], sign folded
    T* sa = sw + 2 * a.chunk * taps * OB;                 // [2 chunk][OB][2]: sign, exp scale
    // Factorised path: [2 chunk][taps][OB] (Ew, Bw), [2 chunk][OB] (Mw, range of w), then one (E, A) buffer per warp.
    constexpr bool FACTOR = can_factorise<T, KW, MODE != 0>();
    float2* seb = reinterpret_cast<float2*>(smem_raw + (reinterpret_cast<unsigned char*>(sa + 2 * a.chunk * OB * 2) - smem_raw + 15) / 16 * 16);
    float2* spair = seb + 2 * a.chunk * taps * OB;
    float4* sea = reinterpret_cast<float4*>(smem_raw + (reinterpret_cast<unsigned char*>(spair + 2 * a.chunk * OB) - smem_raw + 15) / 16 * 16)
                  + (threadIdx.x >> 5) * (FactorLayout<FACTOR ? KW : 3>::BYTES / 16);
    const bool factorise = FACTOR && a.factorise != 0;

    const int tiles = g.tiles_x * g.tiles_y;
    const int og = blockIdx.x % a.o_groups;
    const int tile = (blockIdx.x / a.o_groups) % tiles;
    const int b = blockIdx.x / (a.o_groups * tiles);
    const int tile_h0 = (tile / g.tiles_x) * TILE_H, tile_w0 = (tile % g.tiles_x) * TILE_W;
    int tx, ty, half;
    bool warp_live, split;
    thread_patch_split(tile_h0, tile_w0, g.H, g.W, OB >= 2, tx, ty, warp_live, split, half);
    // Output channels of this warp: slots 0 .. o_count - 1 of the per-channel register arrays hold channels
    // o0 + o_base + slot (all OB of them unless the tile is split between the warps of a row, see thread_patch_split).
    const int o_count = split ? OB / 2 : OB, o_base = half * (OB / 2);
    const int wx = split ? 0 : static_cast<int>((threadIdx.x >> 5) & 1);   // column block of the warp
    const int o0 = og * OB;
    const int64_t plane = g.plane();
    const T* xb = a.x + static_cast<int64_t>(b) * g.Ci * plane;
    const int channels = g.identity ? 1 : g.Ci;
    const int wci = g.identity ? 1 : g.Ci;
    const int first_channel = g.identity ? o0 : 0;

    // Signs of every pair of this CTA: a single sign needs one window per channel, both signs need two.
    bool any_pos = false, any_neg = false;
    for (int e = threadIdx.x; e < channels * OB; e += THREADS)
    {
        const int o = e % OB, c = e / OB;
        if (o0 + o >= g.Co) continue;
        const T al = __ldg(a.alpha + (g.identity ? o0 + o : static_cast<int64_t>(o0 + o) * g.Ci + c));
        any_pos |= al >= T(0);
        any_neg |= al < T(0);
    }
    if constexpr (USE_TMA)
    {
        if (threadIdx.x == 0)
        {
            mbar_init(full, 1);
            mbar_init(full + 1, 1);
            mbar_fence_init();
        }
    }
    any_pos = __syncthreads_or(any_pos);
    any_neg = __syncthreads_or(any_neg);
    const bool mixed = any_pos && any_neg;
    // Channels per stage: with a single sign both slots of a stage hold channels, twice as many per barrier.
    const int span = mixed ? a.chunk : 2 * a.chunk;
    const T fill0 = any_pos ? -Limits<T>::big() : Limits<T>::big();   // slot 0 serves alpha >= 0 unless every alpha is negative
    const uint32_t slot_bytes = static_cast<uint32_t>(a.chunk) * welems * sizeof(T);
    const bool border = window_leaves_image(g, tile_h0, tile_w0);
    // Factorised path: does the warp's block of the window (32 x 8 pixels plus halo) lie inside the image?
    [[maybe_unused]] bool block_inside = false;
    if constexpr (FACTOR)
    {
        const int r0 = tile_h0 - g.halo_top() + 8 * (static_cast<int>(threadIdx.x >> 5) >> 1), c0 = tile_w0 - g.halo_left() + 32 * wx;
        block_inside = r0 >= 0 && r0 + FactorLayout<FACTOR ? KW : 3>::ROWS <= g.H && c0 >= 0 && c0 + FactorLayout<FACTOR ? KW : 3>::WS <= g.W;
    }
    auto issue = [&](int n) {
        uint64_t* bar = full + (n & 1);
        T* stage = sx0 + (n & 1) * 2 * slot_elems;
        const int c_first = first_channel + n * span;
        // The second copy brings the same channels again (other border fill) or the next `chunk` channels; a
        // copy that starts past the last channel is skipped.
        const bool second = mixed || (n * span + a.chunk < channels);
        mbar_expect_tx(bar, second ? 2 * slot_bytes : slot_bytes);
        tma_load_4d(stage, &tmap, bar, tile_w0 - g.halo_left(), tile_h0 - g.halo_top(), c_first, b);
        if (second) tma_load_4d(stage + slot_elems, &tmap, bar, tile_w0 - g.halo_left(), tile_h0 - g.halo_top(), mixed ? c_first : c_first + a.chunk, b);
    };
    if constexpr (USE_TMA)
    {
        if (threadIdx.x == 0) issue(0);
    }

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
                    target[o][rr][j] = (o0 + o_base + o < g.Co && h < g.H && w < g.W)
                                           ? __ldg(a.target + ((static_cast<int64_t>(b) * g.Co + o0 + o_base + o) * g.H + h) * g.W + w) : T(0);
                }
            }

    // Smooth merge: running extremum of sign(beta) c_i and sum of q_i per pixel (merged holds sum q_i c_i).
    [[maybe_unused]] T soft_m[SOFT ? OB : 1][PATCH_H][PATCH_W], soft_s[SOFT ? OB : 1][PATCH_H][PATCH_W];
    [[maybe_unused]] T soft_sign[OB], soft_scale[OB];
    if constexpr (SOFT)
    {
#pragma unroll
        for (int o = 0; o < OB; o++)
        {
            const T bt = o0 + o_base + o < g.Co ? __ldg(a.beta + o0 + o_base + o) : T(0);
            soft_sign[o] = bt >= T(0) ? T(1) : T(-1);
            soft_scale[o] = exp_scale(bt >= T(0) ? bt : -bt);
#pragma unroll
            for (int rr = 0; rr < PATCH_H; rr++)
#pragma unroll
                for (int j = 0; j < PATCH_W; j++)
                {
                    soft_m[o][rr][j] = -Limits<T>::inf();
                    soft_s[o][rr][j] = T(0);
                }
        }
    }
    [[maybe_unused]] T offset[OB];   // factorised path: per-channel constant part of the sum
#pragma unroll
    for (int o = 0; o < OB; o++) offset[o] = T(0);

    // Window of channel c of the stage for a pair of sign s.
    auto window_of = [&](T* stage, int c, bool negative) {
        if (mixed) return stage + (negative ? slot_elems : 0) + c * welems;
        return stage + (c >= a.chunk ? slot_elems + (c - a.chunk) * welems : c * welems);
    };
    int n = 0;
    for (int c0 = 0; c0 < channels; c0 += span, n++)
    {
        const int cc = min(span, channels - c0);
        T* stage = sx0 + (USE_TMA ? (n & 1) * 2 * slot_elems : 0);
        __syncthreads();
        if constexpr (USE_TMA)
        {
            if (threadIdx.x == 0 && c0 + span < channels)
            {
                fence_async_smem();
                issue(n + 1);
            }
        }
        else
        {
            for (int c = 0; c < cc; c++)
            {
                const T* src = xb + static_cast<int64_t>(first_channel + c0 + c) * plane;
                load_window_signed(any_pos ? window_of(stage, c, false) : nullptr, any_neg ? window_of(stage, c, true) : nullptr, src, g, tile_h0,
                                   tile_w0);
            }
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
        if constexpr (FACTOR)
        {
            if (factorise)
            {
                // One warp per pair, one lane per tap: Mw and the range of s w by shuffles, then (Ew, Bw).
                const int lane = threadIdx.x & 31;
                for (int e = threadIdx.x >> 5; e < cc * OB; e += THREADS / 32)
                {
                    const int o = e % OB, c = e / OB;
                    if (o0 + o >= g.Co)
                    {
                        if (lane == 0) spair[e] = make_float2(0.0f, Limits<float>::inf());   // never factorised
                        continue;
                    }
                    const float al = __ldg(a.alpha + (g.identity ? o0 + o : static_cast<int64_t>(o0 + o) * g.Ci + c0 + c));
                    const float sgn = al >= 0.0f ? 1.0f : -1.0f, scale = exp_scale(fabsf(al));
                    const float* wp = a.w + (static_cast<int64_t>(o0 + o) * wci + (g.identity ? 0 : c0 + c)) * taps;
                    float lo = Limits<float>::inf(), hi = -Limits<float>::inf();
                    for (int k = lane; k < taps; k += 32)
                    {
                        const float v = sgn * __ldg(wp + k);
                        lo = fminf(lo, v);
                        hi = fmaxf(hi, v);
                    }
#pragma unroll
                    for (int off = 16; off > 0; off >>= 1)
                    {
                        lo = fminf(lo, __shfl_xor_sync(0xffffffffu, lo, off));
                        hi = fmaxf(hi, __shfl_xor_sync(0xffffffffu, hi, off));
                    }
                    if (lane == 0) spair[e] = make_float2(hi, hi - lo);
                    for (int k = lane; k < taps; k += 32)
                    {
                        const float d = sgn * __ldg(wp + k) - hi;
                        const float ew = exp2_product(d, scale);
                        seb[(c * taps + k) * OB + o] = make_float2(ew, ew * d);
                    }
                }
            }
        }
        if constexpr (USE_TMA)
        {
            if (!mbar_wait(full + (n & 1), (n >> 1) & 1, a.wait_limit_ns))
            {
                if (threadIdx.x == 0 && a.errors != nullptr) atomicAdd(a.errors, 1u);
                return;  // every thread of the CTA waits on the same barrier and gives up together
            }
            if (border)
            {
                const T* src = xb + static_cast<int64_t>(first_channel + c0) * plane;
                fix_window_border(stage, src, plane, min(cc, a.chunk), g, tile_h0, tile_w0, fill0);
                if (mixed) fix_window_border(stage + slot_elems, src, plane, cc, g, tile_h0, tile_w0, Limits<T>::big());
                else if (cc > a.chunk) fix_window_border(stage + slot_elems, src + a.chunk * plane, plane, cc - a.chunk, g, tile_h0, tile_w0, fill0);
            }
        }
        __syncthreads();

        for (int c = 0; c < cc && warp_live; c++)
        {
            // Factorised path: range of x in the warp's block (once per channel) and what the warp's buffer holds.
            [[maybe_unused]] float x_lo = 0.0f, x_hi = 0.0f, held_s = 0.0f, held_scale = -1.0f, held_centre = 0.0f;
            [[maybe_unused]] bool have_range = false;
#pragma unroll
            for (int o = 0; o < OB; o++)
            {
                if (o >= o_count) break;
                const int os = o_base + o;   // position of the channel in the staged tables
                const T s = sa[(c * OB + os) * 2], scale = sa[(c * OB + os) * 2 + 1];
                const T* win = window_of(stage, c, s < T(0));
                T out[PATCH_H][PATCH_W];
                if constexpr (FACTOR)
                {
                    if (factorise)
                    {
                        const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
                        const float* origin = win + (8 * (warp >> 1)) * FactorLayout<KW>::STRIDE + 32 * wx;
                        if (!have_range)
                        {
                            factor_range<KW>(origin, lane, x_lo, x_hi, block_inside);
                            have_range = true;
                        }
                        const float2 pr = spair[c * OB + os];   // (Mw, range of w)
                        if (x_hi >= x_lo && scale * ((x_hi - x_lo) + pr.y) <= FACTOR_RANGE)
                        {
                            if (!(held_s == s && held_scale == scale))
                            {
                                held_centre = s > 0.0f ? x_hi : -x_lo;
                                factor_fill<KW>(origin, sea, s, scale, held_centre, lane);
                                held_s = s;
                                held_scale = scale;
                            }
                            float2 acc[PATCH_H][PATCH_W];
                            float rest[PATCH_H][PATCH_W];
                            factor_pair<KW>(sea, seb + c * taps * OB + os, OB, lane, acc, rest);
                            // out = s (Mx + Mw + N / S); the merge is a sum (a lone pair for identity), so the
                            // constant part is added up per output channel and joins the pixels at the end.
                            offset[o] += s * (held_centre + pr.x);
#pragma unroll
                            for (int rr = 0; rr < PATCH_H; rr++)
#pragma unroll
                                for (int j = 0; j < PATCH_W; j++)
                                    merged[o][rr][j] = fmaf((acc[rr][j].y + rest[rr][j]) * soft_rcp(acc[rr][j].x), s, merged[o][rr][j]);
                            continue;
                        }
                    }
                }
                if constexpr (KW == 3)
                {
#pragma unroll
                    for (int rr = 0; rr < PATCH_H; rr++)
                    {
                        T d[9][PATCH_W], e[9][PATCH_W], ref[PATCH_W], inv_sum[PATCH_W], out_d[PATCH_W];
                        smorph3_values(win, sw + c * taps * OB + os, OB, s, g, tx, ty, rr, d);
                        smorph3_softmax(d, scale, ref, e, inv_sum, out_d);
#pragma unroll
                        for (int j = 0; j < PATCH_W; j++) out[rr][j] = ref[j] + out_d[j];
                    }
                }
                else
                {
                    T ref[PATCH_H][PATCH_W], inv_sum[PATCH_H][PATCH_W];
                    smorph_pair<0, KW>(win, sw + c * taps * OB + os, OB, s, scale, g, tx, ty, ref, inv_sum, out);
                }
                // The merge mode is the same for every pixel: one switch around the pixel loops.
                auto for_pixels = [&](auto f) {
#pragma unroll
                    for (int rr = 0; rr < PATCH_H; rr++)
#pragma unroll
                        for (int j = 0; j < PATCH_W; j++) f(merged[o][rr][j], s * out[rr][j], target[o][rr][j]);
                };
                if constexpr (SOFT)
                {
#pragma unroll
                    for (int rr = 0; rr < PATCH_H; rr++)
#pragma unroll
                        for (int j = 0; j < PATCH_W; j++)
                        {
                            const T c = s * out[rr][j], t = soft_sign[o] * c;
                            const T top = soft_m[o][rr][j] < t ? t : soft_m[o][rr][j];
                            const T keep = soft_exp(soft_m[o][rr][j] - top, soft_scale[o]), q = soft_exp(t - top, soft_scale[o]);
                            soft_s[o][rr][j] = fma(soft_s[o][rr][j], keep, q);
                            merged[o][rr][j] = fma(merged[o][rr][j], keep, q * c);
                            soft_m[o][rr][j] = top;
                        }
                }
                else if constexpr (STATS)
                    for_pixels([](T& m, T v, T t) {
                        const T dist = v - t;
                        if (dist < T(1e-6) && dist > -T(1e-6)) m += T(1);
                    });
                else if (a.merge == MC_MERGE_MAX) for_pixels([](T& m, T v, T) { m = m < v ? v : m; });
                else if (a.merge == MC_MERGE_MIN) for_pixels([](T& m, T v, T) { m = v < m ? v : m; });
                else if (a.merge == MC_MERGE_IDENTITY) for_pixels([](T& m, T v, T) { m = v; });
                else for_pixels([](T& m, T v, T) { m = m + v; });
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
                if (o >= o_count || !warp_live || o0 + o_base + o >= g.Co || h >= g.H || w >= g.W) continue;
                T v = merged[o][rr][j];
                const int64_t at = ((static_cast<int64_t>(b) * g.Co + o0 + o_base + o) * g.H + h) * g.W + w;
                if constexpr (SOFT)
                {
                    const T inv = T(1) / soft_s[o][rr][j];
                    if (a.soft_ref != nullptr)
                    {
                        a.soft_ref[at] = soft_sign[o] * soft_m[o][rr][j];
                        a.soft_inv[at] = inv;
                    }
                    else a.y[at] = v * inv;
                    continue;
                }
                if constexpr (FACTOR) v += offset[o];
                if (!STATS && a.merge == MC_MERGE_AVERAGE) v = v / divisor;
                dst[at] = v;
            }
}

template <typename T, int KW, int OB, int MODE, bool USE_TMA>
int launch_smorph_forward_variant(const SmorphForwardArgs<T>& a, const CUtensorMap& tmap, int64_t blocks, size_t smem, cudaStream_t stream)
{
    auto kernel = smorph_forward_kernel<T, KW, OB, MODE, USE_TMA>;
    if (!allow_shared(kernel, smem))
    {
        set_last_error("cannot opt in to %zu bytes of shared memory", smem);
        return MC_ERR_UNSUPPORTED;
    }
    kernel<<<static_cast<unsigned>(blocks), THREADS, smem, stream>>>(a, tmap);
    return check_launch("smorph_forward_kernel");
}

template <typename T, int KW, int OB>
int launch_smorph_forward(const mc_desc& d, const T* x, const T* w, const T* alpha, T* y, const T* target, T* counts, cudaStream_t stream,
                          const T* beta = nullptr, T* soft_ref = nullptr, T* soft_inv = nullptr)
{
    SmorphForwardArgs<T> a;
    a.g = make_geometry(d, sizeof(T));
    a.g.replicate = false;  // out-of-image taps are excluded, never read
    a.x = x; a.w = w; a.alpha = alpha; a.y = y; a.target = target; a.counts = counts; a.merge = d.merge;
    a.beta = beta; a.soft_ref = soft_ref; a.soft_inv = soft_inv;
    a.o_groups = (d.Co + OB - 1) / OB;
    a.errors = device_error_counter();
    a.wait_limit_ns = wait_limit_ns();
    const int channels = a.g.identity ? 1 : d.Ci;
    const int64_t blocks = static_cast<int64_t>(a.g.tiles_x) * a.g.tiles_y * a.o_groups * d.B;
    if (blocks > 0x7fffffffLL) { set_last_error("too many tiles for one launch"); return MC_ERR_UNSUPPORTED; }
    // Per channel: two window slots (one per sign) per stage, the structuring elements, signs and scales.
    const size_t window = static_cast<size_t>(a.g.window_elems()) * sizeof(T);
    const bool stats = counts != nullptr;
    // The factorised path suits merges without a winner test: MAX / MIN compare the recomputed soft extremum
    // with the stored output within 1e-6, which only the same arithmetic in every pass guarantees.
    constexpr bool FACTOR = can_factorise<T, KW, false>();
    const bool soft = d.merge == MC_MERGE_SMOOTH;
    a.factorise = FACTOR && !stats && !soft && d.merge != MC_MERGE_MAX && d.merge != MC_MERGE_MIN;
    size_t small = 2 * (static_cast<size_t>(a.g.taps()) * OB + 2 * OB) * sizeof(T);  // up to two chunks of channels per stage
    size_t extra = 0;
    if (a.factorise)
    {
        small += 2 * (static_cast<size_t>(a.g.taps()) * OB + OB) * sizeof(float2);
        extra = 32 + (THREADS / 32) * static_cast<size_t>(FactorLayout<FACTOR ? KW : 3>::BYTES);
    }
    auto plan = [&](int stages, int& chunk, size_t& smem) {
        const size_t per_channel = stages * 2 * window + small, fixed = 128 + stages * 2 * 128 + extra;
        if (per_channel + fixed > MAX_SHARED_BYTES) return false;
        chunk = static_cast<int>(((a.factorise ? 112 : 100) * 1024 - fixed) / per_channel);
        chunk = std::max(1, std::min(std::min(chunk, 8), channels));
        smem = fixed + per_channel * chunk;
        return true;
    };
    CUtensorMap tmap{};
    int chunk = 1;
    size_t smem = 0;
    if (plan(2, chunk, smem) && make_window_tensor_map(&tmap, x, sizeof(T), d.B, d.Ci, d.H, d.W, a.g.win_stride, a.g.win_rows, chunk))
    {
        a.chunk = chunk;
        if (soft) return launch_smorph_forward_variant<T, KW, OB, 2, true>(a, tmap, blocks, smem, stream);
        return stats ? launch_smorph_forward_variant<T, KW, OB, 1, true>(a, tmap, blocks, smem, stream)
                     : launch_smorph_forward_variant<T, KW, OB, 0, true>(a, tmap, blocks, smem, stream);
    }
    if (!plan(1, chunk, smem))
    {
        set_last_error("structuring element %dx%d too large for shared memory", d.kH, d.kW);
        return MC_ERR_UNSUPPORTED;
    }
    a.chunk = chunk;
    if (soft) return launch_smorph_forward_variant<T, KW, OB, 2, false>(a, tmap, blocks, smem, stream);
    return stats ? launch_smorph_forward_variant<T, KW, OB, 1, false>(a, tmap, blocks, smem, stream)
                 : launch_smorph_forward_variant<T, KW, OB, 0, false>(a, tmap, blocks, smem, stream);
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
    const T* beta;      // smooth merge: one value per output channel
    const T* soft_ref;  // smooth merge: extremum of the channel outputs per output pixel
    const T* soft_inv;  // smooth merge: 1 / sum_i q_i per output pixel
    T* gbeta;           // smooth merge: gradient of beta
    int o_chunk;      // output channels whose weights and bins are staged together
    int grad_stage;   // byte offset in shared memory of the per-thread slots of grad_output (3 x 3 float kernels)
    int grad_async;   // grad_output is 16-byte aligned row by row: the slots are filled by cp.async one channel ahead
    T scale;          // 1 / Ci for AVERAGE
    int factorise;    // 5 x 5 and 7 x 7 float kernels: S and N of a pair from the factorised sums where that is safe
    int bounded;      // 3 x 3 float kernels: exponentials relative to a bound of the patch where that is safe
};

/// 3 x 3 float kernels may skip the maximum (smorph3_pair_backward_bounded) while scale * (widest range of x in the window
/// of one thread of the warp + range of w) stays below this many binades: with the reference in the middle of the range the
/// exponentials stay within 2^-(48 + range of w) .. 2^48 and their sums of squares below 2^65.
constexpr float BOUND_RANGE = 96.0f;
template <typename T, int KH, int KW, bool SOFT>
__host__ __device__ constexpr bool backward_bounds() { return sizeof(T) == 4 && !SOFT && KH == 3 && KW == 3; }

/// Backward of one pair for the thread's patch. Recomputes the forward state (ref, S, out), then every tap
/// k of every pixel contributes
///     c_k = p_k g + alpha p_k g (v_k - out),   p_k g = e_k (g / S)
/// to grad_input at the pixel the tap read and to grad_weight, and p_k g (v_k - ref)(v_k - out) to
/// grad_alpha (csrc/cpp/smorph_cpu_kernels.hxx:149-206). In the u domain alpha (v_k - out) = |alpha| (u_k - out_u)
/// and (v_k - ref)(v_k - out) = (u_k - ref_u)(u_k - out_u), so with g the gradient of out itself the sums need
/// no sign correction. Excluded taps have e_k = 0 exactly and contribute exact zeros.
/// grad_input: with KH > 0 every tap offset is a compile-time constant and the contributions are summed in
/// the thread's register window gxr (patch + halo); otherwise they go to the shared window with atomics.
/// grad_weight: the 8 pixels of the thread, then the warp, are summed per tap; lane 0 stores the warp's
/// total in the warp's private bins (no atomics, no barrier).
template <int KH, int KW, typename T, int GH, int GW>
__device__ __forceinline__ void smorph_pair_backward(const T* __restrict__ win, const T* __restrict__ swk, T* __restrict__ sg, T* __restrict__ wbin,
                                                     T* __restrict__ abin, T s, T abs_alpha, T scale, const T (&grad)[PATCH_H][PATCH_W],
                                                     const Geometry& g, int tx, int ty, int lane, T (&gxr)[GH][GW])
{
    const int kwr = KW > 0 ? KW : g.kW;
    T ref[PATCH_H][PATCH_W], inv_sum[PATCH_H][PATCH_W], out[PATCH_H][PATCH_W];
    smorph_pair<0, KW>(win, swk, 1, s, scale, g, tx, ty, ref, inv_sum, out);  // kernel rows not unrolled: smaller code, fewer live registers

    T scaled[PATCH_H][PATCH_W], minus_ref[PATCH_H][PATCH_W], out_d[PATCH_H][PATCH_W];
#pragma unroll
    for (int rr = 0; rr < PATCH_H; rr++)
#pragma unroll
        for (int j = 0; j < PATCH_W; j++)
        {
            scaled[rr][j] = grad[rr][j] * inv_sum[rr][j];
            minus_ref[rr][j] = -ref[rr][j];
            out_d[rr][j] = out[rr][j] - ref[rr][j];
        }

    T alpha_sum = T(0), tap_sum = T(0);
    int current = -1;
    auto flush_tap = [&](int k) {
        const T total = warp_sum(tap_sum);
        if (lane == 0) wbin[k] = total;
        tap_sum = T(0);
    };
    for_each_tap<KH, KW>(win, g, tx, ty, [&](int kh, int kw, int rr, int j, T xv) {
        const int k = kh * kwr + kw;
        if (k != current)
        {
            if (current >= 0) flush_tap(current);
            current = k;
        }
        const T d = fma(s, xv, minus_ref[rr][j]) + swk[k];   // as in smorph_pair
        const T pg = soft_exp(d, scale) * scaled[rr][j];
        const T centered = d - out_d[rr][j];
        const T c = fma(abs_alpha * pg, centered, pg);
        if constexpr (KH > 0) gxr[rr + KH - 1 - kh][j + KW - 1 - kw] += c;
        else if (c != T(0)) atomic_add(sg + (ty * PATCH_H + rr + g.kH - 1 - kh) * g.win_stride + tx * PATCH_W + g.seg_off + j + g.kW - 1 - kw, c);
        tap_sum += c;
        alpha_sum = fma(pg * d, centered, alpha_sum);
    });
    flush_tap(current);
    alpha_sum = warp_sum(alpha_sum);
    if (lane == 0) *abin = alpha_sum;
}

/// float kernels with square 5 x 5 and 7 x 7 structuring elements split the backward of a pair into per-pixel
/// statistics (the soft extremum out_u and the sum of the exponentials) and one gradient pass over the taps
/// (smorph_taps_backward); the statistics come from the factorised sums where that is safe (backward_factorises,
/// smorph_stats_factored) and from the max-subtracting passes otherwise (smorph_stats_stable).
template <typename T, int KH, int KW>
__host__ __device__ constexpr bool backward_splits() { return sizeof(T) == 4 && KH == KW && KW >= 5 && KW <= 7; }
template <typename T, int KH, int KW, bool SOFT>
__host__ __device__ constexpr bool backward_factorises() { return backward_splits<T, KH, KW>() && !SOFT; }

/// Statistics of one pair from the factorised form (see "Factorised forward"): `ea` holds (E, A) of the warp's block for
/// this pair's sign and scale, `eb` the pair's (Ew, Bw), and ref = mx + mw (the block's largest s x plus the largest
/// s w_k) bounds every u_k from above. factor_pair gives S = sum_k 2^(scale (u_k - ref)) and
/// N = sum_k 2^(scale (u_k - ref)) (u_k - ref - shift) in three fused multiply-adds per tap, no maximum and no
/// exponential; `shift` (<= 0) is the thread's own largest s x minus mx, and `base` = ref + shift formed directly.
/// Out: centre = out_u = base + N / S, and scaled = g / S' with S' = sum_k 2^(scale (u_k - out_u)) = S 2^(scale (ref - out_u)),
/// the sum the gradient pass works with.
template <int KW>
__device__ __forceinline__ void smorph_stats_factored(const float4* __restrict__ ea, const float2* __restrict__ eb, int lane, float scale, float base,
                                                      float shift, float mx, float mw, bool precise, const float (&grad)[PATCH_H][PATCH_W],
                                                      float (&centre)[PATCH_H][PATCH_W], float (&scaled)[PATCH_H][PATCH_W])
{
    float2 acc[PATCH_H][PATCH_W];
    float rest[PATCH_H][PATCH_W];
    factor_pair<KW, true>(ea, eb, 1, lane, acc, rest, shift);
    float ref_hi, ref_lo;   // Mx + Mw without rounding
    two_sum(mx, mw, ref_hi, ref_lo);
#pragma unroll
    for (int rr = 0; rr < PATCH_H; rr++)
#pragma unroll
        for (int j = 0; j < PATCH_W; j++)
        {
            // A pixel far outside the image (partial tiles) has no tap at all: S = 0, and it carries no gradient.
            const float inv_sum = acc[rr][j].x > 0.0f ? soft_rcp(acc[rr][j].x) : 0.0f;
            // out_u = ref + shift + N / S, with `base` = ref + shift formed by the caller without the detour through ref: the
            // quotient is small, so out_u rounds at its own size. out_u - ref (for S') may round at the size of the range.
            const float quotient = (acc[rr][j].y + rest[rr][j]) * inv_sum;
            centre[rr][j] = base + quotient;
            // 1 / S' = 2^(scale (out_u - Mx - Mw)) / S, a factor of every c_k of the pixel: its exponent has to be as exact
            // as the float out_u the gradient pass will use. Beyond a few binades (`precise`, warp uniform) the difference is
            // taken without rounding (two-sum) and its tail goes into the exponent.
            float factor;
            if (precise)
            {
                float z, tail;
                two_sum(centre[rr][j], -ref_hi, z, tail);
                factor = exp2_product(fminf(z, 0.0f), scale, tail - ref_lo);
            }
            else factor = ex2_approx(fminf(scale * (quotient + shift), 0.0f));
            scaled[rr][j] = grad[rr][j] * (inv_sum * factor);   // 1 / S' <= 1 first: no overflow
        }
}

/// The same statistics from the max-subtracting passes (any alpha, any range of the inputs).
template <int KW>
__device__ __forceinline__ void smorph_stats_stable(const float* __restrict__ win, const float* __restrict__ swk, float s, float scale,
                                                    const Geometry& g, int tx, int ty, const float (&grad)[PATCH_H][PATCH_W],
                                                    float (&centre)[PATCH_H][PATCH_W], float (&scaled)[PATCH_H][PATCH_W])
{
    float ref[PATCH_H][PATCH_W], inv_sum[PATCH_H][PATCH_W];
    smorph_pair<0, KW>(win, swk, 1, s, scale, g, tx, ty, ref, inv_sum, centre);
#pragma unroll
    for (int rr = 0; rr < PATCH_H; rr++)
#pragma unroll
        for (int j = 0; j < PATCH_W; j++)
            // out_u <= ref; the clamp only matters for pixels far outside the image, whose ref and out_u are both -1e30
            // up to rounding and whose gradient is zero.
            scaled[rr][j] = grad[rr][j] * inv_sum[rr][j] * ex2_approx(fminf(scale * (centre[rr][j] - ref[rr][j]), 0.0f));
}

/// Gradient pass of one pair for the thread's patch, exponentials taken relative to the soft extremum itself:
///     t_k = u_k - out_u = s x + (s w_k - out_u),   e_k = 2^(scale t_k),   G = g / sum_k e_k  (`scaled`),
///     c_k = e_k (G + |alpha| G t_k)                      to grad_input (register window) and grad_weight,
///     d out / d alpha = (1 / sum_k e_k) sum_k e_k t_k^2  (the e-weighted mean of t_k is zero).
/// |alpha| (max_k u_k - out_u) is at most about ln(taps), so e_k stays below 2^5, and the taps that carry the weight
/// have small t_k, formed by one fused multiply-add: their exponentials are as exact as with the maximum subtracted.
/// One exponential and ten instructions per tap. The KW tap sums of a kernel row are added over the warp through its
/// scratch `red` (see smorph3_pair_backward).
template <int KW>
__device__ __forceinline__ void smorph_taps_backward(const float* __restrict__ win, const float* __restrict__ swk, float* __restrict__ wbin,
                                                     float* __restrict__ abin, float* __restrict__ red, float s, float abs_alpha, float scale,
                                                     const float (&centre)[PATCH_H][PATCH_W], const float (&scaled)[PATCH_H][PATCH_W], int tx, int ty,
                                                     int lane, float (&gxr)[PATCH_H + KW - 1][PATCH_W + KW - 1])
{
    constexpr int LEN = segment_len(KW, 4), OFF = segment_offset(KW, 4), STRIDE = window_stride(KW, 4);
    static_assert(KW <= RED_ROWS, "one scratch row per tap of a kernel row");
    // Two horizontally adjacent pixels per step: apart from the first difference (scalar, so that the pair is assembled
    // without register moves), the exponentials and the register window of grad_input, every operation is a packed
    // two-lane instruction (add / mul / fma.f32x2).
    float2 steep[PATCH_H][PATCH_W / 2], scaled2[PATCH_H][PATCH_W / 2], spread[PATCH_H][PATCH_W / 2];
    float minus_centre[PATCH_H][PATCH_W];
#pragma unroll
    for (int rr = 0; rr < PATCH_H; rr++)
#pragma unroll
        for (int jp = 0; jp < PATCH_W / 2; jp++)
        {
            scaled2[rr][jp] = make_float2(scaled[rr][2 * jp], scaled[rr][2 * jp + 1]);
            steep[rr][jp] = make_float2(abs_alpha * scaled[rr][2 * jp], abs_alpha * scaled[rr][2 * jp + 1]);
            spread[rr][jp] = make_float2(0.0f, 0.0f);
            minus_centre[rr][2 * jp] = -centre[rr][2 * jp];
            minus_centre[rr][2 * jp + 1] = -centre[rr][2 * jp + 1];
        }
    const float2 scale2 = make_float2(scale, scale);
#pragma unroll
    for (int kh = 0; kh < KW; kh++)
    {
        float seg[PATCH_H][LEN];
#pragma unroll
        for (int rr = 0; rr < PATCH_H; rr++) load_segment<LEN>(seg[rr], win + (ty * PATCH_H + rr + KW - 1 - kh) * STRIDE + tx * PATCH_W);
        float tap_sum[KW];
#pragma unroll
        for (int kw = 0; kw < KW; kw++)
        {
            const float wv = swk[kh * KW + kw];
            const float2 wv2 = make_float2(wv, wv);
            float2 sum = make_float2(0.0f, 0.0f);
#pragma unroll
            for (int rr = 0; rr < PATCH_H; rr++)
#pragma unroll
                for (int jp = 0; jp < PATCH_W / 2; jp++)
                {
                    const int j = 2 * jp, at = OFF + j + KW - 1 - kw;
                    // t = (s x - centre) + s w, as in smorph_pair
                    const float2 t = __fadd2_rn(make_float2(fmaf(s, seg[rr][at], minus_centre[rr][j]), fmaf(s, seg[rr][at + 1], minus_centre[rr][j + 1])), wv2);
                    const float2 arg = __fmul2_rn(t, scale2);
                    const float2 e = make_float2(ex2_approx(arg.x), ex2_approx(arg.y));   // exactly 0 for an excluded tap (t = -1e30)
                    const float2 et = __fmul2_rn(e, t);   // e first: an excluded tap gives 0 * -1e30 = -0, never an overflow
                    const float2 c = __ffma2_rn(steep[rr][jp], et, __fmul2_rn(e, scaled2[rr][jp]));
                    gxr[rr + KW - 1 - kh][j + KW - 1 - kw] += c.x;
                    gxr[rr + KW - 1 - kh][j + KW - kw] += c.y;
                    sum = __fadd2_rn(sum, c);
                    spread[rr][jp] = __ffma2_rn(et, t, spread[rr][jp]);
                }
            tap_sum[kw] = sum.x + sum.y;
        }
        __syncwarp();
#pragma unroll
        for (int kw = 0; kw < KW; kw++) red[kw * RED_STRIDE + lane] = tap_sum[kw];
        __syncwarp();
        float part = 0.0f;
        if (lane < 3 * KW)
        {
            const float* strip = red + (lane / 3) * RED_STRIDE + (lane % 3) * 11;
            const int n = (lane % 3) == 2 ? 10 : 11;
#pragma unroll
            for (int c = 0; c < 11; c++)
                if (c < n) part += strip[c];
        }
        part += __shfl_down_sync(0xffffffffu, part, 1) + __shfl_down_sync(0xffffffffu, part, 2);
        if (lane < 3 * KW && lane % 3 == 0) wbin[kh * KW + lane / 3] = part;
    }
    float alpha_sum = 0.0f;
#pragma unroll
    for (int rr = 0; rr < PATCH_H; rr++)
#pragma unroll
        for (int jp = 0; jp < PATCH_W / 2; jp++)
            alpha_sum = fmaf(spread[rr][jp].y, scaled[rr][2 * jp + 1], fmaf(spread[rr][jp].x, scaled[rr][2 * jp], alpha_sum));
    alpha_sum = warp_sum(alpha_sum);
    if (lane == 0) *abin = alpha_sum;
}

/// CTA = (batch element, input channel, tile), looping over the output channels in chunks: the sign-folded
/// structuring elements and the per-warp gradient bins of a whole chunk live in shared memory, so the loop
/// over the chunk's output channels runs without a barrier.
/// SOFT: the smooth channel merge (its own instantiation, so that the other merges keep their register allocation).
/// FAST (3 x 3 float, sum / mean merges, grad_output aligned for cp.async): the channel loop holds nothing but the
/// staging of the next channel's gradients and the bounded form of the pair, see there.
template <typename T, int KH, int KW, bool SOFT, bool FAST = false>
__global__ void __launch_bounds__(THREADS, (sizeof(T) == 8 || KH >= 5) ? 1 : 2) smorph_backward_kernel(const SmorphBackwardArgs<T> a)
{
    static_assert(!FAST || (sizeof(T) == 4 && KH == 3 && KW == 3 && !SOFT), "the fast loop is the 3 x 3 float kernel's");
    extern __shared__ __align__(16) unsigned char smem_raw[];
    constexpr int WARPS = THREADS / 32;
    constexpr int GH = KH > 0 ? PATCH_H + KH - 1 : 1, GW = KH > 0 ? PATCH_W + KW - 1 : 1;
    const Geometry& g = a.g;
    const int taps = KH > 0 ? KH * KW : g.taps();   // a compile-time constant for the specialised widths
    const int welems = KH > 0 ? (TILE_H + KH - 1) * window_stride(KW > 0 ? KW : 1, sizeof(T)) : g.window_elems();
    const int OC = a.o_chunk;
    T* sx = reinterpret_cast<T*>(smem_raw);   // [2][window]: x with -big / +big outside the image
    T* sg = sx + 2 * welems;                   // gradient window
    T* sw = sg + welems;                       // [OC][taps], sign folded
    T* spar = sw + OC * taps;                  // [OC][3]: sign, |alpha|, exp scale
    T* wbins = spar + OC * 3;                  // [WARPS][OC][taps]
    T* abins = wbins + WARPS * OC * taps;      // [WARPS][OC]
    T* bbins = abins + WARPS * OC;             // [WARPS][OC]: gradient of beta (smooth merge)
    T* red = bbins + WARPS * OC + (threadIdx.x >> 5) * RED_ROWS * RED_STRIDE;  // this warp's reduction scratch
    // Factorised recomputation of S and N (backward_factorises): [OC][taps] (Ew, Bw), [OC] (Mw, range of w), one (E, A) buffer per warp.
    constexpr bool FACTOR = backward_factorises<T, KH, KW, SOFT>();
    constexpr bool BOUNDED = backward_bounds<T, KH, KW, SOFT>();   // needs [OC] (Mw, range of w) and the ranges of x only
    constexpr int FKW = backward_splits<T, KH, KW>() ? KW : 3;
    float2* seb = reinterpret_cast<float2*>(smem_raw + (reinterpret_cast<unsigned char*>(bbins + WARPS * OC + WARPS * RED_ROWS * RED_STRIDE) - smem_raw + 15) / 16 * 16);
    float2* spair = seb + (FACTOR ? OC * taps : 0);
    // 3 x 3 bounded form: [OC][BOUNDED_ROW], scale (s w_k - Mw) twice per tap (smorph3_pair_backward_bounded).
    [[maybe_unused]] float* sshift = reinterpret_cast<float*>(smem_raw + (reinterpret_cast<unsigned char*>(spair + OC) - smem_raw + 15) / 16 * 16);
    float4* sea = reinterpret_cast<float4*>(smem_raw + (reinterpret_cast<unsigned char*>(spair + OC) - smem_raw + 15) / 16 * 16)
                  + (threadIdx.x >> 5) * (FactorLayout<FKW>::BYTES / 16);
    const bool factorise = FACTOR && a.factorise != 0;
    const bool bounded = BOUNDED && a.bounded != 0;

    const int tiles = g.tiles_x * g.tiles_y;
    const int ci = blockIdx.x % g.Ci;
    const int tile = (blockIdx.x / g.Ci) % tiles;
    const int b = blockIdx.x / (g.Ci * tiles);
    const int tile_h0 = (tile / g.tiles_x) * TILE_H, tile_w0 = (tile % g.tiles_x) * TILE_W;
    // When the right half of the tile is outside the image the two warps of a warp row share the left block and
    // take every other output channel of the chunk (thread_patch_split): their register windows of grad_input
    // meet in the shared window, their bins are per warp anyway.
    int tx, ty, half;
    bool warp_live, split;
    thread_patch_split(tile_h0, tile_w0, g.H, g.W, !g.identity, tx, ty, warp_live, split, half);
    const int o_step = split ? 2 : 1;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int64_t plane = g.plane();
    const int wci = g.identity ? 1 : g.Ci;
    const int wi = g.identity ? 0 : ci;
    const bool winner_takes_all = a.merge == MC_MERGE_MAX || a.merge == MC_MERGE_MIN;
    const int o_begin = g.identity ? ci : 0;
    const int o_end = g.identity ? ci + 1 : g.Co;

    bool has_pos = false, has_neg = false;
    for (int o = o_begin + threadIdx.x; o < o_end; o += THREADS)
    {
        const T al = __ldg(a.alpha + (g.identity ? o : static_cast<int64_t>(o) * g.Ci + ci));
        has_pos |= al >= T(0);
        has_neg |= al < T(0);
    }
    has_pos = __syncthreads_or(has_pos);
    has_neg = __syncthreads_or(has_neg);
    load_window_signed(has_pos ? sx : nullptr, has_neg ? sx + welems : nullptr, a.x + (static_cast<int64_t>(b) * g.Ci + ci) * plane, g, tile_h0,
                       tile_w0);
    for (int e = threadIdx.x; e < welems; e += THREADS) sg[e] = T(0);
    for (int e = (threadIdx.x & 31); e < RED_ROWS * RED_STRIDE; e += 32) red[e] = T(0);   // pad columns stay zero
    if (a.grad_stage != 0)
    {
        float4* zero = reinterpret_cast<float4*>(smem_raw + a.grad_stage);
        for (int e = threadIdx.x; e < 2 * THREADS * PATCH_H * PATCH_W / 4; e += THREADS) zero[e] = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    }

    bool live[PATCH_H][PATCH_W];
    int64_t at0[PATCH_H];
#pragma unroll
    for (int rr = 0; rr < PATCH_H; rr++)
    {
        const int h = tile_h0 + ty * PATCH_H + rr;
        at0[rr] = (static_cast<int64_t>(b) * g.Co * g.H + h) * g.W + tile_w0 + tx * PATCH_W;
#pragma unroll
        for (int j = 0; j < PATCH_W; j++) live[rr][j] = h < g.H && tile_w0 + tx * PATCH_W + j < g.W;
    }
    auto load_grad = [&](int o, T (&dst)[PATCH_H][PATCH_W]) {
#pragma unroll
        for (int rr = 0; rr < PATCH_H; rr++)
#pragma unroll
            for (int j = 0; j < PATCH_W; j++) dst[rr][j] = live[rr][j] ? __ldg(a.gy + at0[rr] + static_cast<int64_t>(o) * plane + j) * a.scale : T(0);
    };

    // Register window of grad_input: patch plus halo; column pairs in the 3 x 3 float kernels (GradWindow3).
    constexpr bool PAIRED_WINDOW = sizeof(T) == 4 && KH == 3 && KW == 3;
    std::conditional_t<PAIRED_WINDOW, GradWindow3, T[GH][GW]> gxr;
    auto window = [&](int r, int c) -> T& {
        if constexpr (PAIRED_WINDOW) return window_at(gxr, r, c);
        else return gxr[r][c];
    };
#pragma unroll
    for (int r = 0; r < GH; r++)
#pragma unroll
        for (int c = 0; c < GW; c++) window(r, c) = T(0);

    // Factorised path: the warp's block of the window (32 x 8 pixels plus halo), the range of x in it (taken once, after
    // the first barrier below) and what the warp's (E, A) buffer holds.
    [[maybe_unused]] const int block_at = 8 * (warp >> 1) * g.win_stride + 32 * (split ? 0 : (warp & 1));
    [[maybe_unused]] float x_lo = 0.0f, x_hi = 0.0f, held_s = 0.0f, held_scale = -1.0f, held_centre = 0.0f;
    [[maybe_unused]] bool have_range = false;
    [[maybe_unused]] float local_lo = Limits<float>::inf(), local_hi = -Limits<float>::inf();
    [[maybe_unused]] float local_mid = 0.0f;   // 3 x 3 bounded form: the middle of the thread's own range of x
    [[maybe_unused]] float bound_range = Limits<float>::inf();   // 3 x 3: range of x in the block, infinite while unknown or unusable

    for (int oc0 = o_begin; oc0 < o_end; oc0 += OC)
    {
        const int oc = min(OC, o_end - oc0);
        __syncthreads();
        for (int e = threadIdx.x; e < oc; e += THREADS)
        {
            const T al = __ldg(a.alpha + (g.identity ? oc0 + e : static_cast<int64_t>(oc0 + e) * g.Ci + ci));
            const T ab = al >= T(0) ? al : -al;
            spar[e * 3] = al >= T(0) ? T(1) : T(-1);
            spar[e * 3 + 1] = ab;
            spar[e * 3 + 2] = exp_scale(ab);
        }
        for (int e = threadIdx.x; e < oc * taps; e += THREADS)
        {
            const int k = e % taps, oo = e / taps;
            const T al = __ldg(a.alpha + (g.identity ? oc0 + oo : static_cast<int64_t>(oc0 + oo) * g.Ci + ci));
            const T v = __ldg(a.w + (static_cast<int64_t>(oc0 + oo) * wci + wi) * taps + k);
            sw[e] = al >= T(0) ? v : -v;
        }
        for (int e = threadIdx.x; e < WARPS * OC * (taps + 2); e += THREADS) wbins[e] = T(0);  // bins of warps that skip stay zero
        if constexpr (FACTOR || BOUNDED)
        {
            if (factorise || bounded)
            {
                // One warp per pair, one lane per tap (two for 7 x 7): Mw and the range of s w by shuffles, then (Ew, Bw).
                for (int oo = warp; oo < oc; oo += WARPS)
                {
                    const float al = __ldg(a.alpha + (g.identity ? oc0 + oo : static_cast<int64_t>(oc0 + oo) * g.Ci + ci));
                    const float sgn = al >= 0.0f ? 1.0f : -1.0f, scale = exp_scale(fabsf(al));
                    const float* wp = a.w + (static_cast<int64_t>(oc0 + oo) * wci + wi) * taps;
                    float lo = Limits<float>::inf(), hi = -Limits<float>::inf();
                    for (int k = lane; k < taps; k += 32)
                    {
                        const float v = sgn * __ldg(wp + k);
                        lo = fminf(lo, v);
                        hi = fmaxf(hi, v);
                    }
#pragma unroll
                    for (int off = 16; off > 0; off >>= 1)
                    {
                        lo = fminf(lo, __shfl_xor_sync(0xffffffffu, lo, off));
                        hi = fmaxf(hi, __shfl_xor_sync(0xffffffffu, hi, off));
                    }
                    if (lane == 0) spair[oo] = make_float2(hi, hi - lo);
                    if constexpr (BOUNDED)
                    {
                        if (lane < BOUNDED_PARAMS / 2)
                        {
                            const float v = lane < 9 ? scale * (sgn * __ldg(wp + lane) - hi) : 0.0f;
                            reinterpret_cast<float2*>(sshift + oo * BOUNDED_ROW)[lane] = make_float2(v, v);
                        }
                        else if (lane == BOUNDED_PARAMS / 2)
                        {
                            const bool usable = scale >= BOUNDED_SCALE_MIN && scale <= BOUNDED_SCALE_MAX;
                            *reinterpret_cast<float4*>(sshift + oo * BOUNDED_ROW + BOUNDED_PARAMS) =
                                make_float4(sgn * scale, fabsf(al) / scale, 1.0f / (scale * scale), usable ? BOUND_RANGE / scale - (hi - lo) : -1.0f);
                        }
                    }
                    if constexpr (FACTOR)
                        for (int k = lane; k < taps; k += 32)
                        {
                            const float d = sgn * __ldg(wp + k) - hi;
                            const float ew = exp2_product(d, scale);
                            seb[oo * taps + k] = make_float2(ew, ew * d);
                        }
                }
            }
        }
        __syncthreads();

        if (warp_live)
        {
            if constexpr (FACTOR || BOUNDED)
            {
                if ((factorise || bounded) && !have_range)
                {
                    const int r0 = tile_h0 - g.halo_top() + 8 * (warp >> 1), c0 = tile_w0 - g.halo_left() + 32 * (split ? 0 : (warp & 1));
                    const bool inside = r0 >= 0 && r0 + FactorLayout<FKW>::ROWS <= g.H && c0 >= 0 && c0 + FactorLayout<FKW>::WS <= g.W;
                    factor_range<FKW>((has_pos ? sx : sx + welems) + block_at, lane, x_lo, x_hi, inside);
                    have_range = true;
                    // Largest and smallest x the thread's own pixels can read: the centre of its linear sums (factor_pair).
                    constexpr int LEN = segment_len(FKW, 4), OFF = segment_offset(FKW, 4);
                    for (int r = 0; r < PATCH_H + FKW - 1; r++)
                    {
                        float seg[LEN];
                        load_segment<LEN>(seg, (has_pos ? sx : sx + welems) + (ty * PATCH_H + r) * g.win_stride + tx * PATCH_W);
#pragma unroll
                        for (int c = OFF; c < OFF + PATCH_W + FKW - 1; c++)
                        {
                            local_lo = fminf(local_lo, seg[c] > -1e29f ? seg[c] : Limits<float>::inf());
                            local_hi = fmaxf(local_hi, seg[c] < 1e29f ? seg[c] : -Limits<float>::inf());
                        }
                    }
                    if constexpr (BOUNDED)
                    {
                        // The decision to skip the maximum must be the same for the whole warp (both forms reduce over the
                        // warp): it rests on the widest range any of its threads sees in its own window, which bounds that
                        // thread's exponents. A thread whose window lies outside the image reads no tap that counts and
                        // takes the block's extremes as its (finite) bound.
                        if (!(local_hi >= local_lo))
                        {
                            local_hi = x_hi;
                            local_lo = x_hi;
                        }
                        local_mid = 0.5f * local_lo + 0.5f * local_hi;
                        const float widest = from_ordered(__reduce_max_sync(0xffffffffu, to_ordered(local_hi - local_lo)));
                        if (x_hi >= x_lo) bound_range = widest;
                    }
                }
            }
            // Fast loop of the 3 x 3 float kernels for the usual training case (sum / mean merge, aligned grad_output):
            // nothing but the staging of the next channel's gradients, one read of the pair's parameter row and the
            // bounded form; a pair whose exponents are too wide for it takes the max-subtracting form.
            if constexpr (FAST)
            {
                {
                    constexpr int BUFFER = THREADS * PATCH_H * PATCH_W;
                    float* slot_now = reinterpret_cast<float*>(smem_raw + a.grad_stage) + threadIdx.x * (PATCH_H * PATCH_W);
                    float* slot_next = slot_now + BUFFER;
                    const bool live0 = live[0][0], live1 = live[1][0];
                    const float* gy_next = a.gy + at0[0] + static_cast<int64_t>(oc0 + half) * plane;
                    const int64_t gy_step = static_cast<int64_t>(o_step) * plane;
                    if (half < oc)
                    {
                        if (live0) cp_async_16(slot_now, gy_next);
                        if (live1) cp_async_16(slot_now + PATCH_W, gy_next + g.W);
                    }
                    constexpr float grad_scale = 1.0f;   // the mean merge's 1 / Ci multiplies the totals instead (below)
                    const float* row = sshift + half * BOUNDED_ROW;
                    float* wbin = reinterpret_cast<float*>(wbins) + (warp * OC + half) * 9;
                    float* abin = reinterpret_cast<float*>(abins) + warp * OC + half;
                    for (int oo = half; oo < oc; oo += o_step)
                    {
                        cp_async_wait_all();
                        gy_next += gy_step;
                        if (oo + o_step < oc)
                        {
                            if (live0) cp_async_16(slot_next, gy_next);
                            if (live1) cp_async_16(slot_next + PATCH_W, gy_next + g.W);
                        }
                        const float4 params = *reinterpret_cast<const float4*>(row + BOUNDED_PARAMS);
                        const bool neg = params.x < 0.0f;
                        const float* win = reinterpret_cast<const float*>(sx) + (neg ? welems : 0);
                        if (bound_range <= params.w)
                            smorph3_pair_backward_bounded(win, reinterpret_cast<const float4*>(row), wbin, abin, reinterpret_cast<float*>(red), params,
                                                          neg ? -local_mid : local_mid, slot_now, grad_scale, tx, ty, lane, gxr);
                        else
                        {
                            float grad[PATCH_H][PATCH_W];
#pragma unroll
                            for (int rr = 0; rr < PATCH_H; rr++)
#pragma unroll
                                for (int j = 0; j < PATCH_W; j++) grad[rr][j] = slot_now[rr * PATCH_W + j] * grad_scale;
                            smorph3_pair_backward(win, reinterpret_cast<const float*>(sw) + oo * 9, wbin, abin, reinterpret_cast<float*>(red),
                                                  static_cast<float>(spar[oo * 3]), static_cast<float>(spar[oo * 3 + 1]),
                                                  static_cast<float>(spar[oo * 3 + 2]), grad, g, tx, ty, lane, gxr);
                        }
                        float* swap = slot_now;
                        slot_now = slot_next;
                        slot_next = swap;
                        row += o_step * BOUNDED_ROW;
                        wbin += o_step * 9;
                        abin += o_step;
                    }
                }
            }
            else
            {
                // The 3 x 3 float kernel has no registers to spare for the next channel's gradients (it spills at 128): its
                // loads are covered by the other warps instead.
                constexpr bool PREFETCH = !(KH == 3 && sizeof(T) == 4);
                // Kernels without registers to spare for the next channel's gradients (PREFETCH false) keep them in shared
                // memory instead: the thread's two 16-byte rows of the NEXT output channel travel by cp.async into a private
                // slot while the current channel computes (rows outside the image are never copied and stay zero), and the
                // pair's arithmetic reads each pair of gradients from the slot at the point where it needs them. When
                // grad_output is not 16-byte aligned the slot is filled with plain loads at the top of the iteration.
                [[maybe_unused]] float* slots = nullptr;
                [[maybe_unused]] int staged = 0;
                if constexpr (!PREFETCH)
                {
                    slots = reinterpret_cast<float*>(smem_raw + a.grad_stage) + threadIdx.x * (PATCH_H * PATCH_W);
                    if (a.grad_async != 0 && half < oc)
                    {
    #pragma unroll
                        for (int rr = 0; rr < PATCH_H; rr++)
                            if (live[rr][0]) cp_async_16(slots + rr * PATCH_W, a.gy + at0[rr] + static_cast<int64_t>(oc0 + half) * plane);
                    }
                }
                T grad[PATCH_H][PATCH_W];   // PREFETCH false: a temporary of the steps that need all eight values at once
                [[maybe_unused]] T next[PREFETCH ? PATCH_H : 1][PREFETCH ? PATCH_W : 1];
                if constexpr (PREFETCH)
                    if (half < oc) load_grad(oc0 + half, grad);
                for (int oo = half; oo < oc; oo += o_step)
                {
                    const int o = oc0 + oo;
                    [[maybe_unused]] float* slot = nullptr;      // PREFETCH false: where this channel's gradients are
                    [[maybe_unused]] float grad_scale = 1.0f;    // and what they are still to be multiplied by
                    if constexpr (PREFETCH)
                    {
                        if (oo + o_step < oc) load_grad(o + o_step, next);  // the next channel's gradients arrive while this one computes
                    }
                    else if (a.grad_async != 0)
                    {
                        cp_async_wait_all();
                        slot = slots + (staged & 1) * (THREADS * PATCH_H * PATCH_W);
                        grad_scale = static_cast<float>(a.scale);
                        staged++;
                        if (oo + o_step < oc)
                        {
                            float* next_slot = slots + (staged & 1) * (THREADS * PATCH_H * PATCH_W);
    #pragma unroll
                            for (int rr = 0; rr < PATCH_H; rr++)
                                if (live[rr][0]) cp_async_16(next_slot + rr * PATCH_W, a.gy + at0[rr] + static_cast<int64_t>(o + o_step) * plane);
                        }
                    }
                    else
                    {
                        slot = slots;
    #pragma unroll
                        for (int rr = 0; rr < PATCH_H; rr++)
    #pragma unroll
                            for (int j = 0; j < PATCH_W; j++)
                                slot[rr * PATCH_W + j] = live[rr][j] ? static_cast<float>(__ldg(a.gy + at0[rr] + static_cast<int64_t>(o) * plane + j) * a.scale) : 0.0f;
                    }
                    auto grad_from_slot = [&]() {
                        if constexpr (!PREFETCH)
                        {
    #pragma unroll
                            for (int rr = 0; rr < PATCH_H; rr++)
    #pragma unroll
                                for (int j = 0; j < PATCH_W; j++) grad[rr][j] = slot[rr * PATCH_W + j] * grad_scale;
                        }
                    };
                    auto grad_to_slot = [&]() {
                        if constexpr (!PREFETCH)
                        {
    #pragma unroll
                            for (int rr = 0; rr < PATCH_H; rr++)
    #pragma unroll
                                for (int j = 0; j < PATCH_W; j++) slot[rr * PATCH_W + j] = grad[rr][j];
                            grad_scale = 1.0f;
                        }
                    };
                    const T s = spar[oo * 3], abs_alpha = spar[oo * 3 + 1], scale = spar[oo * 3 + 2];
                    const bool neg = s < T(0);
                    const T* win = sx + (neg ? welems : 0);
                    T* wbin = wbins + (warp * OC + oo) * taps;
                    T* abin = abins + warp * OC + oo;
                    if (winner_takes_all)
                    {
                        grad_from_slot();
                        // MAX / MIN: only the channels within 1e-6 of the merged value receive gradient, shared
                        // equally; the pair's own soft extremum is needed first.
                        // Same arithmetic as the forward kernel, so that the winning channel reproduces y exactly.
                        T out[PATCH_H][PATCH_W];
                        if constexpr (KW == 3)
                        {
    #pragma unroll
                            for (int rr = 0; rr < PATCH_H; rr++)
                            {
                                T d[9][PATCH_W], e[9][PATCH_W], ref[PATCH_W], inv_sum[PATCH_W], out_d[PATCH_W];
                                smorph3_values(win, sw + oo * taps, 1, s, g, tx, ty, rr, d);
                                smorph3_softmax(d, scale, ref, e, inv_sum, out_d);
    #pragma unroll
                                for (int j = 0; j < PATCH_W; j++) out[rr][j] = ref[j] + out_d[j];
                            }
                        }
                        else
                        {
                            T ref[PATCH_H][PATCH_W], inv_sum[PATCH_H][PATCH_W];
                            smorph_pair<0, KW>(win, sw + oo * taps, 1, s, scale, g, tx, ty, ref, inv_sum, out);
                        }
    #pragma unroll
                        for (int rr = 0; rr < PATCH_H; rr++)
    #pragma unroll
                            for (int j = 0; j < PATCH_W; j++)
                            {
                                if (!live[rr][j]) continue;
                                const int64_t at = at0[rr] + static_cast<int64_t>(o) * plane + j;
                                const T winners = __ldg(a.counts + at);
                                const T dist = s * out[rr][j] - __ldg(a.y + at);
                                grad[rr][j] = (dist < T(1e-6) && dist > -T(1e-6)) ? grad[rr][j] / (winners > T(0) ? winners : T(1)) : T(0);
                            }
                        grad_to_slot();
                    }
                    if constexpr (SOFT)
                    {
                        // Smooth merge: channel i receives g (p_i + beta p_i (c_i - final)), p_i = exp(beta (c_i - ref)) / sum_i q_i,
                        // and beta receives sum_i p_i (c_i - ref) (c_i - final) g (csrc/cpp/smorph_cpu_kernels.hxx:478, 520-552).
                        T out[PATCH_H][PATCH_W];
                        if constexpr (KW == 3)
                        {
    #pragma unroll
                            for (int rr = 0; rr < PATCH_H; rr++)
                            {
                                T d[9][PATCH_W], e[9][PATCH_W], ref[PATCH_W], inv_sum[PATCH_W], out_d[PATCH_W];
                                smorph3_values(win, sw + oo * taps, 1, s, g, tx, ty, rr, d);
                                smorph3_softmax(d, scale, ref, e, inv_sum, out_d);
    #pragma unroll
                                for (int j = 0; j < PATCH_W; j++) out[rr][j] = ref[j] + out_d[j];
                            }
                        }
                        else
                        {
                            T ref[PATCH_H][PATCH_W], inv_sum[PATCH_H][PATCH_W];
                            smorph_pair<0, KW>(win, sw + oo * taps, 1, s, scale, g, tx, ty, ref, inv_sum, out);
                        }
                        const T bt = __ldg(a.beta + o);
                        T beta_sum = T(0);
                        grad_from_slot();
    #pragma unroll
                        for (int rr = 0; rr < PATCH_H; rr++)
    #pragma unroll
                            for (int j = 0; j < PATCH_W; j++)
                            {
                                if (!live[rr][j]) continue;
                                const int64_t at = at0[rr] + static_cast<int64_t>(o) * plane + j;
                                const T c = s * out[rr][j], ref = __ldg(a.soft_ref + at), final = __ldg(a.y + at);
                                const T p = exp((c - ref) * bt) * __ldg(a.soft_inv + at);
                                beta_sum = fma(p * (c - ref) * (c - final), grad[rr][j], beta_sum);
                                grad[rr][j] = grad[rr][j] * fma(bt * p, c - final, p);
                            }
                        grad_to_slot();
                        beta_sum = warp_sum(beta_sum);
                        if (lane == 0) bbins[warp * OC + oo] = beta_sum;
                    }
                    if constexpr (backward_splits<T, KH, KW>())
                    {
                        float centre[PATCH_H][PATCH_W], scaled[PATCH_H][PATCH_W];
                        bool have_stats = false;
                        if constexpr (FACTOR)
                        {
                            if (factorise)
                            {
                                const float2 pr = spair[oo];   // (Mw, range of w)
                                if (x_hi >= x_lo && scale * ((x_hi - x_lo) + pr.y) <= FACTOR_RANGE_BACKWARD)
                                {
                                    if (!(held_s == s && held_scale == scale))
                                    {
                                        held_centre = s > 0.0f ? x_hi : -x_lo;
                                        factor_fill<FKW, true>(win + block_at, sea, s, scale, held_centre, lane, scale * (x_hi - x_lo) > FACTOR_PRECISE);
                                        held_s = s;
                                        held_scale = scale;
                                    }
                                    // The thread's own largest s x: centre of its linear sums, and with Mw the base of its soft extrema.
                                    const float local = local_hi >= local_lo ? (s > 0.0f ? local_hi : -local_lo) : held_centre;
                                    smorph_stats_factored<FKW>(sea, seb + oo * taps, lane, scale, local + pr.x, local - held_centre, held_centre, pr.x,
                                                               scale * (x_hi - x_lo) > FACTOR_PRECISE, grad, centre, scaled);
                                    have_stats = true;
                                }
                            }
                        }
                        if (!have_stats) smorph_stats_stable<FKW>(win, sw + oo * taps, s, scale, g, tx, ty, grad, centre, scaled);
                        smorph_taps_backward<FKW>(win, sw + oo * taps, wbin, abin, red, s, abs_alpha, scale, centre, scaled, tx, ty, lane, gxr);
                    }
                    else if constexpr (KH == 3 && KW == 3)
                    {
                        bool done = false;
                        if constexpr (BOUNDED)
                        {
                            if (bounded)
                            {
                                const float4* row = reinterpret_cast<const float4*>(sshift + oo * BOUNDED_ROW);
                                const float4 params = row[BOUNDED_PARAMS / 4];
                                if (bound_range <= params.w)
                                {
                                    smorph3_pair_backward_bounded(win, row, wbin, abin, red, params, s > 0.0f ? local_mid : -local_mid, slot, grad_scale,
                                                                  tx, ty, lane, gxr);
                                    done = true;
                                }
                            }
                        }
                        if (!done)
                        {
                            grad_from_slot();
                            smorph3_pair_backward(win, sw + oo * taps, wbin, abin, red, s, abs_alpha, scale, grad, g, tx, ty, lane, gxr);
                        }
                    }
                    else smorph_pair_backward<KH, KW>(win, sw + oo * taps, sg, wbin, abin, s, abs_alpha, scale, grad, g, tx, ty, lane, gxr);
                    if constexpr (PREFETCH)
                    {
    #pragma unroll
                        for (int rr = 0; rr < PATCH_H; rr++)
    #pragma unroll
                            for (int j = 0; j < PATCH_W; j++) grad[rr][j] = next[rr][j];
                    }
                }
            }
        }
        __syncthreads();
        for (int e = threadIdx.x; e < oc * taps; e += THREADS)
        {
            const int k = e % taps, oo = e / taps;
            T total = T(0);
#pragma unroll
            for (int wp = 0; wp < WARPS; wp++) total += wbins[(wp * OC + oo) * taps + k];
            if constexpr (FAST) total *= a.scale;
            if (total != T(0)) atomic_add(a.gw + (static_cast<int64_t>(oc0 + oo) * wci + wi) * taps + k, total);
        }
        for (int oo = threadIdx.x; oo < oc; oo += THREADS)
        {
            T total = T(0);
#pragma unroll
            for (int wp = 0; wp < WARPS; wp++) total += abins[wp * OC + oo];
            if constexpr (FAST) total *= a.scale;
            if (total != T(0)) atomic_add(a.galpha + (g.identity ? oc0 + oo : static_cast<int64_t>(oc0 + oo) * g.Ci + ci), total);
            if constexpr (SOFT)
            {
                T beta_total = T(0);
#pragma unroll
                for (int wp = 0; wp < WARPS; wp++) beta_total += bbins[wp * OC + oo];
                if (beta_total != T(0)) atomic_add(a.gbeta + oc0 + oo, beta_total);
            }
        }
    }

    if constexpr (KH > 0)
    {
        // One pass of shared atomics per CTA: the register windows of neighbouring threads overlap.
#pragma unroll
        for (int r = 0; r < GH; r++)
#pragma unroll
            for (int c = 0; c < GW; c++)
                if (window(r, c) != T(0))
                    atomic_add(sg + (ty * PATCH_H + r) * g.win_stride + tx * PATCH_W + g.seg_off + c, FAST ? window(r, c) * a.scale : window(r, c));
    }
    __syncthreads();

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

template <typename T, int KH, int KW>
int launch_smorph_backward(const mc_desc& d, const T* x, const T* w, const T* alpha, const T* y, const T* counts, const T* gy, T* gx, T* gw,
                           T* galpha, cudaStream_t stream, const T* beta = nullptr, const T* soft_ref = nullptr, const T* soft_inv = nullptr,
                           T* gbeta = nullptr)
{
    constexpr int WARPS = THREADS / 32;
    SmorphBackwardArgs<T> a;
    a.g = make_geometry(d, sizeof(T));
    a.g.replicate = false;  // out-of-image taps are excluded, never read
    a.x = x; a.w = w; a.alpha = alpha; a.y = y; a.counts = counts; a.gy = gy; a.gx = gx; a.gw = gw; a.galpha = galpha;
    a.merge = d.merge;
    a.beta = beta; a.soft_ref = soft_ref; a.soft_inv = soft_inv; a.gbeta = gbeta;
    a.scale = d.merge == MC_MERGE_AVERAGE ? T(1.0) / static_cast<T>(d.Ci) : T(1.0);
    const size_t taps = static_cast<size_t>(d.kH) * d.kW;
    // The factorised recomputation of S and N suits the merges without a winner test (see launch_smorph_forward).
    constexpr bool FACTOR = backward_factorises<T, KH, KW, false>();
    a.factorise = FACTOR && (d.merge == MC_MERGE_ADD || d.merge == MC_MERGE_AVERAGE || d.merge == MC_MERGE_IDENTITY);
    size_t fixed = (3 * static_cast<size_t>(a.g.window_elems()) + WARPS * RED_ROWS * RED_STRIDE) * sizeof(T);
    size_t per_o = (taps + 3 + WARPS * (taps + 2)) * sizeof(T);
    if (a.factorise)
    {
        fixed += 32 + WARPS * static_cast<size_t>(FactorLayout<FACTOR ? KW : 3>::BYTES);
        per_o += (taps + 1) * sizeof(float2);
    }
    a.bounded = backward_bounds<T, KH, KW, false>() && d.merge != MC_MERGE_SMOOTH;
    if (a.bounded)
    {
        fixed += 48;
        per_o += sizeof(float2) + BOUNDED_ROW * sizeof(float);
    }
    // Staging slots of grad_output for the 3 x 3 float kernel: two buffers of 32 bytes per thread, after everything else.
    constexpr size_t GRAD_SLOTS = 2 * THREADS * PATCH_H * PATCH_W * sizeof(float);
    const bool stage_grad = sizeof(T) == 4 && KH == 3 && KW == 3;
    a.grad_async = stage_grad && d.W % 4 == 0 && reinterpret_cast<uintptr_t>(gy) % 16 == 0;
    if (stage_grad) fixed += GRAD_SLOTS + 16;
    if (fixed + per_o > MAX_SHARED_BYTES)
    {
        set_last_error("structuring element %dx%d too large for shared memory", d.kH, d.kW);
        return MC_ERR_UNSUPPORTED;
    }
    // Chunk of output channels: as many as fit in about 100 KiB (two CTAs per SM).
    // (The 5 x 5 and 7 x 7 float kernels run one CTA per SM anyway: their chunk may take twice that.)
    const size_t budget = fixed + per_o > 100 * 1024 ? MAX_SHARED_BYTES : (a.factorise ? 200 * 1024 : 100 * 1024);
    int chunk = static_cast<int>((budget - fixed) / per_o);
    chunk = std::max(1, std::min(chunk, a.g.identity ? 1 : d.Co));
    a.o_chunk = chunk;
    const size_t smem = fixed + per_o * chunk;
    a.grad_stage = stage_grad ? static_cast<int>((smem - GRAD_SLOTS) / 16 * 16) : 0;
    const int64_t blocks = static_cast<int64_t>(a.g.tiles_x) * a.g.tiles_y * d.Ci * d.B;
    if (blocks > 0x7fffffffLL) { set_last_error("too many tiles for one launch"); return MC_ERR_UNSUPPORTED; }
    auto launch = [&](auto kernel) {
        if (!allow_shared(kernel, smem)) { set_last_error("cannot opt in to %zu bytes of shared memory", smem); return static_cast<int>(MC_ERR_UNSUPPORTED); }
        kernel<<<static_cast<unsigned>(blocks), THREADS, smem, stream>>>(a);
        return check_launch("smorph_backward_kernel");
    };
    if (d.merge == MC_MERGE_SMOOTH) return launch(smorph_backward_kernel<T, KH, KW, true>);
    if constexpr (sizeof(T) == 4 && KH == 3 && KW == 3)
        if (a.bounded && a.grad_async && d.merge != MC_MERGE_MAX && d.merge != MC_MERGE_MIN) return launch(smorph_backward_kernel<T, KH, KW, false, true>);
    return launch(smorph_backward_kernel<T, KH, KW, false>);
}

}  // namespace mc

#include "smorph_forward_lean.cuh"

// Backward of the ADD / AVERAGE / IDENTITY merges for float and square 3 x 3 / 5 x 5 structuring elements, with the
// input window of every thread held in REGISTERS for the whole life of the CTA. Included by morpho_backward.cuh.
//
// The reference recomputes the extremal tap of every (output channel, input channel, pixel) triple with a tracked
// comparison and scatters through shared and global atomics (morphocore/functional/csrc/cuda/morpho_op_kernels.cuh:479-602).
// This kernel keeps the arithmetic and changes everything around it:
//   - A CTA owns (batch element, input channel, 64 x 32 tile) and walks ALL output channels. Every thread copies the
//     (2 + K - 1) x (4 + K - 1) window elements its 4 x 2 pixel patch can reach into registers once; after that the
//     channel loop reads no input from shared memory and contains no CTA barrier (the structuring elements of all
//     output channels are staged up front), so the eight warps drift apart and hide each other's latencies.
//   - Winner of a pair: the K row extrema R_kh come from 3-input max / min instructions, m is their extremum, the
//     winning row is the FIRST row with R_kh == m (a descending chain of selects, which also carries that row's K
//     candidates along), and the winning column is the first candidate of that row equal to m. That is the first tap
//     in kh-major, kw order that attains the extremum, i.e. the tap the reference's strict comparison keeps
//     (csrc/cpp/morpho_op_cpu_kernels.hxx:212-252), NaN candidates never win, and when nothing beats the initial value
//     (every candidate is the initial infinity or NaN) the index is 0 as in the reference. No candidate is ever
//     re-read from shared memory with a data-dependent address.
//   - grad_input: every thread adds into a PRIVATE copy of its patch's footprint, laid out [entry][lane] per warp, so
//     the read-modify-write needs no atomic and never meets a bank conflict; the copies are summed once per CTA.
//   - grad_weight: lane-private, warp-private bins [kh][FC slots][lane]: the bin of tap (kh, kw) sits at slot
//     kh * FC + kw, the same linear form of (kh, kw) that addresses the footprint, so ONE byte offset, assembled by the
//     select chains from constants, serves both read-modify-writes. A lane only ever touches word `lane` of a slot
//     (bank = lane: no conflict, no atomic). After each output channel one lane per tap sums the 32 partial sums of
//     its slot with 128-bit loads that start at a lane-dependent rotation (the eight lanes of a quarter warp hit
//     eight different bank groups), clears them and adds the total to the CTA's table.
#pragma once

namespace mc
{

/// Plain (non-atomic) add to a 32-bit word of shared memory given by its byte address in the shared window.
__device__ __forceinline__ void shared_add(uint32_t address, float v)
{
    float old;
    asm volatile("ld.shared.f32 %0, [%1];" : "=f"(old) : "r"(address));
    old += v;
    asm volatile("st.shared.f32 [%0], %1;" ::"r"(address), "f"(old) : "memory");
}

template <int KW> struct RegsBackwardLayout
{
    static constexpr int WARPS = THREADS / 32, TAPS = KW * KW;
    static constexpr int FR = PATCH_H + KW - 1, FC = PATCH_W + KW - 1;   // footprint of a thread's patch
    static constexpr int WROW = (KW + 3) / 4 * 4;                        // staged kernel row, padded to 128-bit loads
    static constexpr int SLOTS = KW * FC;                                // bin slots of a warp: slot kh * FC + kw
    static constexpr int FOOT_ELEMS = WARPS * FR * FC * 32;
    static constexpr int BIN_ELEMS = WARPS * SLOTS * 32;
    /// Floats of shared memory for `channels` output channels (rounded up to whole 128-bit vectors).
    static size_t elems(const Geometry& g, int channels)
    {
        const size_t foot = std::max<size_t>(FOOT_ELEMS, g.window_elems());
        return foot + static_cast<size_t>(channels) * KW * WROW + BIN_ELEMS + static_cast<size_t>(channels) * TAPS + 4;
    }
};

template <bool IS_MIN, int KW>
__global__ void __launch_bounds__(THREADS, 2) morpho_backward_pairs_regs_kernel(const PairsBackwardArgs<float> a)
{
    using T = float;
    using L = RegsBackwardLayout<KW>;
    constexpr int TAPS = L::TAPS, FR = L::FR, FC = L::FC, WROW = L::WROW, SLOTS = L::SLOTS;
    constexpr int LEN = segment_len(KW, sizeof(T)), OFF = segment_offset(KW, sizeof(T)), STRIDE = window_stride(KW, sizeof(T));
    static_assert(OFF + FC <= LEN, "a thread's footprint row lies inside its row segment");
    extern __shared__ __align__(16) unsigned char smem_raw[];
    const Geometry& g = a.g;

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
    const int wci = g.identity ? 1 : g.Ci;
    const int wi = g.identity ? 0 : ci;
    const int o_begin = g.identity ? ci : 0;
    const int o_end = g.identity ? ci + 1 : g.Co;
    const int channels = o_end - o_begin;

    T* foot = reinterpret_cast<T*>(smem_raw);                                      // [WARPS][FR * FC][32]; first the staged window
    T* sw = foot + (L::FOOT_ELEMS > g.window_elems() ? L::FOOT_ELEMS : (g.window_elems() + 3) / 4 * 4);   // [channels][KW][WROW]
    T* bins = sw + channels * KW * WROW;                                           // [WARPS][SLOTS][32]
    T* totals = bins + L::BIN_ELEMS;                                               // [channels][TAPS]

    // Stage the window (border resolved) and the structuring elements of every output channel, negated for erosion.
    stage_window_async<STRIDE>(foot, a.x + (static_cast<int64_t>(b) * g.Ci + ci) * plane, g, tile_h0, tile_w0, a.fill, [](int c) { return c; });
    {
        const T* wb = a.w + static_cast<int64_t>(b) * g.weight_batch_stride;
        for (int e = threadIdx.x; e < channels * KW * WROW; e += THREADS)
        {
            const int kw = e % WROW, kh = (e / WROW) % KW, o = e / (WROW * KW);
            T v = T(0);
            if (kw < KW) v = __ldg(wb + (static_cast<int64_t>(o_begin + o) * wci + wi) * TAPS + kh * KW + kw);
            sw[e] = IS_MIN ? -v : v;
        }
    }
    for (int e = threadIdx.x; e < L::BIN_ELEMS; e += THREADS) bins[e] = T(0);
    for (int e = threadIdx.x; e < channels * TAPS; e += THREADS) totals[e] = T(0);
    cp_async_wait_all();
    __syncthreads();

    // The thread's window: X[r][c] is window row 2 ty + r, column 4 tx + OFF + c, so that tap (kh, kw) of patch pixel
    // (rr, j) reads X[rr + KW-1-kh][j + KW-1-kw].
    T X[FR][FC];
#pragma unroll
    for (int r = 0; r < FR; r++)
    {
        T seg[LEN];
        load_segment<LEN>(seg, foot + (ty * PATCH_H + r) * STRIDE + tx * PATCH_W);
#pragma unroll
        for (int c = 0; c < FC; c++) X[r][c] = seg[OFF + c];
    }
    __syncthreads();
    for (int e = threadIdx.x; e < L::FOOT_ELEMS; e += THREADS) foot[e] = T(0);
    __syncthreads();

    T* warp_bins = bins + warp * (SLOTS * 32);
    // Byte addresses (shared window) of the lane's word in footprint entry 0 and in bin slot 0.
    const uint32_t foot_base = smem_addr(foot + warp * (FR * FC * 32) + lane);
    const uint32_t bins_base = smem_addr(warp_bins + lane);

    if (warp_live)
    {
        const int h0 = tile_h0 + ty * PATCH_H, w0 = tile_w0 + tx * PATCH_W;
        const bool vec = (g.W % 4 == 0) && (reinterpret_cast<uintptr_t>(a.gy) % 16 == 0) && w0 + PATCH_W <= g.W;
        const T* gy0 = a.gy + ((static_cast<int64_t>(b) * g.Co + o_begin) * g.H + h0) * g.W + w0;
        bool row_ok[PATCH_H];
#pragma unroll
        for (int rr = 0; rr < PATCH_H; rr++) row_ok[rr] = h0 + rr < g.H && w0 < g.W;
        auto load_grad = [&](T (&dst)[PATCH_H][PATCH_W], int o) {
#pragma unroll
            for (int rr = 0; rr < PATCH_H; rr++)
            {
                const T* row = gy0 + static_cast<int64_t>(o) * plane + static_cast<int64_t>(rr) * g.W;
                if (vec)
                {
                    float4 q = make_float4(0.f, 0.f, 0.f, 0.f);
                    if (row_ok[rr]) q = __ldg(reinterpret_cast<const float4*>(row));
                    dst[rr][0] = q.x; dst[rr][1] = q.y; dst[rr][2] = q.z; dst[rr][3] = q.w;
                }
                else
                {
#pragma unroll
                    for (int j = 0; j < PATCH_W; j++) dst[rr][j] = (row_ok[rr] && w0 + j < g.W) ? __ldg(row + j) : T(0);
                }
            }
        };

        T next[PATCH_H][PATCH_W];
        load_grad(next, 0);
        for (int o = 0; o < channels; o++)
        {
            T grad[PATCH_H][PATCH_W];
            bool any = false;
#pragma unroll
            for (int rr = 0; rr < PATCH_H; rr++)
#pragma unroll
                for (int j = 0; j < PATCH_W; j++)
                {
                    grad[rr][j] = next[rr][j] * a.scale;
                    any |= grad[rr][j] != T(0);
                }
            if (o + 1 < channels) load_grad(next, o + 1);   // in flight while this channel computes
            if (!__any_sync(0xffffffffu, any)) continue;

            T W[KW][WROW];
#pragma unroll
            for (int kh = 0; kh < KW; kh++) load_weights<WROW>(W[kh], sw + (o * KW + kh) * WROW);

#pragma unroll
            for (int rr = 0; rr < PATCH_H; rr++)
#pragma unroll
                for (int j = 0; j < PATCH_W; j++)
                {
                    T v[KW][KW], R[KW];
#pragma unroll
                    for (int kh = 0; kh < KW; kh++)
                    {
#pragma unroll
                        for (int kw = 0; kw < KW; kw++) v[kh][kw] = X[rr + KW - 1 - kh][j + KW - 1 - kw] + W[kh][kw];
                        T r = v[kh][0];
#pragma unroll
                        for (int kw = 1; kw + 1 < KW; kw += 2) r = ext3<IS_MIN>(r, v[kh][kw], v[kh][kw + 1]);
                        if constexpr (KW % 2 == 0) r = ext2<IS_MIN>(r, v[kh][KW - 1]);
                        R[kh] = r;
                    }
                    T m = R[0];
#pragma unroll
                    for (int kh = 1; kh + 1 < KW; kh += 2) m = ext3<IS_MIN>(m, R[kh], R[kh + 1]);
                    if constexpr (KW % 2 == 0) m = ext2<IS_MIN>(m, R[KW - 1]);

                    // First row that attains m, with its candidates; then the first of those equal to m. The chains
                    // select byte offsets: (kh * FC + kw) * 128 addresses both the footprint entry and the bin slot.
                    uint32_t off_row = (KW - 1) * FC * 128u;
                    T s[KW];
#pragma unroll
                    for (int kw = 0; kw < KW; kw++) s[kw] = v[KW - 1][kw];
#pragma unroll
                    for (int i = KW - 2; i >= 0; i--)
                    {
                        const bool q = R[i] == m;
                        off_row = q ? i * FC * 128u : off_row;
#pragma unroll
                        for (int kw = 0; kw < KW; kw++) s[kw] = q ? v[i][kw] : s[kw];
                    }
                    uint32_t off_col = (KW - 1) * 128u;
#pragma unroll
                    for (int t = KW - 2; t >= 0; t--) off_col = s[t] == m ? t * 128u : off_col;
                    // Nothing beat the initial value (all candidates are the initial infinity or NaN): index 0.
                    const bool beaten = IS_MIN ? m < Limits<T>::inf() : m > -Limits<T>::inf();
                    const uint32_t off = beaten ? off_row + off_col : 0u;

                    const T gv = grad[rr][j];
                    const uint32_t E0 = ((rr + KW - 1) * FC + (j + KW - 1)) * 128u;
                    shared_add(foot_base + E0 - off, gv);
                    shared_add(bins_base + off, gv);
                }

            // Column sums of the warp's bins: lane k takes tap k. Its eight 128-bit loads start at a rotation of
            // k vectors, so the eight lanes that one shared-memory wavefront serves read eight different bank groups.
            __syncwarp();
            for (int k = lane; k < TAPS; k += 32)
            {
                float4* slot = reinterpret_cast<float4*>(warp_bins + ((k / KW) * FC + k % KW) * 32);
                T sum = T(0);
#pragma unroll
                for (int c = 0; c < 8; c++)
                {
                    const int at = (c + k) & 7;
                    const float4 q = slot[at];
                    slot[at] = make_float4(0.f, 0.f, 0.f, 0.f);
                    sum += (q.x + q.y) + (q.z + q.w);
                }
                if (sum != T(0)) atomic_add(totals + o * TAPS + k, sum);
            }
            __syncwarp();
        }
    }
    __syncthreads();

    for (int e = threadIdx.x; e < channels * TAPS; e += THREADS)
    {
        const T sum = totals[e];
        const int o = o_begin + e / TAPS, k = e % TAPS;
        if (sum != T(0)) atomic_add(a.gw + (static_cast<int64_t>(o) * wci + wi) * TAPS + k, a.sign * sum);
    }

    // Sum the private footprints: window position (t, u), t = 2 ty + r, u = 4 tx + c, is image pixel
    // (tile_h0 - halo_top + t, tile_w0 - halo_left_of(KW) + u) and is covered by up to FR / 2 x FC / 4 threads.
    T* gxp = a.gx + (static_cast<int64_t>(b) * g.Ci + ci) * plane;
    constexpr int SPAN_H = TILE_H + KW - 1, SPAN_W = TILE_W + KW - 1;
    const int row0 = tile_h0 - g.halo_top(), col0 = tile_w0 - halo_left_of(KW);
    for (int e = threadIdx.x; e < SPAN_H * SPAN_W; e += THREADS)
    {
        const int t = e / SPAN_W, u = e - t * SPAN_W;
        const int iy = row0 + t, ix = col0 + u;
        if (iy < 0 || iy >= g.H || ix < 0 || ix >= g.W) continue;
        const int ty_lo = max(0, (t - FR + 2) >> 1), ty_hi = min(TILE_H / PATCH_H - 1, t >> 1);
        const int tx_lo = max(0, (u - FC + 4) >> 2), tx_hi = min(TILE_W / PATCH_W - 1, u >> 2);
        T sum = T(0);
        for (int py = ty_lo; py <= ty_hi; py++)
            for (int px = tx_lo; px <= tx_hi; px++)
            {
                const int w_id = (px >> 3) + 2 * (py >> 2), l_id = (px & 7) + 8 * (py & 3);
                sum += foot[(w_id * (FR * FC) + (t - PATCH_H * py) * FC + (u - PATCH_W * px)) * 32 + l_id];
            }
        if (sum != T(0)) atomic_add(gxp + static_cast<int64_t>(iy) * g.W + ix, sum);
    }
}

/// Shared memory of the kernel above, or 0 when the channel count makes it too large for two CTAs per SM.
template <int KW>
inline size_t pairs_regs_smem(const Geometry& g, int channels)
{
    const size_t bytes = RegsBackwardLayout<KW>::elems(g, channels) * sizeof(float);
    return bytes <= 110 * 1024 ? bytes : 0;
}

}  // namespace mc

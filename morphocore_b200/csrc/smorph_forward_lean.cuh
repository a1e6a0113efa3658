// Smorph forward for the case that dominates training: float, square 3 x 3 structuring element, SUM / MEAN merge,
// one alpha per (output, input) channel pair. Included by smorph.cuh.
//
// Same mathematics as the factorised path of smorph_forward_kernel (which replaces the reference's
// smorph_forward_kernel, morphocore/functional/csrc/cuda/smorph_kernels.cuh:307-407): with u_k = s (x_q + w_k),
//     exp(|a| (u_k - Mx - Mw)) = E_q Ew_k,   E_q = 2^(scale (s x_q - Mx)),   Ew_k = 2^(scale (s w_k - Mw)),
//     S = sum_k E_q Ew_k,   N = sum_k (A_q Ew_k + E_q Bw_k),   A_q = E_q (s x_q - Mx),   Bw_k = Ew_k (s w_k - Mw),
//     out = s (Mx + Mw + N / S),
// three fused multiply-adds per tap once the per-pixel factors (E, A) of the pair are tabulated. When every pair has
// its own alpha (any training run after its first optimiser step) that table must be rebuilt for EVERY pair, and the
// rebuild decides the speed. This kernel is built around a cheap rebuild:
//   - per input channel every lane loads its share of the warp's block of the window (32 x 8 pixels plus halo: 360
//     elements = 180 pairs, six pairs per lane, consecutive lanes taking consecutive pairs) into registers ONCE, and
//     the block's range of x comes from two warp-reduce instructions;
//   - per pair the rebuild is register arithmetic only: one fused multiply-add, one multiply, one ex2 and one
//     multiply per element, then one 128-bit store (E, A, E, A) per pair of elements. Nothing is re-read, no loop
//     has a run-time trip count;
//   - the table has ONE copy of every element: its 16-byte chunks are swizzled (chunk q of a row sits at
//     q ^ ((q >> 3) & 1)), which makes the tap loop's 128-bit loads (thread column t reads chunks 2 t ..: lanes 32
//     bytes apart) and the rebuild's stores conflict free without the duplicated columns of FactorLayout;
//   - taps outside the image are excluded by value: a lane overwrites its out-of-image elements with -s * 1e30 when it
//     loads them (E = A = 0 follow from the arithmetic; the sentinels are flipped if a later pair of the channel has
//     the other sign), so the staged window is the raw TMA copy: no border patching pass and no second copy of the
//     window for pairs of the other sign.
// A pair whose exponent range |alpha| log2(e) (range of x in the block + range of w) exceeds LEAN_RANGE binades takes the
// max-subtracting evaluation instead (warp-uniform branch: large |alpha|, or inputs spread widely inside one block).
#pragma once

namespace mc
{

struct LeanForwardArgs
{
    Geometry g;
    const float* x;
    const float* w;
    const float* alpha;
    float* y;
    int merge;
    int o_groups;
    int chunk;               // input channels staged per barrier
    unsigned int* errors;    // counter of timed-out waits
    uint64_t wait_limit_ns;  // bound of one wait on a TMA copy
};

constexpr int LEAN_OB = 4;   // output channels of a CTA: they share the registers that hold the block of x
// Largest exponent range, in binades, that a pair may span and still be factorised here: every product E_q Ew_k is then at
// least 2^-112, fourteen binades above the smallest normal float (the exponentials flush denormal results to zero), and
// the reciprocal of the smallest possible S, 2^112, is far from overflow. Activations of a deep stack (values of a few
// hundred, spread over tens of units inside one 32 x 8 block) reach 100 binades at |alpha| = 2.
constexpr float LEAN_RANGE = 112.0f;

/// Soft extrema (u domain) of the four pixels of patch row rr for one 3 x 3 pair, by the max-subtracting evaluation with
/// the nine candidates of each pixel in registers (smorph3_values, smorph3_softmax: one ex2 per tap). `win` is the raw
/// window (zeros outside the image): with `masked`, candidates whose tap lies outside the image are excluded here.
/// Not inlined on purpose: the factorised path around its call site keeps its registers.
static __device__ __noinline__ float4 lean_stable_row(const float* __restrict__ win, const float* __restrict__ swk, float s, float scale, int H, int W, int h,
                                               int w0, int tx, int ty, int rr, bool masked)
{
    constexpr int LEN = segment_len(3, 4), OFF = segment_offset(3, 4), STRIDE = window_stride(3, 4);
    float d[9][PATCH_W], e[9][PATCH_W], ref[PATCH_W], inv_sum[PATCH_W], out_d[PATCH_W];
#pragma unroll
    for (int kh = 0; kh < 3; kh++)
    {
        float seg[LEN];
        load_segment<LEN>(seg, win + (ty * PATCH_H + rr + 2 - kh) * STRIDE + tx * PATCH_W);
#pragma unroll
        for (int kw = 0; kw < 3; kw++)
        {
            const float wv = swk[(kh * 3 + kw) * LEAN_OB];
#pragma unroll
            for (int j = 0; j < PATCH_W; j++)
            {
                const int iy = h + 1 - kh, ix = w0 + j + 1 - kw;
                const bool out = masked && (iy < 0 || iy >= H || ix < 0 || ix >= W);
                d[kh * 3 + kw][j] = out ? -Limits<float>::big() : fmaf(s, seg[OFF + j + 2 - kw], wv);
            }
        }
    }
    smorph3_softmax(d, scale, ref, e, inv_sum, out_d);
    return make_float4(ref[0] + out_d[0], ref[1] + out_d[1], ref[2] + out_d[2], ref[3] + out_d[3]);
}

/// The warp's (E, A) table: ROWS rows of CHUNKS 16-byte chunks (E, A, E, A) of two pixels, chunk q stored at swz(q).
template <int KW> struct LeanTable
{
    using F = FactorLayout<KW>;
    static constexpr int ROWS = F::ROWS, CHUNKS = F::WS / 2, PAIRS = ROWS * CHUNKS;
    static constexpr int SWEEPS = (PAIRS + 31) / 32;
    static constexpr int BYTES = ROWS * CHUNKS * 16;
    __host__ __device__ static constexpr int swz(int q) { return q ^ ((q >> 3) & 1); }
};

/// factor_pair on the swizzled table. `rows` is the table row of the thread's first patch row, `at[v]` the stored
/// position of chunk 2 t + v of a row for the thread's column t.
template <int KW>
__device__ __forceinline__ void lean_factor_pair(const float4* __restrict__ rows, const int (&at)[FactorLayout<KW>::LEN / 2], const float2* __restrict__ eb,
                                                 int wstride, float2 (&acc)[PATCH_H][PATCH_W], float (&rest)[PATCH_H][PATCH_W])
{
    using L = FactorLayout<KW>;
    using Tb = LeanTable<KW>;
    static_assert(PATCH_H == 2, "the row schedule below is written for two patch rows");
    // Table row r (relative to the thread's first patch row) is read by patch row rr through kernel row kh = rr + KW - 1 - r:
    // both patch rows meet kernel row KW - 1 first, whose first tap initialises the sums (no zeroing pass).
    auto row = [&](int r, bool first, bool second) {
        float2 seg[L::LEN];
        const float4* src = rows + r * Tb::CHUNKS;
#pragma unroll
        for (int v = 0; v < L::LEN / 2; v++)
        {
            const float4 t = src[at[v]];
            seg[2 * v] = make_float2(t.x, t.y);
            seg[2 * v + 1] = make_float2(t.z, t.w);
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
                    if (kh == KW - 1 && kw == 0)
                    {
                        acc[rr][j] = __fmul2_rn(q, ew2);
                        rest[rr][j] = q.x * t.y;
                    }
                    else
                    {
                        acc[rr][j] = __ffma2_rn(q, ew2, acc[rr][j]);
                        rest[rr][j] = fmaf(q.x, t.y, rest[rr][j]);
                    }
                }
            }
        };
        if (first) apply(0, KW - 1 - r);
        if (second) apply(1, KW - r);
    };
    row(0, true, false);
#pragma unroll
    for (int r = 1; r < KW; r++) row(r, true, true);
    row(KW, false, true);
}

/// Bytes of shared memory per staged channel besides its two window buffers, and the fixed part.
template <int KW> constexpr size_t lean_channel_bytes() { return static_cast<size_t>(KW * KW) * LEAN_OB * (sizeof(float2) + sizeof(float)) + LEAN_OB * sizeof(float4); }
template <int KW> constexpr size_t lean_fixed_bytes() { return 128 + 2 * 128 + 16 + (THREADS / 32) * static_cast<size_t>(LeanTable<KW>::BYTES); }

template <int KW>
__global__ void __launch_bounds__(THREADS, 2) smorph_forward_lean_kernel(const LeanForwardArgs a, const __grid_constant__ CUtensorMap tmap)
{
    using L = FactorLayout<KW>;
    constexpr int OB = LEAN_OB, TAPS = KW * KW, STRIDE = L::STRIDE;
    constexpr int WELEMS = (TILE_H + KW - 1) * STRIDE;
    using Tb = LeanTable<KW>;
    constexpr int SWEEPS = Tb::SWEEPS;          // pairs lane, lane + 32, ... of the block's PAIRS pairs
    extern __shared__ __align__(128) unsigned char smem_raw[];
    const Geometry& g = a.g;

    uint64_t* full = reinterpret_cast<uint64_t*>(smem_raw);
    const int stage_elems = (a.chunk * WELEMS * 4 + 127) / 128 * 128 / 4;
    float* sx0 = reinterpret_cast<float*>(smem_raw + 128);                      // two stages of `chunk` raw windows
    float4* spar = reinterpret_cast<float4*>(sx0 + 2 * stage_elems);            // [chunk][OB]: sign, exp scale, Mw, range of s w
    float2* seb = reinterpret_cast<float2*>(spar + a.chunk * OB);               // [chunk][TAPS][OB]: (Ew, Bw)
    float* sw = reinterpret_cast<float*>(seb + a.chunk * TAPS * OB);            // [chunk][TAPS][OB]: s w (max-subtracting evaluation)
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    float4* sea = reinterpret_cast<float4*>(smem_raw + (reinterpret_cast<unsigned char*>(sw + a.chunk * TAPS * OB) - smem_raw + 15) / 16 * 16)
                  + warp * (Tb::BYTES / 16);                                    // this warp's (E, A) table

    const int tiles = g.tiles_x * g.tiles_y;
    const int og = blockIdx.x % a.o_groups;
    const int tile = (blockIdx.x / a.o_groups) % tiles;
    const int b = blockIdx.x / (a.o_groups * tiles);
    const int tile_h0 = (tile / g.tiles_x) * TILE_H, tile_w0 = (tile % g.tiles_x) * TILE_W;
    int tx, ty, half;
    bool warp_live, split;
    thread_patch_split(tile_h0, tile_w0, g.H, g.W, true, tx, ty, warp_live, split, half);
    // When the right half of the tile is outside the image the two warps of a warp row share the left block and each
    // takes half of the output channels.
    const int o_count = split ? OB / 2 : OB, o_base = half * (OB / 2);
    const int wx = split ? 0 : (warp & 1);
    const int o0 = og * OB;

    if (threadIdx.x == 0)
    {
        mbar_init(full, 1);
        mbar_init(full + 1, 1);
        mbar_fence_init();
    }
    __syncthreads();
    const uint32_t stage_bytes = static_cast<uint32_t>(a.chunk) * WELEMS * 4;
    auto issue = [&](int n) {
        uint64_t* bar = full + (n & 1);
        mbar_expect_tx(bar, stage_bytes);
        tma_load_4d(sx0 + (n & 1) * stage_elems, &tmap, bar, tile_w0 - g.halo_left(), tile_h0 - g.halo_top(), n * a.chunk, b);
    };
    if (threadIdx.x == 0) issue(0);

    // The lane's share of the warp's block: pairs u = lane + 32 i of the block's PAIRS pairs of elements (row u / CHUNKS,
    // chunk u % CHUNKS), where each comes from in a window, where it goes in the table, and which of its two elements
    // lie inside the image.
    const int block_row0 = 8 * (warp >> 1), block_col0 = 32 * wx;
    int src_at[SWEEPS], dst_at[SWEEPS];
    unsigned int inside_mask = 0;
#pragma unroll
    for (int i = 0; i < SWEEPS; i++)
    {
        const int u = min(lane + 32 * i, Tb::PAIRS - 1), r = u / Tb::CHUNKS, q = u - r * Tb::CHUNKS;
        src_at[i] = (block_row0 + r) * STRIDE + block_col0 + 2 * q;
        dst_at[i] = r * Tb::CHUNKS + Tb::swz(q);
        const int iy = tile_h0 - g.halo_top() + block_row0 + r, ix = tile_w0 - g.halo_left() + block_col0 + 2 * q;
#pragma unroll
        for (int e = 0; e < 2; e++)
            if (lane + 32 * i < Tb::PAIRS && iy >= 0 && iy < g.H && ix + e >= 0 && ix + e < g.W) inside_mask |= 1u << (2 * i + e);
    }
    const bool last_sweep = lane + 32 * (SWEEPS - 1) < Tb::PAIRS;   // the last sweep is partial
    // Does the warp's block of the window lie inside the image (no candidate to exclude)?
    const bool block_inside = tile_h0 - g.halo_top() + block_row0 >= 0 && tile_h0 - g.halo_top() + block_row0 + Tb::ROWS <= g.H
                              && tile_w0 - g.halo_left() + block_col0 >= 0 && tile_w0 - g.halo_left() + block_col0 + L::WS <= g.W;
    // Table positions of the chunks 2 t .. of a row that thread column t reads (lean_factor_pair).
    int read_at[L::LEN / 2];
#pragma unroll
    for (int v = 0; v < L::LEN / 2; v++) read_at[v] = Tb::swz(2 * (lane & 7) + v);
    const float4* table_rows = sea + ((lane >> 3) * PATCH_H) * Tb::CHUNKS;

    float merged[OB][PATCH_H][PATCH_W], offset[OB];
#pragma unroll
    for (int o = 0; o < OB; o++)
    {
        offset[o] = 0.0f;
#pragma unroll
        for (int rr = 0; rr < PATCH_H; rr++)
#pragma unroll
            for (int j = 0; j < PATCH_W; j++) merged[o][rr][j] = 0.0f;
    }

    int n = 0;
    for (int c0 = 0; c0 < g.Ci; c0 += a.chunk, n++)
    {
        const int cc = min(a.chunk, g.Ci - c0);
        const float* stage = sx0 + (n & 1) * stage_elems;
        __syncthreads();   // every warp is done with the other stage's windows and with the tables below
        if (threadIdx.x == 0 && c0 + a.chunk < g.Ci)
        {
            fence_async_smem();
            issue(n + 1);
        }
        // Tables of the stage's pairs, one warp per pair and one lane per tap: sign, scale, Mw = max_k s w_k and the
        // range of s w by shuffles, then (Ew, Bw).
        for (int e = warp; e < cc * OB; e += THREADS / 32)
        {
            const int o = e % OB, c = e / OB;
            if (o0 + o >= g.Co)
            {
                if (lane == 0) spar[e] = make_float4(1.0f, 1.0f, 0.0f, 0.0f);   // never evaluated
                continue;
            }
            const float al = __ldg(a.alpha + static_cast<int64_t>(o0 + o) * g.Ci + c0 + c);
            const float sgn = al >= 0.0f ? 1.0f : -1.0f, scale = exp_scale(fabsf(al));
            const float* wp = a.w + (static_cast<int64_t>(o0 + o) * g.Ci + c0 + c) * TAPS;
            float lo = Limits<float>::inf(), hi = -Limits<float>::inf();
            for (int k = lane; k < TAPS; k += 32)
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
            if (lane == 0) spar[e] = make_float4(sgn, scale, hi, hi - lo);
            for (int k = lane; k < TAPS; k += 32)
            {
                const float v = sgn * __ldg(wp + k), d = v - hi;
                const float ew = exp2_product(d, scale);
                seb[(c * TAPS + k) * OB + o] = make_float2(ew, ew * d);
                sw[(c * TAPS + k) * OB + o] = v;
            }
        }
        if (!mbar_wait(full + (n & 1), (n >> 1) & 1, a.wait_limit_ns))
        {
            if (threadIdx.x == 0 && a.errors != nullptr) atomicAdd(a.errors, 1u);
            return;  // every thread of the CTA waits on the same barrier and gives up together
        }
        __syncthreads();
        if (!warp_live) continue;

        for (int c = 0; c < cc; c++)
        {
            const float* win = stage + c * WELEMS;
            // The lane's elements of the block and the block's range of in-image x. Out-of-image elements then hold
            // -x_sign * 1e30, so that s x - centre is -1e30 for a pair of sign s = x_sign: E = 2^(-huge) = 0 and A = 0.
            float X[SWEEPS][2];
            float x_lo = Limits<float>::inf(), x_hi = -Limits<float>::inf();
            float x_sign = spar[c * OB + o_base].x;
#pragma unroll
            for (int i = 0; i < SWEEPS; i++)
            {
                const float2 v = *reinterpret_cast<const float2*>(win + src_at[i]);
                X[i][0] = v.x; X[i][1] = v.y;
            }
            if (block_inside)
            {
                // Nothing to exclude (the clamped extra pair of a lane past the end of the block repeats the last one).
#pragma unroll
                for (int i = 0; i < SWEEPS; i++)
                {
                    x_lo = fminf(x_lo, fminf(X[i][0], X[i][1]));
                    x_hi = fmaxf(x_hi, fmaxf(X[i][0], X[i][1]));
                }
            }
            else
            {
#pragma unroll
                for (int i = 0; i < SWEEPS; i++)
#pragma unroll
                    for (int e = 0; e < 2; e++)
                    {
                        const bool in = (inside_mask >> (2 * i + e)) & 1u;
                        x_lo = fminf(x_lo, in ? X[i][e] : Limits<float>::inf());
                        x_hi = fmaxf(x_hi, in ? X[i][e] : -Limits<float>::inf());
                        X[i][e] = in ? X[i][e] : -x_sign * Limits<float>::big();
                    }
            }
            x_lo = from_ordered(__reduce_min_sync(0xffffffffu, to_ordered(x_lo)));
            x_hi = from_ordered(__reduce_max_sync(0xffffffffu, to_ordered(x_hi)));
            float held_s = 0.0f, held_scale = -1.0f;

#pragma unroll
            for (int o = 0; o < OB; o++)
            {
                if (o >= o_count) break;
                const int os = o_base + o;
                if (o0 + os >= g.Co) break;
                const float4 par = spar[c * OB + os];   // sign, scale, Mw, range of s w
                const float s = par.x, scale = par.y;
                if (x_hi >= x_lo && scale * ((x_hi - x_lo) + par.w) <= LEAN_RANGE)
                {
                    const float centre = s > 0.0f ? x_hi : -x_lo;
                    if (!(held_s == s && held_scale == scale))
                    {
                        if (s != x_sign)
                        {
                            // A pair of the other sign: flip the sentinels of the out-of-image elements.
#pragma unroll
                            for (int i = 0; i < SWEEPS; i++)
#pragma unroll
                                for (int e = 0; e < 2; e++)
                                    if (!((inside_mask >> (2 * i + e)) & 1u)) X[i][e] = -s * Limits<float>::big();
                            x_sign = s;
                        }
                        __syncwarp();   // every lane is done reading the previous table
#pragma unroll
                        for (int i = 0; i < SWEEPS; i++)
                        {
                            const float xp0 = fmaf(s, X[i][0], -centre), xp1 = fmaf(s, X[i][1], -centre);
                            const float e0 = ex2_approx(xp0 * scale), e1 = ex2_approx(xp1 * scale);
                            const float4 chunk = make_float4(e0, e0 * xp0, e1, e1 * xp1);
                            if (i + 1 < SWEEPS || last_sweep) sea[dst_at[i]] = chunk;
                        }
                        __syncwarp();
                        held_s = s;
                        held_scale = scale;
                    }
                    float2 acc[PATCH_H][PATCH_W];
                    float rest[PATCH_H][PATCH_W];
                    lean_factor_pair<KW>(table_rows, read_at, seb + c * TAPS * OB + os, OB, acc, rest);
                    // out = s (Mx + Mw + N / S): the constant part is summed per output channel and joins at the end.
                    offset[o] += s * (centre + par.z);
#pragma unroll
                    for (int rr = 0; rr < PATCH_H; rr++)
#pragma unroll
                        for (int j = 0; j < PATCH_W; j++)
                            merged[o][rr][j] = fmaf((acc[rr][j].y + rest[rr][j]) * soft_rcp(acc[rr][j].x), s, merged[o][rr][j]);
                }
                else
                {
                    // Max-subtracting evaluation (lean_stable_row), kept out of line: its 72 registers of candidates and
                    // exponentials must not weigh on the factorised path.
                    const float* swk = sw + c * TAPS * OB + os;
#pragma unroll
                    for (int rr = 0; rr < PATCH_H; rr++)
                    {
                        const float4 out = lean_stable_row(win, swk, s, scale, g.H, g.W, tile_h0 + ty * PATCH_H + rr, tile_w0 + tx * PATCH_W, tx, ty, rr,
                                                           !block_inside);
                        merged[o][rr][0] = fmaf(s, out.x, merged[o][rr][0]);
                        merged[o][rr][1] = fmaf(s, out.y, merged[o][rr][1]);
                        merged[o][rr][2] = fmaf(s, out.z, merged[o][rr][2]);
                        merged[o][rr][3] = fmaf(s, out.w, merged[o][rr][3]);
                    }
                }
            }
        }
    }

    if (!warp_live) return;
    const float divisor = static_cast<float>(g.Ci);
    const bool vec_store = (g.W % 4 == 0) && (reinterpret_cast<uintptr_t>(a.y) % 16 == 0);
#pragma unroll
    for (int o = 0; o < OB; o++)
    {
        if (o >= o_count || o0 + o_base + o >= g.Co) break;
#pragma unroll
        for (int rr = 0; rr < PATCH_H; rr++)
        {
            const int h = tile_h0 + ty * PATCH_H + rr, w0 = tile_w0 + tx * PATCH_W;
            if (h >= g.H || w0 >= g.W) continue;
            float out[PATCH_W];
#pragma unroll
            for (int j = 0; j < PATCH_W; j++)
            {
                const float v = merged[o][rr][j] + offset[o];
                out[j] = a.merge == MC_MERGE_AVERAGE ? v / divisor : v;
            }
            float* dst = a.y + ((static_cast<int64_t>(b) * g.Co + o0 + o_base + o) * g.H + h) * g.W + w0;
            if (vec_store && w0 + PATCH_W <= g.W) *reinterpret_cast<float4*>(dst) = make_float4(out[0], out[1], out[2], out[3]);
            else
            {
#pragma unroll
                for (int j = 0; j < PATCH_W; j++)
                    if (w0 + j < g.W) dst[j] = out[j];
            }
        }
    }
}

/// Launches the kernel above when the tensor can be staged by TMA; returns MC_ERR_UNSUPPORTED (and launches nothing) when
/// it cannot, so that the caller falls back to the general kernel.
template <int KW>
int launch_smorph_forward_lean(const mc_desc& d, const float* x, const float* w, const float* alpha, float* y, cudaStream_t stream)
{
    LeanForwardArgs a;
    a.g = make_geometry(d, sizeof(float));
    a.g.replicate = false;
    a.x = x; a.w = w; a.alpha = alpha; a.y = y; a.merge = d.merge;
    a.o_groups = (d.Co + LEAN_OB - 1) / LEAN_OB;
    a.errors = device_error_counter();
    a.wait_limit_ns = wait_limit_ns();
    const int64_t blocks = static_cast<int64_t>(a.g.tiles_x) * a.g.tiles_y * a.o_groups * d.B;
    if (blocks > 0x7fffffffLL) return MC_ERR_UNSUPPORTED;
    const size_t window = static_cast<size_t>(a.g.window_elems()) * sizeof(float);
    const size_t per_channel = 2 * ((window + 127) / 128 * 128) + lean_channel_bytes<KW>(), fixed = lean_fixed_bytes<KW>();
    int chunk = static_cast<int>((100 * 1024 - fixed) / per_channel);
    chunk = std::max(1, std::min(std::min(chunk, 8), d.Ci));
    const size_t smem = fixed + per_channel * chunk + 256;
    CUtensorMap tmap{};
    if (!make_window_tensor_map(&tmap, x, sizeof(float), d.B, d.Ci, d.H, d.W, a.g.win_stride, a.g.win_rows, chunk)) return MC_ERR_UNSUPPORTED;
    a.chunk = chunk;
    auto kernel = smorph_forward_lean_kernel<KW>;
    if (!allow_shared(kernel, smem)) return MC_ERR_UNSUPPORTED;
    kernel<<<static_cast<unsigned>(blocks), THREADS, smem, stream>>>(a, tmap);
    return check_launch("smorph_forward_lean_kernel");
}

/// Double precision has no such kernel: the caller takes the general one.
template <int KW>
int launch_smorph_forward_lean(const mc_desc&, const double*, const double*, const double*, double*, cudaStream_t) { return MC_ERR_UNSUPPORTED; }

}  // namespace mc

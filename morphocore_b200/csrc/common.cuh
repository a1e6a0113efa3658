// Shared device / host helpers of the sm_100a morphology kernels.
//
// Tiling used by every tile kernel in this folder: a CTA of 256 threads owns a 64 x 32 tile of output
// pixels of one image plane; thread (tx, ty) owns the 4 x 2 pixel patch at columns 4 tx .. 4 tx + 3 and
// rows 2 ty, 2 ty + 1. A warp is 8 threads wide and 4 tall, a 32 x 8 pixel block of the tile (see
// thread_patch): its 128-bit shared loads are conflict free (8 lanes = 128 contiguous bytes of one window
// row), and a warp whose block lies entirely outside the image (partial tiles of a 224-wide image) skips
// its arithmetic. The shared window of a tile holds the tile plus the halo of the
// structuring element with the border already resolved:
//     window row r    <-> image row  tile_h0 - (kH - 1 - kH/2) + r
//     window column c <-> image col  tile_w0 - left + c,  left = (kW - 1 - kW/2) rounded up to 16 bytes
// so that tap (kh, kw) of the output pixel at tile offset (y, x) reads window (y + kH-1-kh, off + x + kW-1-kw)
// with off = left - (kW - 1 - kW/2),
// which is image pixel (h + kH/2 - kh, w + kW/2 - kw): the reference's tap convention
// (morphocore/functional/csrc/cuda/morpho_cuda_common.cuh:19, csrc/cpp/morpho_op_cpu_kernels.hxx:256-265).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include <algorithm>
#include <limits>

#include "../../include/morphocore_b200.h"

namespace mc
{

constexpr int TILE_W = 64;
constexpr int TILE_H = 32;
constexpr int THREADS = 256;
constexpr int PATCH_W = 4;  // output pixels per thread along a row
constexpr int PATCH_H = 2;  // output rows per thread

/// Columns a tap can reach to the left of its pixel: tap kw of pixel w reads column w + kW/2 - kw.
__host__ __device__ constexpr int halo_left_of(int kw) { return kw - 1 - kw / 2; }

/// The window starts this many columns left of the tile: the left halo rounded up to a 16-byte multiple,
/// so that the window's first column is a legal TMA x coordinate and rows stay 128-bit aligned.
__host__ __device__ constexpr int halo_left_aligned(int kw, int elem_bytes)
{
    const int per_vec = 16 / elem_bytes;
    return (halo_left_of(kw) + per_vec - 1) / per_vec * per_vec;
}

/// Unused columns at the start of every thread's row segment (the alignment slack above).
__host__ __device__ constexpr int segment_offset(int kw, int elem_bytes) { return halo_left_aligned(kw, elem_bytes) - halo_left_of(kw); }

/// Registers per thread row segment: the slack, the patch and the kernel width, rounded up to whole 128-bit
/// loads. Tap kw of patch pixel j is element segment_offset + j + kW - 1 - kw.
__host__ __device__ constexpr int segment_len(int kw, int elem_bytes)
{
    const int per_vec = 16 / elem_bytes;
    return (segment_offset(kw, elem_bytes) + PATCH_W + kw - 1 + per_vec - 1) / per_vec * per_vec;
}

/// Row stride of the shared window, in elements: every thread may read a whole segment.
__host__ __device__ constexpr int window_stride(int kw, int elem_bytes)
{
    return TILE_W - PATCH_W + segment_len(kw, elem_bytes);
}

struct Geometry
{
    int B, Ci, Co, H, W, kH, kW;
    int pH, pW;        // kH / 2, kW / 2
    int tiles_x, tiles_y;
    int win_rows;      // TILE_H + kH - 1
    int win_stride;    // window_stride(kW)
    int seg_off;       // segment_offset(kW)
    int left;          // halo_left_aligned(kW): window column 0 is image column tile_w0 - left
    int64_t weight_batch_stride;
    bool replicate;
    bool identity;

    __host__ __device__ int taps() const { return kH * kW; }
    __host__ __device__ int64_t plane() const { return static_cast<int64_t>(H) * W; }
    __host__ __device__ int window_elems() const { return win_rows * win_stride; }
    __host__ __device__ int halo_top() const { return kH - 1 - pH; }
    __host__ __device__ int halo_left() const { return left; }
    __host__ __device__ int used_cols() const { return seg_off + TILE_W + kW - 1; }
};

inline Geometry make_geometry(const mc_desc& d, int elem_bytes)
{
    Geometry g;
    g.B = d.B; g.Ci = d.Ci; g.Co = d.Co; g.H = d.H; g.W = d.W; g.kH = d.kH; g.kW = d.kW;
    g.pH = d.kH / 2; g.pW = d.kW / 2;
    g.tiles_x = (d.W + TILE_W - 1) / TILE_W;
    g.tiles_y = (d.H + TILE_H - 1) / TILE_H;
    g.win_rows = TILE_H + d.kH - 1;
    g.win_stride = window_stride(d.kW, elem_bytes);
    g.seg_off = segment_offset(d.kW, elem_bytes);
    g.left = halo_left_aligned(d.kW, elem_bytes);
    g.weight_batch_stride = d.weight_batch_stride;
    g.replicate = d.pad_kind == MC_PAD_REPLICATE;
    g.identity = d.merge == MC_MERGE_IDENTITY;
    return g;
}

/// Patch coordinates of the calling thread and whether its warp's 32 x 8 pixel block has any pixel
/// inside the image.
__device__ __forceinline__ void thread_patch(int tile_h0, int tile_w0, int H, int W, int& tx, int& ty, bool& warp_live)
{
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    tx = (lane & 7) + 8 * (warp & 1);
    ty = (lane >> 3) + 4 * (warp >> 1);
    warp_live = tile_w0 + 32 * (warp & 1) < W && tile_h0 + 8 * (warp >> 1) < H;
}

/// thread_patch for kernels that can divide their output channels between two warps: when the right half of the
/// tile lies outside the image (the last tile column of a 224-wide image), both warps of a warp row take the
/// left 32 x 8 block and `half` (0 or 1) tells which half of the CTA's output channels the warp computes, so that
/// no warp idles. `split` is false (and the mapping that of thread_patch) when `allow` is false.
__device__ __forceinline__ void thread_patch_split(int tile_h0, int tile_w0, int H, int W, bool allow, int& tx, int& ty, bool& warp_live, bool& split,
                                                   int& half)
{
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    split = allow && tile_w0 + 32 >= W;
    half = split ? (warp & 1) : 0;
    tx = (lane & 7) + (split ? 0 : 8 * (warp & 1));
    ty = (lane >> 3) + 4 * (warp >> 1);
    warp_live = (split || tile_w0 + 32 * (warp & 1) < W) && tile_h0 + 8 * (warp >> 1) < H;
}

template <typename T> struct Limits;
template <> struct Limits<float>
{
    __host__ __device__ static constexpr float inf() { return __builtin_huge_valf(); }
    __host__ __device__ static constexpr float max() { return 3.402823466e+38f; }
    // "Never wins, never overflows": sums of a few hundred of these stay finite.
    __host__ __device__ static constexpr float big() { return 1e30f; }
    __host__ __device__ static constexpr float tiny() { return 1e-20f; }
};
template <> struct Limits<double>
{
    __host__ __device__ static constexpr double inf() { return __builtin_huge_val(); }
    __host__ __device__ static constexpr double max() { return 1.7976931348623157e+308; }
    __host__ __device__ static constexpr double big() { return 1e300; }
    __host__ __device__ static constexpr double tiny() { return 1e-200; }
};

/// Stage the window of one image plane into shared memory, border resolved: REPLICATE clamps to the edge
/// pixel, otherwise out-of-image elements read `outside` (the fill value, or NaN for smorph).
/// Warps take rows, lanes take columns, so global reads are coalesced. Columns past the last one a tap
/// can reach are set to `outside` too.
template <typename T>
__device__ __forceinline__ void load_window(T* __restrict__ dst, const T* __restrict__ plane, const Geometry& g, int tile_h0, int tile_w0,
                                            T outside)
{
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int row0 = tile_h0 - g.halo_top(), col0 = tile_w0 - g.halo_left();
    for (int r = warp; r < g.win_rows; r += THREADS / 32)
    {
        const int iy = row0 + r;
        const bool row_in = iy >= 0 && iy < g.H;
        const int cy = min(max(iy, 0), g.H - 1);
        const T* src = plane + static_cast<int64_t>(cy) * g.W;
        T* out = dst + r * g.win_stride;
        for (int c = lane; c < g.win_stride; c += 32)
        {
            const int ix = col0 + c;
            const bool in = row_in && ix >= 0 && ix < g.W;
            T v = outside;
            if (in || g.replicate) v = __ldg(src + min(max(ix, 0), g.W - 1));
            out[c] = v;
        }
    }
}

/// Asynchronous copy of one element from global to shared memory (cp.async: no register staging, completion awaited
/// with cp_async_wait_all). 4 or 8 bytes.
template <typename T>
__device__ __forceinline__ void cp_async_element(T* dst, const T* src)
{
    static_assert(sizeof(T) == 4 || sizeof(T) == 8, "float or double");
    const uint32_t d = static_cast<uint32_t>(__cvta_generic_to_shared(dst));
    if constexpr (sizeof(T) == 4) asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(d), "l"(src) : "memory");
    else asm volatile("cp.async.ca.shared.global [%0], [%1], 8;" ::"r"(d), "l"(src) : "memory");
}
/// Asynchronous copy of 16 bytes (both addresses 16-byte aligned), bypassing L1.
__device__ __forceinline__ void cp_async_16(void* dst, const void* src)
{
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(static_cast<uint32_t>(__cvta_generic_to_shared(dst))), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_all;" ::: "memory"); }

/// load_window with every copy of a thread in flight at once: in-image (or clamped, for REPLICATE) elements travel by
/// cp.async straight into shared memory, out-of-image ones are stored as `outside`. The window's row stride is the
/// compile-time STRIDE and `at(c)` maps a column to its element offset inside the stored row (identity, or a swizzle).
/// The caller runs cp_async_wait_all() and a CTA barrier before reading the window.
template <int STRIDE, typename T, typename At>
__device__ __forceinline__ void stage_window_async(T* __restrict__ dst, const T* __restrict__ plane, const Geometry& g, int tile_h0, int tile_w0,
                                                   T outside, At at)
{
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int row0 = tile_h0 - g.halo_top(), col0 = tile_w0 - g.halo_left();
    // Warps take rows, lanes take columns: no division, one clamped row pointer per row.
    for (int r = warp; r < g.win_rows; r += THREADS / 32)
    {
        const int iy = row0 + r;
        const bool row_in = iy >= 0 && iy < g.H;
        const T* src = plane + static_cast<int64_t>(min(max(iy, 0), g.H - 1)) * g.W;
        T* out = dst + r * STRIDE;
#pragma unroll
        for (int m = 0; m < (STRIDE + 31) / 32; m++)
        {
            const int c = lane + 32 * m;
            if (c >= STRIDE) break;
            const int ix = col0 + c;
            if ((row_in && ix >= 0 && ix < g.W) || g.replicate) cp_async_element(out + at(c), src + min(max(ix, 0), g.W - 1));
            else out[at(c)] = outside;
        }
    }
}

/// Stage the window of one plane for the smorph kernels, whose taps outside the image are excluded. Both
/// windows hold x inside the image; outside, `low` (read by pairs with alpha >= 0, u = x + w) holds -big and
/// `high` (read by pairs with alpha < 0, u = -x - w) holds +big, so that u = -big there: a value that never
/// wins the maximum and whose exponential is exactly zero. Either pointer may be null.
template <typename T>
__device__ __forceinline__ void load_window_signed(T* __restrict__ low, T* __restrict__ high, const T* __restrict__ plane, const Geometry& g,
                                                   int tile_h0, int tile_w0)
{
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int row0 = tile_h0 - g.halo_top(), col0 = tile_w0 - g.halo_left();
    for (int r = warp; r < g.win_rows; r += THREADS / 32)
    {
        const int iy = row0 + r;
        const bool row_in = iy >= 0 && iy < g.H;
        const T* src = plane + static_cast<int64_t>(min(max(iy, 0), g.H - 1)) * g.W;
        for (int c = lane; c < g.win_stride; c += 32)
        {
            const int ix = col0 + c;
            const bool in = row_in && ix >= 0 && ix < g.W;
            const T v = in ? __ldg(src + ix) : T(0);
            if (low != nullptr) low[r * g.win_stride + c] = in ? v : -Limits<T>::big();
            if (high != nullptr) high[r * g.win_stride + c] = in ? v : Limits<T>::big();
        }
    }
}

/// One 128-bit shared load of 16 / sizeof(T) consecutive elements.
__device__ __forceinline__ void lds128(float* dst, const float* src)
{
    const float4 v = *reinterpret_cast<const float4*>(src);
    dst[0] = v.x; dst[1] = v.y; dst[2] = v.z; dst[3] = v.w;
}
__device__ __forceinline__ void lds128(double* dst, const double* src)
{
    const double2 v = *reinterpret_cast<const double2*>(src);
    dst[0] = v.x; dst[1] = v.y;
}

/// Load a thread's row segment of LEN elements (LEN a multiple of the 128-bit vector) from shared memory.
template <int LEN, typename T>
__device__ __forceinline__ void load_segment(T (&dst)[LEN], const T* src)
{
    constexpr int PER = 16 / sizeof(T);
#pragma unroll
    for (int v = 0; v < LEN / PER; v++) lds128(&dst[v * PER], src + v * PER);
}

// max / min with "the other operand when one is NaN" semantics, like the reference's strict
// comparison from an initial value that is never NaN.
template <bool IS_MIN> __device__ __forceinline__ float ext2(float a, float b) { return IS_MIN ? fminf(a, b) : fmaxf(a, b); }
// double: compare + select is more than twice as fast as fmax / fmin on this part (DSETP + 2 SEL against a
// multi-instruction NaN-aware sequence) and has the same result: b replaces a only when strictly better,
// so a NaN in b never wins.
template <bool IS_MIN> __device__ __forceinline__ double ext2(double a, double b) { return (IS_MIN ? b < a : b > a) ? b : a; }

/// Three-input max / min: one sm_100 instruction for two taps.
template <bool IS_MIN> __device__ __forceinline__ float ext3(float a, float b, float c)
{
    // The accumulator is a read-write operand so that the result stays in its register (no move per use).
    if (IS_MIN) asm("min.f32 %0, %0, %1, %2;" : "+f"(a) : "f"(b), "f"(c));
    else asm("max.f32 %0, %0, %1, %2;" : "+f"(a) : "f"(b), "f"(c));
    return a;
}
template <bool IS_MIN> __device__ __forceinline__ double ext3(double a, double b, double c) { return ext2<IS_MIN>(ext2<IS_MIN>(a, b), c); }

template <bool IS_MIN, typename T> __device__ __forceinline__ bool strictly_better(T v, T best) { return IS_MIN ? v < best : v > best; }

/// Value of input pixel (iy, ix) of a plane under the border rule, for the per-pixel re-scans.
template <typename T>
__device__ __forceinline__ T read_border(const T* __restrict__ plane, const Geometry& g, int iy, int ix, T fill)
{
    const bool in = iy >= 0 && iy < g.H && ix >= 0 && ix < g.W;
    if (!in && !g.replicate) return fill;
    return __ldg(plane + static_cast<int64_t>(min(max(iy, 0), g.H - 1)) * g.W + min(max(ix, 0), g.W - 1));
}

// ---------------------------------------------------------------------------------------------
// Host side
// ---------------------------------------------------------------------------------------------
void set_last_error(const char* fmt, ...);
void count_launch();

/// Checks shared by every entry point (sizes, enums, identity shape, index limits); `morph` selects the dilation /
/// erosion fields, `smooth` the smooth-merge entry points. MC_OK or a negative status with the message set.
int validate(const mc_desc* d, bool morph, bool smooth = false);

/// Opt in to more than 48 KiB of dynamic shared memory for a kernel; returns false if the device refuses.
template <typename K> inline bool allow_shared(K kernel, size_t bytes)
{
    if (bytes <= 48 * 1024) return true;
    return cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(bytes)) == cudaSuccess;
}

constexpr size_t MAX_SHARED_BYTES = 227 * 1024;

inline int check_launch(const char* what)
{
    const cudaError_t err = cudaGetLastError();
    if (err != cudaSuccess)
    {
        set_last_error("%s: %s", what, cudaGetErrorString(err));
        return MC_ERR_CUDA;
    }
    count_launch();
    return MC_OK;
}

// Entry points of the translation units, called by api.cu after validation.
template <typename T> int morpho_forward(const mc_desc& d, const T* x, const T* w, T* y, int32_t* idx, cudaStream_t stream);
/// Dilation and erosion (with the flipped structuring element) of one input in one pass; MC_ERR_UNSUPPORTED, with nothing
/// launched, for the cases the fused kernel does not cover.
int morpho_pair_forward(const mc_desc& d, const float* x, const float* w, float* y_dilation, float* y_erosion, cudaStream_t stream);
template <typename T> int morpho_backward(const mc_desc& d, const T* x, const T* w, const int32_t* idx, const T* gy, T* gx, T* gw, void* ws,
                                          cudaStream_t stream);
template <typename T> int smorph_forward(const mc_desc& d, const T* x, const T* w, const T* alpha, T* y, T* counts, cudaStream_t stream);
template <typename T> int smorph_backward(const mc_desc& d, const T* x, const T* w, const T* alpha, const T* y, const T* gy, T* gx, T* gw,
                                          T* galpha, void* ws, cudaStream_t stream);
template <typename T> int smorph_scm_forward(const mc_desc& d, const T* x, const T* w, const T* alpha, const T* beta, T* y, cudaStream_t stream);
template <typename T> int smorph_scm_backward(const mc_desc& d, const T* x, const T* w, const T* alpha, const T* beta, const T* y, const T* gy, T* gx,
                                              T* gw, T* galpha, T* gbeta, void* ws, cudaStream_t stream);

}  // namespace mc

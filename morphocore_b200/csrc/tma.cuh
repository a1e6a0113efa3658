// TMA staging of tile windows: tensor-map creation on the host, mbarrier and cp.async.bulk.tensor wrappers
// on the device. One 4-D tiled copy (no multicast) brings the windows of a whole chunk of input channels
// of one tile into shared memory, out-of-image elements zero filled, while the CTA computes on the
// previous chunk. Every wait on an mbarrier is bounded in time (the device's global timer): when it runs out the
// kernel records the fact in g_device_error and returns instead of spinning.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "common.cuh"

namespace mc
{

/// Device address, on the current device, of the counter a kernel increments when its bounded wait on a
/// TMA copy runs out (read back with mc_device_error_count()); nullptr if it cannot be resolved.
unsigned int* device_error_counter();

/// Tensor map over a contiguous [B, C, H, W] tensor with a box of box_w x box_rows x box_c x 1 elements.
/// Returns false when the tensor cannot be described (row pitch or base not a multiple of 16 bytes, the
/// driver entry point is missing, or the driver rejects the shape): the caller then stages with plain loads.
inline bool make_window_tensor_map(CUtensorMap* map, const void* base, int elem_bytes, int B, int C, int H, int W, int box_w, int box_rows,
                                   int box_c)
{
    using EncodeFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
    static EncodeFn encode = []() -> EncodeFn {
        void* fn = nullptr;
        cudaDriverEntryPointQueryResult status;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &status) != cudaSuccess || status != cudaDriverEntryPointSuccess)
        {
            (void)cudaGetLastError();
            return nullptr;
        }
        return reinterpret_cast<EncodeFn>(fn);
    }();
    if (encode == nullptr) return false;
    const uint64_t row_bytes = static_cast<uint64_t>(W) * elem_bytes;
    if (row_bytes % 16 != 0 || reinterpret_cast<uintptr_t>(base) % 16 != 0) return false;
    if (box_w > 256 || box_rows > 256 || box_c > 256 || (static_cast<uint64_t>(box_w) * elem_bytes) % 16 != 0) return false;
    const cuuint64_t dims[4] = {static_cast<cuuint64_t>(W), static_cast<cuuint64_t>(H), static_cast<cuuint64_t>(C), static_cast<cuuint64_t>(B)};
    const cuuint64_t strides[3] = {row_bytes, row_bytes * H, row_bytes * H * C};
    const cuuint32_t box[4] = {static_cast<cuuint32_t>(box_w), static_cast<cuuint32_t>(box_rows), static_cast<cuuint32_t>(box_c), 1};
    const cuuint32_t elem_strides[4] = {1, 1, 1, 1};
    const CUresult rc = encode(map, elem_bytes == 4 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_FLOAT64, 4, const_cast<void*>(base), dims,
                               strides, box, elem_strides, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                               CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return rc == CUDA_SUCCESS;
}

__device__ __forceinline__ uint32_t smem_addr(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count)
{
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_addr(bar)), "r"(count));
}

/// Makes the barrier initialisation visible to the async proxy.
__device__ __forceinline__ void mbar_fence_init() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }

/// Orders this thread's earlier generic-proxy accesses to shared memory before later async-proxy copies.
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes)
{
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_addr(bar)), "r"(bytes) : "memory");
}

/// Nanoseconds a kernel waits for one TMA copy before it gives up (host side; mc_set_wait_limit_ns changes it, the
/// launchers copy it into the kernel arguments).
uint64_t wait_limit_ns();

__device__ __forceinline__ uint64_t global_timer_ns()
{
    uint64_t t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

/// Bounded wait for the phase with the given parity: tries until `limit_ns` nanoseconds of the device's global
/// timer have passed since the first failed try, then returns false. The timer is only read once a try has failed,
/// so a copy that has already landed costs one try.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, uint64_t limit_ns)
{
    const uint32_t addr = smem_addr(bar);
    uint64_t start = 0;
    for (;;)
    {
        uint32_t done;
        asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.b32 %0, 1, 0, p;\n\t}"
                     : "=r"(done)
                     : "r"(addr), "r"(parity)
                     : "memory");
        if (done) return true;
        const uint64_t now = global_timer_ns();
        if (start == 0) start = now;
        else if (now - start > limit_ns) return false;
    }
}

/// 4-D tiled TMA load (no multicast) of the box at (x, y, c, b) into shared memory; completion is
/// signalled on `bar` by transaction bytes. x * element size must be a multiple of 16 bytes.
__device__ __forceinline__ void tma_load_4d(void* dst, const CUtensorMap* map, uint64_t* bar, int x, int y, int c, int b)
{
    asm volatile("cp.async.bulk.tensor.4d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];" ::"r"(smem_addr(dst)),
                 "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_addr(bar)), "r"(x), "r"(y), "r"(c), "r"(b)
                 : "memory");
}

/// After a TMA copy of a window (zero filled outside the image): overwrite the out-of-image elements of
/// `channels` staged windows with the border rule. Only CTAs whose window leaves the image call this.
/// Only the part of the window that a live warp can read is visited (see thread_patch: the warps of a
/// partial tile whose 32 x 8 block lies outside the image do no arithmetic), which for the half-empty last
/// tile column of a 224-wide image is 4 columns instead of 36.
template <typename T>
__device__ __forceinline__ void fix_window_border(T* __restrict__ win, const T* __restrict__ planes, int64_t plane_stride, int channels,
                                                  const Geometry& g, int tile_h0, int tile_w0, T outside)
{
    const int row0 = tile_h0 - g.halo_top(), col0 = tile_w0 - g.halo_left();
    const int live_cols = g.win_stride - 32 * (TILE_W / 32 - (min(g.W - tile_w0, TILE_W) + 31) / 32);
    const int live_rows = g.win_rows - 8 * (TILE_H / 8 - (min(g.H - tile_h0, TILE_H) + 7) / 8);
    // Window rows [r_lo, r_hi) are image rows; of those, columns [0, n_left) and [first_right, live_cols) lie outside.
    const int r_lo = min(max(-row0, 0), live_rows), r_hi = min(max(g.H - row0, 0), live_rows);
    const int n_left = min(max(-col0, 0), live_cols);
    const int first_right = min(max(g.W - col0, 0), live_cols);
    const int n_side = n_left + live_cols - first_right;
    const int welems = g.window_elems();
    auto put = [&](int c, int wr, int col) {
        T v = outside;
        if (g.replicate)
            v = __ldg(planes + c * plane_stride + static_cast<int64_t>(min(max(row0 + wr, 0), g.H - 1)) * g.W + min(max(col0 + col, 0), g.W - 1));
        win[c * welems + wr * g.win_stride + col] = v;
    };
    if (n_side > 0)
    {
        const int per_channel = (r_hi - r_lo) * n_side;
        for (int e = threadIdx.x; e < channels * per_channel; e += THREADS)
        {
            const int c = e / per_channel, rest = e - c * per_channel;
            const int r = rest / n_side, i = rest - r * n_side;
            put(c, r_lo + r, i < n_left ? i : first_right + i - n_left);
        }
    }
    const int n_out = r_lo + live_rows - r_hi;   // rows above and below the image
    if (n_out > 0)
    {
        const int per_channel = n_out * live_cols;
        for (int e = threadIdx.x; e < channels * per_channel; e += THREADS)
        {
            const int c = e / per_channel, rest = e - c * per_channel;
            const int r = rest / live_cols, col = rest - r * live_cols;
            put(c, r < r_lo ? r : r_hi + r - r_lo, col);
        }
    }
}

__device__ __forceinline__ bool window_leaves_image(const Geometry& g, int tile_h0, int tile_w0)
{
    const int row0 = tile_h0 - g.halo_top(), col0 = tile_w0 - g.halo_left();
    return row0 < 0 || col0 < 0 || row0 + g.win_rows > g.H || col0 + g.win_stride > g.W;
}

}  // namespace mc

/* C-ABI of the B200 (sm_100a) dilation / erosion / smorph kernels.
 *
 * The reference has no C interface of its own: its Python operators (torch.ops.morphocore.*) call four
 * C++ templates over at::Tensor. Each function below replaces one of those templates with plain
 * device pointers and sizes, so that any host language can bind it. Paths are relative to the
 * reference project root, "CU/" = morphocore/functional/csrc/cuda/, "CPP/" = morphocore/functional/csrc/cpp/.
 *
 * Conventions
 *  - Every pointer is a device pointer on the device that is current when the call is made, tensors are
 *    contiguous NCHW (input, output, gradients) or OIHW (structuring element), float32 or float64.
 *  - The compute functions never allocate, free or synchronise: work is queued on `stream` (a cudaStream_t
 *    passed as void*, NULL = the legacy default stream), scratch memory is passed in by the caller. The one
 *    exception is mc_morpho_backward_noalloc, whose scratch is an array inside the library (see there).
 *  - The return value is MC_OK or a negative mc_status; mc_status_string() names it and
 *    mc_last_error() gives the detail of the last failure of the calling thread.
 *  - The compute functions are re-entrant and thread safe, except mc_morpho_backward_noalloc, whose calls on one
 *    device share one scratch array. Process state: the per-kernel shared-memory opt-in, the wait limit
 *    (mc_set_wait_limit_ns), the launch counter and, per device, the counter of timed-out waits
 *    (mc_device_error_count), which hosts should poll at their own synchronisation points: a thread block whose
 *    wait ran out returns without writing its tile, and the call that launched it has long returned MC_OK.
 */
#ifndef MORPHOCORE_B200_H
#define MORPHOCORE_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* MORPHO_OPERATION, CPP/morpho_op_enum.hpp:4-8. */
enum mc_op { MC_OP_DILATION = 0, MC_OP_EROSION = 1 };

/* Channel merge, the integers of MORPHO_MERGE (CPP/morpho_op_enum.hpp:18-26) that
 * morphocore/functional/merge_enum.py:4-11 sends through the operator schema. SMOOTH (4) is the merge of the
 * mc_smorph_scm_* entry points only. */
enum mc_merge { MC_MERGE_MAX = 0, MC_MERGE_MIN = 1, MC_MERGE_ADD = 2, MC_MERGE_AVERAGE = 3, MC_MERGE_SMOOTH = 4, MC_MERGE_IDENTITY = 5 };

/* Padding family, MORPHO_PADDING_KIND (CPP/morpho_op_enum.hpp:41-45): out-of-image taps read `fill`
 * (zero, geodesic and constant modes, resolved to a value by morpho_fill_value,
 * CPP/morpho_padding_policy.hpp:23-33) or the clamped edge pixel. */
enum mc_pad_kind { MC_PAD_FILL = 0, MC_PAD_REPLICATE = 1 };

enum mc_dtype { MC_F32 = 0, MC_F64 = 1 };

enum mc_status
{
    MC_OK = 0,
    MC_ERR_INVALID_ARGUMENT = -1, /* NULL pointer, non-positive size, unknown enum, identity with Co != Ci */
    MC_ERR_UNSUPPORTED = -2,      /* structuring element too large for shared memory or for packed indices */
    MC_ERR_WORKSPACE = -3,        /* workspace smaller than mc_*_workspace_bytes() */
    MC_ERR_CUDA = -4              /* a CUDA runtime call failed; mc_last_error() has the message */
};

/* Shapes and modes of one call; replaces MorphoGeometryCUDA (CU/morpho_cuda_launch.cuh:17-38) plus the
 * merge / border arguments of the reference launchers. For MC_MERGE_IDENTITY the structuring element is
 * [Co, 1, kH, kW] and Co must equal Ci (CPP/morpho_op_wrap.hxx:75-76). */
typedef struct mc_desc
{
    int32_t B, Ci, Co, H, W, kH, kW;
    int32_t op;       /* mc_op; ignored by the smorph functions */
    int32_t merge;    /* mc_merge */
    int32_t pad_kind; /* mc_pad_kind; ignored by the smorph functions (out-of-image taps are excluded) */
    int32_t dtype;    /* mc_dtype */
    int32_t reserved; /* must be 0 */
    double fill;      /* border value of MC_PAD_FILL */
    int64_t weight_batch_stride; /* elements between the structuring elements of two batch elements
                                    ([B, Co, Ci', kH, kW] weights of the noise path, CU/morpho_cuda_launch.cuh:36); 0 = shared */
} mc_desc;

/* Forward dilation / erosion with the fused channel merge.
 * Replaces morpho_forward_cuda<op, T> (CU/morpho_op.cuh:16-19, CU/morpho_op.cu:30-74).
 * y[b,o,h,w] = merge_i ext_{kh,kw} ( x[b,i,h+kH/2-kh,w+kW/2-kw] (+|-) w[o,i,kh,kw] ); erosion subtracts `w` as
 * given (the Python layer passes the flipped structuring element, morphocore/functional/erosion.py:89).
 * idx (nullable, int32 [B,Co,H,W]) receives (channel << 16) | tap of the winner, MAX / MIN merges only. */
int mc_morpho_forward(const mc_desc* desc, const void* x, const void* w, void* y, int32_t* idx, void* stream);

/* Dilation AND erosion of one input with one structuring element in a single pass: the two halves of the reference's
 * sigma_layer composition (morphocore/functional/sigma_layer.py:73-83), which calls erosion(x, w) and dilation(x, w) one
 * after the other. `w` is the structuring element as the user holds it: the erosion half uses its flipped copy, as
 * morphocore/functional/erosion.py:89 does, and desc->op is ignored. Results are bit-identical to two mc_morpho_forward
 * calls. Covers float, square 3 x 3 / 5 x 5 / 7 x 7 structuring elements, shared (not per-sample) weights and borders
 * that are the same for both operations (replicate, zero, a finite constant); no winner index is produced. Every other
 * case returns MC_ERR_UNSUPPORTED with nothing launched: run the two passes separately. */
int mc_morpho_pair_forward(const mc_desc* desc, const void* x, const void* w, void* y_dilation, void* y_erosion, void* stream);

/* Scratch bytes mc_morpho_backward needs: the recomputed winners when idx is NULL for a MAX / MIN merge,
 * otherwise 0. */
size_t mc_morpho_backward_workspace_bytes(const mc_desc* desc, int have_idx);

/* Backward dilation / erosion. Replaces morpho_backward_cuda<op, T> (CU/morpho_op.cuh:21-24,
 * CU/morpho_op.cu:102-177). gx [B,Ci,H,W] and gw (shape of the shared structuring element) are
 * overwritten (zeroed then accumulated). idx is the tensor written by mc_morpho_forward or NULL. */
int mc_morpho_backward(const mc_desc* desc, const void* x, const void* w, const int32_t* idx, const void* gy, void* gx, void* gw,
                       void* workspace, size_t workspace_bytes, void* stream);

/* Backward dilation / erosion for hosts that cannot allocate device memory (a server whose arena owns the
 * whole GPU, a plugin inside another framework's pool, a loop that cannot afford cudaMalloc's device
 * synchronisation). Same results as mc_morpho_backward called with idx = NULL, but the winners of MAX /
 * MIN merges are recomputed into a fixed MC_NOALLOC_SCRATCH_BYTES array inside the library image instead
 * of a caller workspace: no allocation by either side. This entry point has no counterpart in the
 * reference, whose wrapper always allocates with torch.
 *  - limit: B*Co*H*W <= MC_NOALLOC_SCRATCH_BYTES / 4 output pixels for MAX / MIN merges (other merges need
 *    no scratch and have no limit); larger calls return MC_ERR_UNSUPPORTED;
 *  - every GPU that loads the library holds the array until the process exits;
 *  - the first call on each device resolves the array's address: make it before any stream capture;
 *  - calls on one device share the array (it keeps the last call's winners; nothing needs zeroing, each
 *    call overwrites what it reads), so calls that overlap on the GPU race: serialise them. */
#define MC_NOALLOC_SCRATCH_BYTES (16u * 1024u * 1024u)
int mc_morpho_backward_noalloc(const mc_desc* desc, const void* x, const void* w, const void* gy, void* gx, void* gw, void* stream);

/* Forward smorph (alpha-softmax soft extremum) with the fused channel merge.
 * Replaces smorph_forward_cuda<T> (CU/smorph.cuh:15-18, CU/smorph.cu:52-61) for every merge but SMOOTH
 * (mc_smorph_scm_forward).
 * alpha_pairs holds one value per (o, i) pair, [Co, Ci] ([Co] for identity), as produced by
 * smorph_pair_alphas (CPP/smorph_cpu_kernels.hxx:643-649). `w` is the re-parametrised structuring element. */
int mc_smorph_forward(const mc_desc* desc, const void* x, const void* w, const void* alpha_pairs, void* y, void* stream);

/* Scratch bytes mc_smorph_backward needs: per output pixel winner counts for MAX / MIN merges, else 0. */
size_t mc_smorph_backward_workspace_bytes(const mc_desc* desc);

/* Backward smorph. Replaces smorph_backward_cuda<T> (CU/smorph.cuh:20-25, CU/smorph.cu:63-103).
 * y is the forward output (the merge target of MAX / MIN). gx, gw and galpha_pairs (one value per pair,
 * like alpha_pairs) are overwritten. */
int mc_smorph_backward(const mc_desc* desc, const void* x, const void* w, const void* alpha_pairs, const void* y, const void* gy, void* gx,
                       void* gw, void* galpha_pairs, void* workspace, size_t workspace_bytes, void* stream);

/* Smorph with the smooth channel merge ("Smorph SCM"): the Ci soft extrema c_i of an output pixel are merged by a
 * second soft extremum, final = sum_i q_i c_i / sum_i q_i with q_i = exp(beta[o] (c_i - ref)), ref = max_i c_i for
 * beta[o] >= 0 and min_i c_i otherwise (CPP/smorph_cpu_kernels.hxx:231-266).
 * Replaces smorph_forward_cuda<T> called with MORPHO_MERGE::SMOOTH (CU/smorph.cuh:15-18, CPP/smorph_scm.cpp:13-56).
 * desc->merge must be MC_MERGE_SMOOTH; alpha_pairs is [Co, Ci], beta [Co]. */
int mc_smorph_scm_forward(const mc_desc* desc, const void* x, const void* w, const void* alpha_pairs, const void* beta, void* y, void* stream);

/* Scratch bytes mc_smorph_scm_backward needs: ref and 1 / sum_i q_i of every output pixel. */
size_t mc_smorph_scm_backward_workspace_bytes(const mc_desc* desc);

/* Backward of mc_smorph_scm_forward. Replaces smorph_backward_cuda<T> called with MORPHO_MERGE::SMOOTH
 * (CU/smorph.cuh:20-25, CPP/smorph_scm.cpp:58-96). y is the forward output. gx, gw, galpha_pairs ([Co, Ci]) and
 * gbeta ([Co]) are overwritten. */
int mc_smorph_scm_backward(const mc_desc* desc, const void* x, const void* w, const void* alpha_pairs, const void* beta, const void* y,
                           const void* gy, void* gx, void* gw, void* galpha_pairs, void* gbeta, void* workspace, size_t workspace_bytes,
                           void* stream);

const char* mc_status_string(int status);
const char* mc_last_error(void);

/* Number of thread blocks, on the current device since the library was loaded, whose bounded wait on an
 * asynchronous (TMA) copy ran out and which therefore returned early: 0 in a healthy run. Synchronises
 * the device; negative mc_status on failure. No counterpart in the reference (its kernels do not wait). */
int mc_device_error_count(void);

/* Sets the counter read by mc_device_error_count back to zero on the current device. */
int mc_device_error_reset(void);

/* Time limit, in nanoseconds of the GPU's global timer, of every wait on an asynchronous copy in kernels launched
 * from now on (default 1 s). No counterpart in the reference. */
int mc_set_wait_limit_ns(uint64_t limit_ns);

/* Self-test of the time-out path: queues one thread block that waits, with the same bounded wait as the kernels,
 * for a copy that is never issued. After limit_ns (at most 1 s) it gives up, adds one to the counter of
 * mc_device_error_count and returns; the context stays usable. No counterpart in the reference. */
int mc_selftest_wait_timeout(uint64_t limit_ns, void* stream);

/* Number of kernels this library has launched in the calling process since it was loaded. */
uint64_t mc_launch_count(void);

/* Library version, major * 10000 + minor * 100 + patch. */
int mc_version(void);

#ifdef __cplusplus
}
#endif

#endif /* MORPHOCORE_B200_H */

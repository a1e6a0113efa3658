// Thin PyTorch extension: registers torch.ops.morphocore.{dilation, erosion, smorph, smorph_scm} with the
// reference's schemas (morphocore/functional/csrc/cpp/bindings.cpp:130-148) and forwards them, through two
// autograd Functions, to the C-ABI of include/morphocore_b200.h. It mirrors the reference wrappers
// (csrc/cpp/morpho_op_wrap.hxx:25-211, csrc/cpp/smorph.cpp:21-111): 2-D / 3-D inputs and 2-D weights are
// lifted to 4-D, the same checks raise the same messages, the wrapper owns every allocation and the
// kernels only write into caller buffers. There is no CPU path: CPU tensors are rejected.
#include <nvtx3/nvToolsExt.h>
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/all.h>
#include <torch/library.h>

#include "morphocore_b200.h"

namespace
{

constexpr int64_t PAD_ZERO = 0, PAD_GEODESIC = 1, PAD_CONSTANT = 2, PAD_REPLICATE = 3;

/// NVTX range around one operator call (forward or backward), so that the kernels of a layer group under its name in a
/// timeline. The reference has no tracing of its own. NVTX 3 is header only: without a profiler attached a range costs a
/// few nanoseconds.
struct TraceRange
{
    explicit TraceRange(const char* name) { nvtxRangePushA(name); }
    ~TraceRange() { nvtxRangePop(); }
    TraceRange(const TraceRange&) = delete;
    TraceRange& operator=(const TraceRange&) = delete;
};

void check_status(int rc)
{
    TORCH_CHECK(rc == MC_OK, mc_status_string(rc), ": ", mc_last_error());
}

/// Lift a 2-D / 3-D / 4-D input to [B, C, H, W] (csrc/cpp/reshaper.cpp:3-56).
torch::Tensor input_to_4d(const torch::Tensor& input)
{
    switch (input.dim())
    {
        case 4: return input;
        case 3: return input.unsqueeze(0);
        case 2: return input.unsqueeze(0).unsqueeze(0);
        default:
            TORCH_CHECK(false, "Invalid input tensor: please give a 2D, 3D or 4D input tensor, received: ", input.dim(), " dimensions !");
    }
}

/// Lift a 2-D / 4-D weight to [Co, Ci, kH, kW] (csrc/cpp/reshaper.cpp:82-128).
torch::Tensor weight_to_4d(const torch::Tensor& weight)
{
    switch (weight.dim())
    {
        case 4: return weight;
        case 2: return weight.unsqueeze(0).unsqueeze(0);
        default: TORCH_CHECK(false, "Invalid weight tensor dimensions: expected 2D or 4D tensor, received ", weight.dim(), "D tensor");
    }
}

torch::Tensor output_to_original(const torch::Tensor& output, int64_t original_dims)
{
    if (original_dims == 3) return output.squeeze(0);
    if (original_dims == 2) return output.squeeze(0).squeeze(0);
    return output;
}

int dtype_of(const torch::Tensor& t)
{
    TORCH_CHECK(t.scalar_type() == torch::kFloat || t.scalar_type() == torch::kDouble, "morphocore kernels take float32 or float64 tensors, got ",
                t.scalar_type());
    return t.scalar_type() == torch::kFloat ? MC_F32 : MC_F64;
}

void require_cuda(const torch::Tensor& t, const char* what)
{
    TORCH_CHECK(t.is_cuda(), "morphocore_b200 runs on CUDA devices only and has no CPU path: ", what, " is on ", t.device());
}

mc_desc make_desc(const torch::Tensor& input4d, const torch::Tensor& weight4d, int64_t op, int64_t merge)
{
    mc_desc d{};
    d.B = static_cast<int32_t>(input4d.size(0));
    d.Ci = static_cast<int32_t>(input4d.size(1));
    d.H = static_cast<int32_t>(input4d.size(2));
    d.W = static_cast<int32_t>(input4d.size(3));
    d.Co = static_cast<int32_t>(weight4d.size(0));
    d.kH = static_cast<int32_t>(weight4d.size(2));
    d.kW = static_cast<int32_t>(weight4d.size(3));
    d.op = static_cast<int32_t>(op);
    d.merge = static_cast<int32_t>(merge);
    d.dtype = dtype_of(input4d);
    return d;
}

/// Border value of the FILL family (csrc/cpp/morpho_padding_policy.hpp:23-33).
double fill_value(int64_t op, int64_t padding, double padding_value, bool single)
{
    if (padding == PAD_ZERO) return 0.0;
    if (padding == PAD_CONSTANT) return single ? static_cast<double>(static_cast<float>(padding_value)) : padding_value;
    return op == MC_OP_DILATION ? -std::numeric_limits<double>::infinity() : std::numeric_limits<double>::infinity();
}

class MorphoFunction : public torch::autograd::Function<MorphoFunction>
{
public:
    static torch::Tensor forward(torch::autograd::AutogradContext* ctx, torch::Tensor input, torch::Tensor weight, int64_t op, int64_t merge,
                                 int64_t padding, double padding_value, bool save_indices, double noise_scale)
    {
        TORCH_CHECK(noise_scale >= 0.0, "noise_scale must be non negative");
        const int64_t original_dims = input.dim();
        torch::Tensor input4d = input_to_4d(input);
        torch::Tensor weight4d = weight_to_4d(weight);
        const bool identity = merge == MC_MERGE_IDENTITY;
        TORCH_CHECK(input4d.size(1) == weight4d.size(1) || identity, "Input channels must match weight input channels");
        require_cuda(input, "input");
        require_cuda(weight, "weight");
        TORCH_CHECK(input.device() == weight.device(), "input and weight must be on the same device");
        TORCH_CHECK(input.scalar_type() == weight.scalar_type(), "input and weight must have the same dtype");
        if (identity)
        {
            TORCH_CHECK(weight4d.size(0) == input4d.size(1), "Identity mode requires weight.shape[0] == input.shape[1]");
            TORCH_CHECK(weight4d.size(1) == 1, "Identity mode requires weight.shape[1] == 1");
        }
        const c10::cuda::CUDAGuard device_guard(input.device());
        input4d = input4d.contiguous();
        weight4d = weight4d.contiguous();

        mc_desc d = make_desc(input4d, weight4d, op, merge);
        d.pad_kind = padding == PAD_REPLICATE ? MC_PAD_REPLICATE : MC_PAD_FILL;
        d.fill = fill_value(op, padding, padding_value, d.dtype == MC_F32);

        // One structuring element per batch element, drawn on the weight's device from its generator
        // (csrc/cpp/morpho_op_wrap.hxx:55-64).
        torch::Tensor sample_weight;
        if (noise_scale > 0.0)
        {
            const torch::Tensor noise =
                (torch::rand({input4d.size(0), weight4d.size(0), weight4d.size(1), weight4d.size(2), weight4d.size(3)}, weight4d.options()) * 2.0 - 1.0)
                * noise_scale;
            sample_weight = (weight4d.unsqueeze(0) + noise).contiguous();
            d.weight_batch_stride = weight4d.numel();
        }
        const torch::Tensor& kernel_weight = sample_weight.defined() ? sample_weight : weight4d;

        torch::Tensor output = torch::empty({input4d.size(0), weight4d.size(0), input4d.size(2), input4d.size(3)}, input4d.options());
        torch::Tensor indices;
        if (save_indices && (merge == MC_MERGE_MAX || merge == MC_MERGE_MIN))
            indices = torch::empty(output.sizes(), input4d.options().dtype(torch::kInt));

        const TraceRange trace("morphocore::morpho_forward");
        check_status(mc_morpho_forward(&d, input4d.data_ptr(), kernel_weight.data_ptr(), output.data_ptr(),
                                       indices.defined() ? indices.data_ptr<int32_t>() : nullptr, at::cuda::getCurrentCUDAStream().stream()));

        ctx->save_for_backward({input4d, weight4d, indices, sample_weight});
        ctx->saved_data["op"] = op;
        ctx->saved_data["merge"] = merge;
        ctx->saved_data["pad_kind"] = static_cast<int64_t>(d.pad_kind);
        ctx->saved_data["fill"] = d.fill;
        ctx->saved_data["input_dims"] = original_dims;
        ctx->saved_data["weight_dims"] = weight.dim();
        return output_to_original(output, original_dims);
    }

    static torch::autograd::tensor_list backward(torch::autograd::AutogradContext* ctx, torch::autograd::tensor_list grad_outputs)
    {
        const auto saved = ctx->get_saved_variables();
        const torch::Tensor& input = saved[0];
        const torch::Tensor& weight = saved[1];
        const torch::Tensor& indices = saved[2];
        const torch::Tensor& sample_weight = saved[3];
        torch::Tensor grad_output = input_to_4d(grad_outputs[0]).contiguous();

        std::vector<int64_t> expected = input.sizes().vec();
        expected[1] = weight.size(0);
        TORCH_CHECK(grad_output.sizes() == c10::IntArrayRef(expected), "grad_output shape mismatch: expected [", c10::IntArrayRef(expected),
                    "] but got [", grad_output.sizes(), "]");
        TORCH_CHECK(grad_output.device() == input.device(), "grad_output must be on the same device as input");
        TORCH_CHECK(grad_output.scalar_type() == input.scalar_type(), "grad_output must have the same dtype as input");

        const c10::cuda::CUDAGuard device_guard(input.device());
        mc_desc d = make_desc(input, weight, ctx->saved_data["op"].toInt(), ctx->saved_data["merge"].toInt());
        d.pad_kind = static_cast<int32_t>(ctx->saved_data["pad_kind"].toInt());
        d.fill = ctx->saved_data["fill"].toDouble();
        // The noisy weights chose the winning taps; grad_weight keeps the shared shape, summed over the batch.
        const torch::Tensor& kernel_weight = sample_weight.defined() ? sample_weight : weight;
        if (sample_weight.defined()) d.weight_batch_stride = weight.numel();

        torch::Tensor grad_input = torch::empty_like(input);
        torch::Tensor grad_weight = torch::empty_like(weight);
        const bool have_idx = indices.defined() && indices.numel() > 0;
        const size_t ws_bytes = mc_morpho_backward_workspace_bytes(&d, have_idx);
        torch::Tensor workspace;
        if (ws_bytes > 0) workspace = torch::empty({static_cast<int64_t>(ws_bytes)}, input.options().dtype(torch::kByte));

        const TraceRange trace("morphocore::morpho_backward");
        check_status(mc_morpho_backward(&d, input.data_ptr(), kernel_weight.data_ptr(), have_idx ? indices.data_ptr<int32_t>() : nullptr,
                                        grad_output.data_ptr(), grad_input.data_ptr(), grad_weight.data_ptr(),
                                        workspace.defined() ? workspace.data_ptr() : nullptr, ws_bytes, at::cuda::getCurrentCUDAStream().stream()));

        grad_input = output_to_original(grad_input, ctx->saved_data["input_dims"].toInt());
        if (ctx->saved_data["weight_dims"].toInt() == 2) grad_weight = grad_weight.squeeze(0).squeeze(0);
        return {grad_input, grad_weight, torch::Tensor(), torch::Tensor(), torch::Tensor(), torch::Tensor(), torch::Tensor(), torch::Tensor()};
    }
};

/// dilation(x, w) and erosion(x, w) of the SAME input and structuring element, the two halves of the reference's
/// sigma_layer (morphocore/functional/sigma_layer.py:73-83). The forward pass is one fused kernel where
/// mc_morpho_pair_forward covers the case and two mc_morpho_forward calls otherwise; the backward pass is the two
/// mc_morpho_backward calls the separate operators would make (winners recomputed: no index is kept), their input
/// gradients added and the erosion's weight gradient flipped back (erosion works on the flipped structuring element,
/// morphocore/functional/erosion.py:89).
class MorphoPairFunction : public torch::autograd::Function<MorphoPairFunction>
{
public:
    static torch::autograd::tensor_list forward(torch::autograd::AutogradContext* ctx, torch::Tensor input, torch::Tensor weight, int64_t merge,
                                                int64_t padding, double padding_value)
    {
        const int64_t original_dims = input.dim();
        torch::Tensor input4d = input_to_4d(input);
        torch::Tensor weight4d = weight_to_4d(weight);
        const bool identity = merge == MC_MERGE_IDENTITY;
        TORCH_CHECK(input4d.size(1) == weight4d.size(1) || identity, "Input channels must match weight input channels");
        require_cuda(input, "input");
        require_cuda(weight, "weight");
        TORCH_CHECK(input.device() == weight.device(), "input and weight must be on the same device");
        TORCH_CHECK(input.scalar_type() == weight.scalar_type(), "input and weight must have the same dtype");
        if (identity)
        {
            TORCH_CHECK(weight4d.size(0) == input4d.size(1), "Identity mode requires weight.shape[0] == input.shape[1]");
            TORCH_CHECK(weight4d.size(1) == 1, "Identity mode requires weight.shape[1] == 1");
        }
        const c10::cuda::CUDAGuard device_guard(input.device());
        input4d = input4d.contiguous();
        weight4d = weight4d.contiguous();
        const torch::Tensor flipped = weight4d.flip({2, 3}).contiguous();

        mc_desc d = make_desc(input4d, weight4d, MC_OP_DILATION, merge);
        d.pad_kind = padding == PAD_REPLICATE ? MC_PAD_REPLICATE : MC_PAD_FILL;
        d.fill = fill_value(MC_OP_DILATION, padding, padding_value, d.dtype == MC_F32);
        torch::Tensor out_dilation = torch::empty({input4d.size(0), weight4d.size(0), input4d.size(2), input4d.size(3)}, input4d.options());
        torch::Tensor out_erosion = torch::empty_like(out_dilation);
        const cudaStream_t stream = at::cuda::getCurrentCUDAStream().stream();
        {
            const TraceRange trace("morphocore::morpho_pair_forward");
            const int rc = mc_morpho_pair_forward(&d, input4d.data_ptr(), weight4d.data_ptr(), out_dilation.data_ptr(), out_erosion.data_ptr(), stream);
            if (rc == MC_ERR_UNSUPPORTED)
            {
                check_status(mc_morpho_forward(&d, input4d.data_ptr(), weight4d.data_ptr(), out_dilation.data_ptr(), nullptr, stream));
                mc_desc e = d;
                e.op = MC_OP_EROSION;
                e.fill = fill_value(MC_OP_EROSION, padding, padding_value, d.dtype == MC_F32);
                check_status(mc_morpho_forward(&e, input4d.data_ptr(), flipped.data_ptr(), out_erosion.data_ptr(), nullptr, stream));
            }
            else check_status(rc);
        }
        ctx->save_for_backward({input4d, weight4d, flipped});
        ctx->saved_data["merge"] = merge;
        ctx->saved_data["padding"] = padding;
        ctx->saved_data["padding_value"] = padding_value;
        ctx->saved_data["input_dims"] = original_dims;
        ctx->saved_data["weight_dims"] = weight.dim();
        return {output_to_original(out_dilation, original_dims), output_to_original(out_erosion, original_dims)};
    }

    static torch::autograd::tensor_list backward(torch::autograd::AutogradContext* ctx, torch::autograd::tensor_list grad_outputs)
    {
        const auto saved = ctx->get_saved_variables();
        const torch::Tensor& input = saved[0];
        const torch::Tensor& weight = saved[1];
        const torch::Tensor& flipped = saved[2];
        const int64_t merge = ctx->saved_data["merge"].toInt(), padding = ctx->saved_data["padding"].toInt();
        const double padding_value = ctx->saved_data["padding_value"].toDouble();
        const c10::cuda::CUDAGuard device_guard(input.device());
        const cudaStream_t stream = at::cuda::getCurrentCUDAStream().stream();

        torch::Tensor grad_input, grad_weight;
        for (int op = MC_OP_DILATION; op <= MC_OP_EROSION; op++)
        {
            const torch::Tensor& upstream = grad_outputs[op == MC_OP_DILATION ? 0 : 1];
            if (!upstream.defined()) continue;   // that half of the pair was not used
            torch::Tensor grad_output = input_to_4d(upstream).contiguous();
            std::vector<int64_t> expected = input.sizes().vec();
            expected[1] = weight.size(0);
            TORCH_CHECK(grad_output.sizes() == c10::IntArrayRef(expected), "grad_output shape mismatch: expected [", c10::IntArrayRef(expected),
                        "] but got [", grad_output.sizes(), "]");
            TORCH_CHECK(grad_output.device() == input.device(), "grad_output must be on the same device as input");
            TORCH_CHECK(grad_output.scalar_type() == input.scalar_type(), "grad_output must have the same dtype as input");
            mc_desc d = make_desc(input, weight, op, merge);
            d.pad_kind = padding == PAD_REPLICATE ? MC_PAD_REPLICATE : MC_PAD_FILL;
            d.fill = fill_value(op, padding, padding_value, d.dtype == MC_F32);
            const torch::Tensor& kernel_weight = op == MC_OP_DILATION ? weight : flipped;
            torch::Tensor gx = torch::empty_like(input), gw = torch::empty_like(weight);
            const size_t ws_bytes = mc_morpho_backward_workspace_bytes(&d, 0);
            torch::Tensor workspace;
            if (ws_bytes > 0) workspace = torch::empty({static_cast<int64_t>(ws_bytes)}, input.options().dtype(torch::kByte));
            const TraceRange trace("morphocore::morpho_backward");
            check_status(mc_morpho_backward(&d, input.data_ptr(), kernel_weight.data_ptr(), nullptr, grad_output.data_ptr(), gx.data_ptr(), gw.data_ptr(),
                                            workspace.defined() ? workspace.data_ptr() : nullptr, ws_bytes, stream));
            if (op == MC_OP_EROSION) gw = gw.flip({2, 3});
            grad_input = grad_input.defined() ? grad_input + gx : gx;
            grad_weight = grad_weight.defined() ? grad_weight + gw : gw;
        }
        if (grad_input.defined())
        {
            grad_input = output_to_original(grad_input, ctx->saved_data["input_dims"].toInt());
            if (ctx->saved_data["weight_dims"].toInt() == 2) grad_weight = grad_weight.squeeze(0).squeeze(0);
        }
        return {grad_input, grad_weight, torch::Tensor(), torch::Tensor(), torch::Tensor()};
    }
};

/// One alpha per (o, i) pair, a single value being shared by all (csrc/cpp/smorph_cpu_kernels.hxx:643-649).
torch::Tensor pair_alphas(const torch::Tensor& alpha, int64_t merge, int64_t out_channels, int64_t in_channels)
{
    const bool identity = merge == MC_MERGE_IDENTITY;
    const int64_t pairs = identity ? out_channels : out_channels * in_channels;
    TORCH_CHECK(alpha.numel() == pairs || alpha.numel() == 1, "Alpha must have one value, or shape ",
                identity ? "[channels]" : "[out_channels, in_channels]");
    return alpha.numel() == pairs ? alpha.contiguous() : alpha.reshape({1}).expand({pairs}).contiguous();
}

class SmorphFunction : public torch::autograd::Function<SmorphFunction>
{
public:
    static torch::Tensor forward(torch::autograd::AutogradContext* ctx, torch::Tensor input, torch::Tensor weight, torch::Tensor alpha, int64_t merge)
    {
        const int64_t original_dims = input.dim();
        torch::Tensor input4d = input_to_4d(input);
        torch::Tensor weight4d = weight_to_4d(weight);
        require_cuda(input, "input");
        require_cuda(weight, "weight");
        require_cuda(alpha, "alpha");
        TORCH_CHECK(weight.device() == input.device() && alpha.device() == input.device(),
                    "input, weight and alpha must be on the same device (input on ", input.device(), ", weight on ", weight.device(),
                    ", alpha on ", alpha.device(), ")");
        TORCH_CHECK(input.scalar_type() == weight.scalar_type() && input.scalar_type() == alpha.scalar_type(),
                    "input, weight and alpha must have the same dtype");
        const bool identity = merge == MC_MERGE_IDENTITY;
        if (identity)
        {
            TORCH_CHECK(weight4d.size(0) == input4d.size(1), "Identity mode requires weight.shape[0] == input.shape[1]");
            TORCH_CHECK(weight4d.size(1) == 1, "Identity mode requires weight.shape[1] == 1, got ", weight4d.size(1));
        }
        else
        {
            TORCH_CHECK(input4d.size(1) == weight4d.size(1), "Input channels must match weight input channels");
        }
        const c10::cuda::CUDAGuard device_guard(input.device());
        input4d = input4d.contiguous();
        weight4d = weight4d.contiguous();
        const torch::Tensor alphas = pair_alphas(alpha, merge, weight4d.size(0), input4d.size(1));

        const mc_desc d = make_desc(input4d, weight4d, MC_OP_DILATION, merge);
        torch::Tensor output = torch::empty({input4d.size(0), weight4d.size(0), input4d.size(2), input4d.size(3)}, input4d.options());
        const TraceRange trace("morphocore::smorph_forward");
        check_status(mc_smorph_forward(&d, input4d.data_ptr(), weight4d.data_ptr(), alphas.data_ptr(), output.data_ptr(),
                                       at::cuda::getCurrentCUDAStream().stream()));

        // The backward pass reads the 4-D output: the merge target of MAX and MIN.
        ctx->save_for_backward({output, alpha, input4d, weight4d});
        ctx->saved_data["merge"] = merge;
        ctx->saved_data["input_dims"] = original_dims;
        ctx->saved_data["weight_dims"] = weight.dim();
        return output_to_original(output, original_dims);
    }

    static torch::autograd::tensor_list backward(torch::autograd::AutogradContext* ctx, torch::autograd::tensor_list grad_outputs)
    {
        const auto saved = ctx->get_saved_variables();
        const torch::Tensor& output = saved[0];
        const torch::Tensor& alpha = saved[1];
        const torch::Tensor& input = saved[2];
        const torch::Tensor& weight = saved[3];
        const int64_t merge = ctx->saved_data["merge"].toInt();
        torch::Tensor grad_output = input_to_4d(grad_outputs[0]).contiguous();
        TORCH_CHECK(grad_output.sizes() == output.sizes(), "grad_output shape mismatch: expected [", output.sizes(), "] but got [",
                    grad_output.sizes(), "]");
        TORCH_CHECK(grad_output.scalar_type() == input.scalar_type(), "grad_output must have the same dtype as input");
        TORCH_CHECK(grad_output.device() == input.device(), "grad_output must be on the same device as input");

        const c10::cuda::CUDAGuard device_guard(input.device());
        const mc_desc d = make_desc(input, weight, MC_OP_DILATION, merge);
        const torch::Tensor alphas = pair_alphas(alpha, merge, weight.size(0), input.size(1));
        torch::Tensor grad_input = torch::empty_like(input);
        torch::Tensor grad_weight = torch::empty_like(weight);
        torch::Tensor grad_alpha_pairs = torch::empty_like(alphas);
        const size_t ws_bytes = mc_smorph_backward_workspace_bytes(&d);
        torch::Tensor workspace;
        if (ws_bytes > 0) workspace = torch::empty({static_cast<int64_t>(ws_bytes)}, input.options().dtype(torch::kByte));

        const TraceRange trace("morphocore::smorph_backward");
        check_status(mc_smorph_backward(&d, input.data_ptr(), weight.data_ptr(), alphas.data_ptr(), output.data_ptr(), grad_output.data_ptr(),
                                        grad_input.data_ptr(), grad_weight.data_ptr(), grad_alpha_pairs.data_ptr(),
                                        workspace.defined() ? workspace.data_ptr() : nullptr, ws_bytes, at::cuda::getCurrentCUDAStream().stream()));

        // A single alpha shared by every pair receives the gradient of all of them (csrc/cpp/smorph.cpp:96-98).
        torch::Tensor grad_alpha =
            alpha.numel() == grad_alpha_pairs.numel() ? grad_alpha_pairs.view_as(alpha) : grad_alpha_pairs.sum().view_as(alpha);
        grad_input = output_to_original(grad_input, ctx->saved_data["input_dims"].toInt());
        if (ctx->saved_data["weight_dims"].toInt() == 2) grad_weight = grad_weight.squeeze(0).squeeze(0);
        return {grad_input, grad_weight, grad_alpha, torch::Tensor()};
    }
};

/// Smorph with the smooth channel merge, the autograd function of torch.ops.morphocore.smorph_scm
/// (reference: csrc/cpp/smorph_scm.cpp:13-96). beta holds one value per output channel.
class SmorphScmFunction : public torch::autograd::Function<SmorphScmFunction>
{
public:
    static torch::Tensor forward(torch::autograd::AutogradContext* ctx, torch::Tensor input, torch::Tensor weight, torch::Tensor alpha,
                                 torch::Tensor beta)
    {
        const int64_t original_dims = input.dim();
        torch::Tensor input4d = input_to_4d(input);
        torch::Tensor weight4d = weight_to_4d(weight);
        require_cuda(input, "input");
        require_cuda(weight, "weight");
        require_cuda(alpha, "alpha");
        require_cuda(beta, "beta");
        TORCH_CHECK(weight.device() == input.device() && alpha.device() == input.device() && beta.device() == input.device(),
                    "input, weight, alpha and beta must be on the same device (input on ", input.device(), ", weight on ", weight.device(),
                    ", alpha on ", alpha.device(), ", beta on ", beta.device(), ")");
        TORCH_CHECK(input.scalar_type() == weight.scalar_type() && input.scalar_type() == alpha.scalar_type()
                        && input.scalar_type() == beta.scalar_type(),
                    "input, weight, alpha and beta must have the same dtype");
        TORCH_CHECK(input4d.size(1) == weight4d.size(1), "Input channels must match weight input channels");
        TORCH_CHECK(beta.numel() == weight4d.size(0), "Beta must have shape [out_channels]");
        const c10::cuda::CUDAGuard device_guard(input.device());
        input4d = input4d.contiguous();
        weight4d = weight4d.contiguous();
        const torch::Tensor alphas = pair_alphas(alpha, MC_MERGE_SMOOTH, weight4d.size(0), input4d.size(1));
        const torch::Tensor betas = beta.contiguous();

        const mc_desc d = make_desc(input4d, weight4d, MC_OP_DILATION, MC_MERGE_SMOOTH);
        torch::Tensor output = torch::empty({input4d.size(0), weight4d.size(0), input4d.size(2), input4d.size(3)}, input4d.options());
        const TraceRange trace("morphocore::smorph_scm_forward");
        check_status(mc_smorph_scm_forward(&d, input4d.data_ptr(), weight4d.data_ptr(), alphas.data_ptr(), betas.data_ptr(), output.data_ptr(),
                                           at::cuda::getCurrentCUDAStream().stream()));
        // The backward pass reads the 4-D output: the final value of the soft merge.
        ctx->save_for_backward({output, alpha, betas, input4d, weight4d});
        ctx->saved_data["input_dims"] = original_dims;
        ctx->saved_data["weight_dims"] = weight.dim();
        return output_to_original(output, original_dims);
    }

    static torch::autograd::tensor_list backward(torch::autograd::AutogradContext* ctx, torch::autograd::tensor_list grad_outputs)
    {
        const auto saved = ctx->get_saved_variables();
        const torch::Tensor& output = saved[0];
        const torch::Tensor& alpha = saved[1];
        const torch::Tensor& beta = saved[2];
        const torch::Tensor& input = saved[3];
        const torch::Tensor& weight = saved[4];
        torch::Tensor grad_output = input_to_4d(grad_outputs[0]).contiguous();
        TORCH_CHECK(grad_output.sizes() == output.sizes(), "grad_output shape mismatch: expected [", output.sizes(), "] but got [",
                    grad_output.sizes(), "]");
        TORCH_CHECK(grad_output.scalar_type() == input.scalar_type(), "grad_output must have the same dtype as input");
        TORCH_CHECK(grad_output.device() == input.device(), "grad_output must be on the same device as input");

        const c10::cuda::CUDAGuard device_guard(input.device());
        const mc_desc d = make_desc(input, weight, MC_OP_DILATION, MC_MERGE_SMOOTH);
        const torch::Tensor alphas = pair_alphas(alpha, MC_MERGE_SMOOTH, weight.size(0), input.size(1));
        torch::Tensor grad_input = torch::empty_like(input);
        torch::Tensor grad_weight = torch::empty_like(weight);
        torch::Tensor grad_alpha_pairs = torch::empty_like(alphas);
        torch::Tensor grad_beta = torch::empty_like(beta);
        const size_t ws_bytes = mc_smorph_scm_backward_workspace_bytes(&d);
        torch::Tensor workspace = torch::empty({static_cast<int64_t>(ws_bytes)}, input.options().dtype(torch::kByte));
        const TraceRange trace("morphocore::smorph_scm_backward");
        check_status(mc_smorph_scm_backward(&d, input.data_ptr(), weight.data_ptr(), alphas.data_ptr(), beta.data_ptr(), output.data_ptr(),
                                            grad_output.data_ptr(), grad_input.data_ptr(), grad_weight.data_ptr(), grad_alpha_pairs.data_ptr(),
                                            grad_beta.data_ptr(), workspace.data_ptr(), ws_bytes, at::cuda::getCurrentCUDAStream().stream()));

        // A single alpha shared by every pair receives the gradient of all of them (csrc/cpp/smorph_scm.cpp:81-83).
        torch::Tensor grad_alpha =
            alpha.numel() == grad_alpha_pairs.numel() ? grad_alpha_pairs.view_as(alpha) : grad_alpha_pairs.sum().view_as(alpha);
        grad_input = output_to_original(grad_input, ctx->saved_data["input_dims"].toInt());
        if (ctx->saved_data["weight_dims"].toInt() == 2) grad_weight = grad_weight.squeeze(0).squeeze(0);
        return {grad_input, grad_weight, grad_alpha, grad_beta};
    }
};

int64_t checked_merge(int64_t merge)
{
    TORCH_CHECK(merge >= 0 && merge <= MC_MERGE_IDENTITY, "Unknown merge mode ", merge);
    TORCH_CHECK(merge != MC_MERGE_SMOOTH, "Unsupported merge operation");
    return merge;
}

int64_t checked_padding(int64_t padding)
{
    TORCH_CHECK(padding >= 0 && padding <= PAD_REPLICATE, "Unknown padding mode ", padding);
    return padding;
}

/// float16 / bfloat16 tensors: half precision is a STORAGE type here. The operators widen to float, run the float
/// kernels and narrow the result; they are composite operators, so autograd differentiates through the two casts
/// and the gradients come back in the input's type. The reference accepts float and double only ("TODO: Add float16
/// support", csrc/cpp/morpho_op.cpp:7). Every tensor argument must share the input's type.
bool is_reduced(const torch::Tensor& t) { return t.scalar_type() == torch::kHalf || t.scalar_type() == torch::kBFloat16; }

torch::Tensor widen(const torch::Tensor& t, const torch::Tensor& like, const char* what)
{
    TORCH_CHECK(t.scalar_type() == like.scalar_type(), what, " must have the input's dtype (", like.scalar_type(), "), got ", t.scalar_type());
    return t.to(torch::kFloat);
}

torch::Tensor dilation(torch::Tensor input, torch::Tensor weight, int64_t merge, int64_t padding, double padding_value, bool save_indices,
                       double noise_scale)
{
    if (is_reduced(input))
        return dilation(input.to(torch::kFloat), widen(weight, input, "weight"), merge, padding, padding_value, save_indices, noise_scale)
            .to(input.scalar_type());
    return MorphoFunction::apply(input, weight, static_cast<int64_t>(MC_OP_DILATION), checked_merge(merge), checked_padding(padding), padding_value,
                                 save_indices, noise_scale);
}

torch::Tensor erosion(torch::Tensor input, torch::Tensor weight, int64_t merge, int64_t padding, double padding_value, bool save_indices,
                      double noise_scale)
{
    if (is_reduced(input))
        return erosion(input.to(torch::kFloat), widen(weight, input, "weight"), merge, padding, padding_value, save_indices, noise_scale)
            .to(input.scalar_type());
    return MorphoFunction::apply(input, weight, static_cast<int64_t>(MC_OP_EROSION), checked_merge(merge), checked_padding(padding), padding_value,
                                 save_indices, noise_scale);
}

/// Extension (not an operator of the reference): both halves of sigma_layer at once. MAX / MIN merges that keep their
/// winner indices for the backward pass run the two separate operators, which is what saves them.
std::tuple<torch::Tensor, torch::Tensor> dilation_erosion(torch::Tensor input, torch::Tensor weight, int64_t merge, int64_t padding, double padding_value,
                                                          bool save_indices)
{
    if (is_reduced(input))
    {
        auto [d, e] = dilation_erosion(input.to(torch::kFloat), widen(weight, input, "weight"), merge, padding, padding_value, save_indices);
        return {d.to(input.scalar_type()), e.to(input.scalar_type())};
    }
    merge = checked_merge(merge);
    padding = checked_padding(padding);
    if (save_indices && (merge == MC_MERGE_MAX || merge == MC_MERGE_MIN))
        return {dilation(input, weight, merge, padding, padding_value, true, 0.0),
                erosion(input, weight.flip({-2, -1}), merge, padding, padding_value, true, 0.0)};
    const auto out = MorphoPairFunction::apply(input, weight, merge, padding, padding_value);
    return {out[0], out[1]};
}

torch::Tensor smorph(torch::Tensor input, torch::Tensor weight, torch::Tensor alpha, int64_t merge)
{
    TORCH_CHECK(merge >= 0 && merge <= MC_MERGE_IDENTITY && merge != MC_MERGE_SMOOTH, "Unsupported merge operation for smorph");
    if (is_reduced(input))
        return smorph(input.to(torch::kFloat), widen(weight, input, "weight"), widen(alpha, input, "alpha"), merge).to(input.scalar_type());
    return SmorphFunction::apply(input, weight, alpha, merge);
}

torch::Tensor smorph_scm(torch::Tensor input, torch::Tensor weight, torch::Tensor alpha, torch::Tensor beta)
{
    if (is_reduced(input))
        return smorph_scm(input.to(torch::kFloat), widen(weight, input, "weight"), widen(alpha, input, "alpha"), widen(beta, input, "beta"))
            .to(input.scalar_type());
    return SmorphScmFunction::apply(input, weight, alpha, beta);
}

}  // namespace

TORCH_LIBRARY(morphocore, m)
{
    m.def("dilation(Tensor input, Tensor weight, int merge, int padding, float padding_value=0., bool save_indices=True, "
          "float noise_scale=0.) -> Tensor");
    m.def("erosion(Tensor input, Tensor weight, int merge, int padding, float padding_value=0., bool save_indices=True, "
          "float noise_scale=0.) -> Tensor");
    m.def("smorph(Tensor input, Tensor weight, Tensor alpha, int merge) -> Tensor");
    m.def("smorph_scm(Tensor input, Tensor weight, Tensor alpha, Tensor beta) -> Tensor");
    m.def("dilation_erosion(Tensor input, Tensor weight, int merge, int padding, float padding_value=0., bool save_indices=True) -> (Tensor, Tensor)");
}

TORCH_LIBRARY_IMPL(morphocore, CompositeImplicitAutograd, m)
{
    m.impl("dilation", &dilation);
    m.impl("erosion", &erosion);
    m.impl("smorph", &smorph);
    m.impl("smorph_scm", &smorph_scm);
    m.impl("dilation_erosion", &dilation_erosion);
}

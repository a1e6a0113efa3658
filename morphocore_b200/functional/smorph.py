import torch

from ._ops import ops
from .merge_enum import str_to_merge


def smorph(x: torch.Tensor, w: torch.Tensor, alpha: torch.Tensor, beta: torch.Tensor = None,
           channel_merge_mode: str = "sum") -> torch.Tensor:
    """Smooth morphological operation: an alpha-softmax that tends to dilation as alpha -> +inf and to
    erosion as alpha -> -inf, on the GPU.

    Same signature and semantics as the reference `morphocore.functional.smorph`
    (morphocore/functional/smorph.py:6-75). The structuring element is first re-parametrised in PyTorch,

        w~(alpha) = tanh(alpha) * ( (1 - tanh alpha)/2 * flip(w) + (1 + tanh alpha)/2 * w ),

    then, per channel pair and over the taps that fall inside the image, with v_k = x_k + w~_k:
    out = sum_k softmax_k(alpha v_k) v_k, followed by the channel merge.

    x : (N, C_in, H, W); w : (C_out, C_in, K_h, K_w) ((C, 1, K_h, K_w) for 'identity').
    alpha : (C_out, C_in) ((C,) or (C, 1) for 'identity'), or a single value shared by every pair.
    beta : (C_out,), optional. When given, the channels are merged by a second soft extremum instead of
        `channel_merge_mode` (Smorph SCM, `torch.ops.morphocore.smorph_scm`): with c_i the soft extremum of channel
        i, out = sum_i softmax_i(beta c_i) c_i (reference: morphocore/functional/csrc/cpp/smorph_scm.cpp:13-56).
    channel_merge_mode : 'sum', 'max', 'min', 'mean' or 'identity'.
    """
    if channel_merge_mode == 'identity' or alpha.dim() == 1:
        tanh_alpha = torch.tanh(alpha).view(-1, 1, 1, 1)
    else:
        tanh_alpha = torch.tanh(alpha).unsqueeze(-1).unsqueeze(-1)

    term1 = (1 + tanh_alpha) / 2
    term2 = (1 - tanh_alpha) / 2
    w_tilde_alpha = tanh_alpha * (term2 * w.flip(dims=(-2, -1)) + term1 * w)

    if beta is not None:
        return ops.smorph_scm(x, w_tilde_alpha, alpha, beta)
    return ops.smorph(x, w_tilde_alpha, alpha, str_to_merge(channel_merge_mode))

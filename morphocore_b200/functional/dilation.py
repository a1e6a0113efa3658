import torch

from ._dropout import drop_weights
from ._ops import ops
from .merge_enum import str_to_merge, str_to_padding


def dilation(x: torch.Tensor, w: torch.Tensor, channel_merge_mode: str = 'sum',
             padding_mode: str = 'replicate', save_indices: bool = True,
             weight_dropout: float = 0.0, training: bool = False,
             padding_value: float = 0.0, noise_scale: float = 0.0) -> torch.Tensor:
    """Grey-scale dilation with a learnable structuring element, on the GPU.

    y[n, o, h, w] = merge_i max_{kh, kw} ( x[n, i, h + kH//2 - kh, w + kW//2 - kw] + w[o, i, kh, kw] )

    Same signature and semantics as the reference `morphocore.functional.dilation`
    (morphocore/functional/dilation.py:5-91).

    x : (N, C_in, H, W), (C_in, H, W) or (H, W), float32 or float64, CUDA.
    w : (C_out, C_in, K_h, K_w) ((C, 1, K_h, K_w) for 'identity') or (K_h, K_w).
    channel_merge_mode : 'sum', 'max', 'min', 'mean' or 'identity'.
    padding_mode : 'zero' (border reads 0), 'geodesic' (-inf, never wins), 'constant' (padding_value)
        or 'replicate' (nearest edge pixel).
    save_indices : keep the winning tap of 'max' / 'min' merges for the backward pass instead of
        recomputing it.
    weight_dropout, training : in training, drop weights (set to -inf) with this probability.
    noise_scale : in training, every batch element adds its own uniform noise in [-noise_scale, noise_scale]
        to the structuring element.
    """
    if training and weight_dropout > 0.0:
        w = drop_weights(w, weight_dropout)
    return ops.dilation(x, w, str_to_merge(channel_merge_mode), str_to_padding(padding_mode),
                        padding_value, save_indices, noise_scale if training else 0.0)

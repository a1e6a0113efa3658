import torch

from ._dropout import drop_weights
from ._ops import ops
from .merge_enum import str_to_merge, str_to_padding


def erosion(x: torch.Tensor, w: torch.Tensor, channel_merge_mode: str = 'sum',
            padding_mode: str = 'replicate', save_indices: bool = True,
            weight_dropout: float = 0.0, training: bool = False,
            padding_value: float = 0.0, noise_scale: float = 0.0) -> torch.Tensor:
    """Grey-scale erosion with a learnable structuring element, on the GPU.

    y[n, o, h, w] = merge_i min_{kh, kw} ( x[n, i, h + kH//2 - kh, w + kW//2 - kw] - wf[o, i, kh, kw] ),
    wf = w flipped along both kernel axes.

    Same signature and semantics as the reference `morphocore.functional.erosion`
    (morphocore/functional/erosion.py:5-91): the operator receives the flipped structuring element and
    autograd un-flips its gradient. 'geodesic' padding reads +inf. Dropped weights are -inf, so that
    x - (-inf) = +inf never wins the minimum. See `dilation` for the arguments.
    """
    if training and weight_dropout > 0.0:
        w = drop_weights(w, weight_dropout)
    return ops.erosion(x, w.flip((-2, -1)), str_to_merge(channel_merge_mode),
                       str_to_padding(padding_mode), padding_value, save_indices,
                       noise_scale if training else 0.0)

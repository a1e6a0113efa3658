"""Compositions of the dilation / erosion kernels, kept in Python like in the reference
(morphocore/functional/opening.py:96-101, closing.py:96-101, sigma_layer.py:73-83): same signatures."""
import torch

from ._ops import ops
from .dilation import dilation
from .erosion import erosion
from .merge_enum import str_to_merge, str_to_padding


def opening(x: torch.Tensor, w_erosion: torch.Tensor, w_dilation: torch.Tensor, channel_merge_mode: str = 'sum',
            padding_mode: str = 'replicate', save_indices: bool = True, padding_value: float = 0.0,
            weight_dropout: float = 0.0, training: bool = False, noise_scale: float = 0.0) -> torch.Tensor:
    """Erosion (merging channels with `channel_merge_mode`) followed by a per-channel ('identity') dilation."""
    eroded = erosion(x, w_erosion, channel_merge_mode, padding_mode, save_indices, weight_dropout=weight_dropout,
                     training=training, padding_value=padding_value, noise_scale=noise_scale)
    return dilation(eroded, w_dilation, 'identity', padding_mode, save_indices, weight_dropout=weight_dropout,
                    training=training, padding_value=padding_value, noise_scale=noise_scale)


def closing(x: torch.Tensor, w_dilation: torch.Tensor, w_erosion: torch.Tensor, channel_merge_mode: str = 'sum',
            padding_mode: str = 'replicate', save_indices: bool = True, padding_value: float = 0.0,
            weight_dropout: float = 0.0, training: bool = False, noise_scale: float = 0.0) -> torch.Tensor:
    """Dilation (merging channels with `channel_merge_mode`) followed by a per-channel ('identity') erosion."""
    dilated = dilation(x, w_dilation, channel_merge_mode, padding_mode, save_indices, weight_dropout=weight_dropout,
                       training=training, padding_value=padding_value, noise_scale=noise_scale)
    return erosion(dilated, w_erosion, 'identity', padding_mode, save_indices, weight_dropout=weight_dropout,
                   training=training, padding_value=padding_value, noise_scale=noise_scale)


def sigma_layer(x: torch.Tensor, w: torch.Tensor, alpha: torch.Tensor, channel_merge_mode: str = 'sum',
                padding_mode: str = 'replicate', save_indices: bool = True, padding_value: float = 0.0,
                weight_dropout: float = 0.0, training: bool = False, noise_scale: float = 0.0) -> torch.Tensor:
    """Y = sigmoid(mean_i alpha[o, i]) * dilation(x, w) + (1 - sigmoid(...)) * erosion(x, w)."""
    if not (training and (weight_dropout > 0.0 or noise_scale > 0.0)):
        # Both stages see the same structuring element: one operator computes the two (a single fused pass over x where the
        # kernel covers the case, the two separate passes otherwise; same values either way).
        out_dilation, out_erosion = ops.dilation_erosion(x, w, str_to_merge(channel_merge_mode), str_to_padding(padding_mode),
                                                         padding_value, save_indices)
    else:
        # Each stage draws its own dropout mask and noise (morphocore/functional/sigma_layer.py:73-78).
        kwargs = dict(channel_merge_mode=channel_merge_mode, padding_mode=padding_mode, save_indices=save_indices,
                      padding_value=padding_value, weight_dropout=weight_dropout, training=training, noise_scale=noise_scale)
        out_erosion = erosion(x, w, **kwargs)
        out_dilation = dilation(x, w, **kwargs)
    soft = torch.sigmoid(alpha.mean(dim=1)).view(1, -1, 1, 1)
    return out_erosion * (1.0 - soft) + out_dilation * soft

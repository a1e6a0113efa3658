"""Compositions of the dilation / erosion kernels, kept in Python like in the reference
(morphocore/functional/opening.py:96-101, closing.py:96-101, sigma_layer.py:73-83): same signatures."""
import torch

from .dilation import dilation
from .erosion import erosion


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
    kwargs = dict(channel_merge_mode=channel_merge_mode, padding_mode=padding_mode, save_indices=save_indices,
                  padding_value=padding_value, weight_dropout=weight_dropout, training=training, noise_scale=noise_scale)
    out_erosion = erosion(x, w, **kwargs)
    out_dilation = dilation(x, w, **kwargs)
    soft = torch.sigmoid(alpha.mean(dim=1)).view(1, -1, 1, 1)
    return out_erosion * (1.0 - soft) + out_dilation * soft

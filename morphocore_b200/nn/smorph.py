import torch
import torch.nn as nn

from morphocore_b200.functional import smorph
from .alpha_module import AlphaModule


class SMorph(AlphaModule):
    """Learnable smooth morphological layer whose `alpha` moves it between erosion (alpha -> -inf) and
    dilation (alpha -> +inf); same constructor as the reference `morphocore.nn.SMorph`
    (morphocore/nn/smorph.py:89-112). `init_beta` creates the `beta` parameter of the smooth channel
    merge with the reference's shape (out_channels, in_channels); the operator wants one beta per output
    channel (morphocore/functional/csrc/cpp/smorph_scm.cpp:31), so, as in the reference, the forward
    pass of such a module raises unless in_channels == 1. functional.smorph takes a (out_channels,) beta."""

    def __init__(self, in_channels: int, out_channels: int, kernel_size: tuple, channel_merge_mode: str = "sum",
                 init_alpha: float = 0.0, dtype: torch.dtype = torch.float32, init_beta: float = None):
        if type(kernel_size) is int:
            kernel_size = (kernel_size, kernel_size)
        super(SMorph, self).__init__(in_channels, out_channels, kernel_size, channel_merge_mode, init_alpha, dtype)
        if init_beta is not None:
            self.beta = nn.Parameter(torch.full((out_channels, in_channels), init_beta, dtype=dtype))
        else:
            self.beta = None

    def forward(self, x: torch.Tensor):
        return smorph(x=x, w=self.weight, alpha=self.alpha, beta=self.beta, channel_merge_mode=self.channel_merge_mode)

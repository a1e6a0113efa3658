from .dilation import dilation
from .erosion import erosion
from .compositions import opening, closing, sigma_layer
from .smorph import smorph

__all__ = ['dilation', 'erosion', 'opening', 'closing', 'sigma_layer', 'smorph']

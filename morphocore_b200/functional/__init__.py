from .dilation import dilation
from .erosion import erosion
from .smorph import smorph

__all__ = ['dilation', 'erosion', 'smorph']

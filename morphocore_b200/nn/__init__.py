from .dilation import Dilation
from .erosion import Erosion
from .smorph import SMorph

__all__ = ['Dilation', 'Erosion', 'SMorph']

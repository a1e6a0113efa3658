from .dilation import Dilation
from .erosion import Erosion
from .compositions import Opening, Closing, SigmaLayer
from .smorph import SMorph

__all__ = ['Dilation', 'Erosion', 'Opening', 'Closing', 'SigmaLayer', 'SMorph']

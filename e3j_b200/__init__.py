"""e3j_b200: B200-native fused equivariant message-passing convolution.

Public surface mirrors the pieces of e3j that sit on the convolution path:
``Convolution`` (e3j.core.Convolution), ``Harmonics`` (e3j.core.Harmonics),
``GraphCSR`` (e3j.data.GraphCSR), the ``convolution`` / ``convolution_bwd``
primitives (e3j.ops.convolution) and the ``Coef4D`` packing (e3j.ops.coef).
"""

from .coef import Coef, Coef4D
from .convolution import Convolution
from .graph import DUMMY_INDEX, GraphCSR
from .harmonics import Harmonics
from .ops import ConvGraph, CUDAConvolutionParams, convolution, convolution_bwd
from .spaces import O3Irrep, O3Space
from .tensor_product import TensorProduct

__all__ = [
    "Coef", "Coef4D", "Convolution", "ConvGraph", "CUDAConvolutionParams", "DUMMY_INDEX", "GraphCSR",
    "Harmonics", "O3Irrep", "O3Space", "TensorProduct", "convolution", "convolution_bwd",
]  # fmt: skip
__version__ = "0.1.0"

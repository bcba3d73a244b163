"""Convolution layers with the reference's class names (pccnn_lib/pc/layers of phermosilla/pccnn_lib)."""
from .IConvLayer import IConvLayer, IConvLayerFactory
from .MCConv import MCConv, MCConvFactory
from .PointConv import PointConv, PointConvFactory
from .KPConv import KPConv, KPConvFactory, prepare_kernel_points
from .KPConvN import KPConvN, KPConvNFactory
from .SPHConv import SPHConv, SPHConvFactory
from .PCCNN import PCCNN, PCCNNFactory

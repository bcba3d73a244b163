"""Convolution layers of the hot path (KPConv, MCConv) with the reference's class names."""
from .IConvLayer import IConvLayer, IConvLayerFactory
from .KPConv import KPConv, KPConvFactory, prepare_kernel_points
from .MCConv import MCConv, MCConvFactory

"""Geometry classes with the constructor signatures and attribute names of the reference's
pccnn_lib/pc package (phermosilla/pccnn_lib); they orchestrate the operators of the hot path."""
from .Pointcloud import Pointcloud
from .BoundingBox import BoundingBox
from .Grid import Grid
from .Neighborhood import GridNeighborhood, Neighborhood
from .PointPooling import PointPooling
from .layers import *  # noqa: F401,F403

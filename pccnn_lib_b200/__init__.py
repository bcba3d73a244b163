"""pccnn_lib_b200 -- sm_100a implementation of the point-convolution hot path of
phermosilla/pccnn_lib behind the reference's own operator and class interfaces.

``pccnn_lib_b200.ops`` has the functions of the reference's ``pccnn_lib_ops`` extension;
``pccnn_lib_b200.op_wrappers`` and ``pccnn_lib_b200.pc`` mirror ``pccnn_lib.op_wrappers`` and
``pccnn_lib.pc``.  ``install_as_reference_modules()`` registers them under the reference's module
names so that existing code keeps its imports.
"""
import sys

from . import ops  # loads libpccnn_b200.so; raises if it is missing
from . import op_wrappers, pc


def install_as_reference_modules():
    """Make ``import pccnn_lib_ops`` / ``import pccnn_lib`` resolve to this package."""
    sys.modules.setdefault("pccnn_lib_ops", ops)
    this = sys.modules[__name__]
    sys.modules.setdefault("pccnn_lib", this)
    sys.modules.setdefault("pccnn_lib.pc", pc)
    sys.modules.setdefault("pccnn_lib.op_wrappers", op_wrappers)
    return this

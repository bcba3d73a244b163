"""``kernel_pts_dict['<dims>_<points>']``: the KPConv kernel-point dispositions of the reference
(pccnn_lib/pc/layers/kernel_points/kernel_points.py of phermosilla/pccnn_lib: float64 [points, dims], row 0
the centre; 2, 3 and 4 dimensions with 8, 16, 32 and 64 points), loaded from kernel_points.npz next to this
file.  The .npz is written by oracle/make_kernel_points.py, which imports the reference's module, so a new
KPConv layer starts from the reference's kernel points and sigma."""
import os

import numpy as np

_data = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "kernel_points.npz"))
kernel_pts_dict = {k: _data[k] for k in _data.files}

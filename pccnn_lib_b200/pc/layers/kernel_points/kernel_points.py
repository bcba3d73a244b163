"""``kernel_pts_dict['<dims>_<points>']``: kernel-point dispositions (float64 [points, dims], row 0 the
centre), loaded from kernel_points.npz next to this file (see make_kernel_points.py)."""
import os

import numpy as np

_data = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "kernel_points.npz"))
kernel_pts_dict = {k: _data[k] for k in _data.files}

"""Point-cloud helpers the layers need (subset of the reference's pccnn_lib/py_utils/pc_utils.py)."""
import numpy as np


def rotate_pc_3d(p_random_state, p_pts, p_max_angle=2.0 * np.pi, p_axes=(0, 1, 2)):
    """Rotates a 3-D cloud by random angles about the selected axes; returns (points, matrix).

    Same contract and the same use of the random state as rotate_pc_3d of
    pccnn_lib/py_utils/pc_utils.py:77-125 of the reference: three uniform samples give the
    angles in [-max, max), the matrix is Rz @ Ry @ Rx and the points are multiplied from the left.
    """
    ax, ay, az = (p_random_state.random_sample((3)) - 0.5) * 2.0 * p_max_angle
    rot = np.eye(3)
    if 0 in p_axes:
        rot = np.array([[1.0, 0.0, 0.0], [0.0, np.cos(ax), -np.sin(ax)], [0.0, np.sin(ax), np.cos(ax)]])
    if 1 in p_axes:
        rot = np.array([[np.cos(ay), 0.0, np.sin(ay)], [0.0, 1.0, 0.0], [-np.sin(ay), 0.0, np.cos(ay)]]) @ rot
    if 2 in p_axes:
        rot = np.array([[np.cos(az), -np.sin(az), 0.0], [np.sin(az), np.cos(az), 0.0], [0.0, 0.0, 1.0]]) @ rot
    return np.dot(p_pts, rot), rot

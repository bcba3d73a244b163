from .pc_utils import rotate_pc_3d

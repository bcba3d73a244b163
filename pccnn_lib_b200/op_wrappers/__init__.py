"""autograd.Function wrappers with the names and argument orders of the reference's
pccnn_lib/op_wrappers package (phermosilla/pccnn_lib), for the operators on the hot path."""
from .build_grid_ds_funct import BuildGridDS
from .compute_keys import ComputeKeys
from .find_neighbors import FindNeighbors
from .compute_pdf import ComputePDF
from .poisson_disk_sampling import PoissonDiskSamlping
from .compute_kpconv import ComputeKPConv
from .compute_mcconv import ComputeMCConv

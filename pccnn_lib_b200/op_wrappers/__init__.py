"""autograd.Function wrappers with the names and argument orders of the reference's
pccnn_lib/op_wrappers package (phermosilla/pccnn_lib)."""
from .build_grid_ds_funct import BuildGridDS
from .compute_keys import ComputeKeys
from .find_neighbors import FindNeighbors
from .compute_pdf import ComputePDF
from .poisson_disk_sampling import PoissonDiskSamlping
from .compute_mcconv import ComputeMCConv, ComputeMCConvWeightVar
from .compute_pointconv import ComputePointConvBasis, ComputePointConv, ComputePointConvWeightVar
from .compute_kpconv import ComputeKPConv, ComputeKPConvWeightVar
from .compute_kpconvn import ComputeKPConvN, ComputeKPConvNWeightVar
from .compute_sphconv import ComputeSPHConv, ComputeSPHConvWeightVar
from .compute_pccnn import ComputePCCNN, ComputePCCNNWeightVar

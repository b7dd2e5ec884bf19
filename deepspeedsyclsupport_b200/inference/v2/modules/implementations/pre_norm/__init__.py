from .cuda_group_rms import DSGroupRMSNorm
from .cuda_pre_ln import DSPreLNCUDAModule
from .cuda_pre_rms import DSPreRMSCUDAModule
from .cuda_sandwich_rms import DSSandwichRMSNorm

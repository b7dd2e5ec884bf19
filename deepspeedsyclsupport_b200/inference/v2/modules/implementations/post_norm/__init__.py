from .cuda_post_ln import DSPostLNCUDAModule
from .cuda_post_sum_rms import DSPostSumRMSNorm

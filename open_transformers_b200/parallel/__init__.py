from .env import dist_info, init_distributed, set_determinism, set_seed, shutdown_distributed
from .parallel_dims import ParallelDims

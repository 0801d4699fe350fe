"""Data-parallel training: DistributedDataParallel and the gradient reducers."""
from .ddp import DistributedDataParallel, DDP  # noqa: F401
from .reducer import Reducer, reduce_master_gradients  # noqa: F401

"""Import path parity with the reference layout (python/orthon/distributed/ddp.py)."""
from ..parallel.ddp import DistributedDataParallel, DDP  # noqa: F401

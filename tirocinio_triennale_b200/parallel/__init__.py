from .comm import CompressedAllreduce  # noqa: F401
from .cpu_ring import cpu_compressed_allreduce, PeerTimeout  # noqa: F401
from .ddp_hook import CompressedHookState, compressed_allreduce_hook  # noqa: F401

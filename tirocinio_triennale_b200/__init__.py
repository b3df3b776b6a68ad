"""homcomp-b200: error-bounded lossy compression with a homomorphic add, and compressed
collectives, written for NVIDIA B200 (sm_100a).

``ops``       codec and homomorphic add (CPU oracle and the sm_100a kernels)
``parallel``  compressed allreduce over peer-mapped buffers, DDP communication hook
``models``    GPT-2-shaped model used by the data-parallel benchmark
``utils``     data generators, error metrics, result checker, timing helpers
"""
MODE_OUTLIER, MODE_PLAIN, MODE_VEC = 0, 1, 2
MODES = {"outlier": MODE_OUTLIER, "plain": MODE_PLAIN, "vec": MODE_VEC}
BLOCK = 32
CHUNK = 32768

from . import ops  # noqa: E402,F401

__all__ = ["ops", "MODE_OUTLIER", "MODE_PLAIN", "MODE_VEC", "MODES", "BLOCK", "CHUNK"]

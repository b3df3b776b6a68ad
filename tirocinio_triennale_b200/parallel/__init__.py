from .comm import CompressedAllreduce  # noqa: F401

from .cpu_codec import (  # noqa: F401
    cpu_compress, cpu_decompress, cpu_decode_quant, cpu_hom_add, cpu_hom_add_deltas, cpu_hom_add_streams,
    cpu_quant_pred, cpu_quantize, cpu_dequantize, cpu_ring_allreduce, cpu_stream_size, max_compressed_bytes,
    rate_bytes, chunk_elems,
)
from .codec import Codec  # noqa: F401
from . import stream_io  # noqa: F401

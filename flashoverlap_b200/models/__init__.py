from .rmsnorm import RMSNorm, ReorderRMSNorm  # noqa: F401
from .row_parallel import OverlapRowParallelLayer, RowParallelLayer  # noqa: F401
from .decoder_layer import DecoderConfig, TPDecoderLayer  # noqa: F401

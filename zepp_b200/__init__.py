"""B200 (sm_100a) build of Zepp's expert-parallel MoE layer.

Importing this package does not touch the GPU; the CUDA library (zepp_b200/lib/libzepp_b200.so) is
loaded on first use and its absence is an error: there is no CPU path.
"""
from . import config as _config
from . import layer as _layer

SHAPES = _config.SHAPES
ModelShape = _config.ModelShape
EPMoEConfig = _config.EPMoEConfig
tokens_per_rank = _config.tokens_per_rank
EPMoE = _layer.EPMoE
Marks = _layer.Marks
activation = _layer.activation
token_buckets = _layer.token_buckets

__all__ = ["SHAPES", "ModelShape", "EPMoEConfig", "tokens_per_rank", "EPMoE", "Marks", "activation", "token_buckets"]
__version__ = "0.1.0"

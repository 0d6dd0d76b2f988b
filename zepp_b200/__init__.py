"""zepp_b200: the expert-parallel MoE layer of Zepp, built for B200 (sm_100a)."""
__version__ = "0.1.0"

from .config import SHAPES, EPMoEConfig, ModelShape, tokens_per_rank  # noqa: F401
from .layer import EPMoE, Marks, activation  # noqa: F401

"""Public configuration of the layer.

The class, field and property names (and which argument errors are AssertionErrors) are those of the
reference's python/zepp/config.py:5-79, so a caller can switch packages without touching its code;
everything else in this module is this package's own.
"""
from dataclasses import dataclass

# rows of W1 per hidden ffn unit: the gated activation stores gate rows, then up rows
_W1_BLOCKS = {"gelu": 1, "swiglu": 2}
_STRATEGIES = ("overlap", "direct")
_BF16_BYTES = 2
_MIB = 1 << 20


def _require(ok, what=""):
    if not ok:
        raise AssertionError(what)


@dataclass(frozen=True)
class ModelShape:
    """One MoE layer: E experts, top-k routing, hidden size H, expert FFN size I, activation."""
    num_experts: int
    topk: int
    hidden: int
    ffn_hidden: int
    act: str = "gelu"

    def __post_init__(self):
        _require(self.act in _W1_BLOCKS, self.act)

    @property
    def ffn1(self) -> int:
        """Rows of one expert's first weight matrix: I for GELU, 2 I (gate | up) for SwiGLU."""
        return _W1_BLOCKS[self.act] * self.ffn_hidden

    @property
    def chunk_bytes(self) -> int:
        """Size of one token row in bf16."""
        return _BF16_BYTES * self.hidden


def tokens_per_rank(budget_mib: float, shape: ModelShape) -> int:
    """Tokens a rank sends under a pre-top-k budget of `budget_mib` MiB: budget / (row bytes * k) rounded to the
    nearest integer (Python's round), times k, and never fewer than k."""
    per_token_group = shape.chunk_bytes * shape.topk
    groups = round(budget_mib * _MIB / per_token_group)
    return shape.topk * max(1, groups)


def _shape_table():
    rows = (
        # key          E    k  H     I
        ("qwen3",      128, 8, 4096, 1536),
        ("k2",         384, 8, 7168, 2048),
        ("qwen3-30b",  128, 8, 2048, 768),     # not in the reference's table: the Qwen3-30B-A3B layer
    )
    return {key: ModelShape(num_experts=e, topk=k, hidden=h, ffn_hidden=i) for key, e, k, h, i in rows}


SHAPES = _shape_table()


@dataclass(frozen=True)
class EPMoEConfig:
    """Expert-parallel layout and policy of one layer.

    ranks / ranks_per_node   expert-parallel world and its (virtual) node size
    max_tokens_per_rank      tokens a rank brings to a step; sizes every buffer
    comm_strategy            "overlap": token movement fused into the GEMM kernels; "direct": separate copy kernels
    swap                     let hot experts change slots between steps
    router_c                 slack C of the capacity-constrained routing
    redundant_slots_per_rank spare expert slots per rank (replicas, swap targets)
    sm_margin, gpu_plan      accepted for compatibility; planning always runs on the GPU here
    """
    shape: ModelShape
    ranks: int
    ranks_per_node: int
    max_tokens_per_rank: int
    comm_strategy: str = "overlap"
    swap: bool = False
    router_c: float = 0.25
    redundant_slots_per_rank: int = 2
    sm_margin: int = 8
    gpu_plan: bool = True

    def __post_init__(self):
        _require(self.comm_strategy in _STRATEGIES, self.comm_strategy)
        _require(self.shape.num_experts % self.ranks == 0, "num_experts must divide by ranks")
        _require(self.ranks % self.ranks_per_node == 0)
        _require(0.0 <= self.router_c <= 1.0)
        _require(self.max_tokens_per_rank % self.shape.topk == 0)

    @property
    def nodes(self) -> int:
        return self.ranks // self.ranks_per_node

    @property
    def slots_per_rank(self) -> int:
        home = self.shape.num_experts // self.ranks
        return home + self.redundant_slots_per_rank

    @property
    def groups_per_rank(self) -> int:
        """GEMM groups of a rank: local group 0 is an always-empty pad group, groups 1.. are the slots."""
        return 1 + self.slots_per_rank

    @property
    def virtual_experts(self) -> int:
        return self.groups_per_rank * self.ranks

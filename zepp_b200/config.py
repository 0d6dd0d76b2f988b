"""Model shapes and the layer configuration: the public knobs of the layer, with the names and
meaning of the reference's python/zepp/config.py:5-79 so callers can switch packages unchanged."""
from dataclasses import dataclass


@dataclass(frozen=True)
class ModelShape:
    num_experts: int
    topk: int
    hidden: int
    ffn_hidden: int
    act: str = "gelu"          # "gelu": one up matrix; "swiglu": gate|up rows, silu(gate) * up

    def __post_init__(self):
        assert self.act in ("gelu", "swiglu"), self.act

    @property
    def ffn1(self) -> int:
        """Rows of one expert's first weight matrix (N of GEMM 1)."""
        return 2 * self.ffn_hidden if self.act == "swiglu" else self.ffn_hidden

    @property
    def chunk_bytes(self) -> int:
        """Bytes of one bf16 token row."""
        return 2 * self.hidden


def tokens_per_rank(budget_mib: float, shape: ModelShape) -> int:
    """Tokens per rank of a pre-top-k send budget in MiB, a positive multiple of top-k."""
    rows = round(budget_mib * (1 << 20) / (shape.chunk_bytes * shape.topk))
    return max(shape.topk, rows * shape.topk)


SHAPES = {
    "qwen3": ModelShape(num_experts=128, topk=8, hidden=4096, ffn_hidden=1536),
    "k2": ModelShape(num_experts=384, topk=8, hidden=7168, ffn_hidden=2048),
    # extra key (not in the reference's table): the Qwen3-30B-A3B layer shape
    "qwen3-30b": ModelShape(num_experts=128, topk=8, hidden=2048, ffn_hidden=768),
}


@dataclass(frozen=True)
class EPMoEConfig:
    shape: ModelShape
    ranks: int
    ranks_per_node: int
    max_tokens_per_rank: int
    comm_strategy: str = "overlap"    # "overlap": transfers fused into the GEMM kernels; "direct": unfused
    swap: bool = False
    router_c: float = 0.25
    redundant_slots_per_rank: int = 2
    sm_margin: int = 8
    gpu_plan: bool = True

    def __post_init__(self):
        assert self.comm_strategy in ("overlap", "direct"), self.comm_strategy
        assert self.shape.num_experts % self.ranks == 0, "num_experts must divide by ranks"
        assert self.ranks % self.ranks_per_node == 0
        assert 0.0 <= self.router_c <= 1.0
        assert self.max_tokens_per_rank % self.shape.topk == 0

    @property
    def nodes(self) -> int:
        return self.ranks // self.ranks_per_node

    @property
    def slots_per_rank(self) -> int:
        return self.shape.num_experts // self.ranks + self.redundant_slots_per_rank

    @property
    def groups_per_rank(self) -> int:
        """Slots plus the always-empty pad group at local index 0."""
        return self.slots_per_rank + 1

    @property
    def virtual_experts(self) -> int:
        return self.ranks * self.groups_per_rank

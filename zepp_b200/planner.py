"""Per-step routing products (names of the reference's python/zepp/planner.py:20-28)."""


class Plan:
    """One iteration's routing products; the tensors live in the layer's runtime buffers."""
    __slots__ = ("vce", "probs_all", "stable", "epoch")

    def __init__(self, vce, probs_all, stable=True, epoch=0):
        self.vce = vce              # [R*S, K] int32 virtual group ids (device)
        self.probs_all = probs_all  # [R*S, K] fp32 gate weights (device)
        self.stable = stable
        self.epoch = epoch

"""Per-step buffer demands and the capacity check (API of the reference's python/zepp/capacity.py).
The demands themselves are computed on the device by the metadata kernels; this module names
them, tells which capacity each must fit in, and grows capacities."""
from dataclasses import dataclass, fields
import math

from .routing import Capacities


@dataclass(frozen=True)
class Demands:
    recv_rows: int
    dispatch_recv: int
    dispatch_stage: int
    dispatch_relay: int
    combine_conv: int
    combine_wire: int
    pair_rows: int


_FIT = (("recv_rows", "recv_cap"), ("dispatch_recv", "dispatch_recv"), ("dispatch_stage", "dispatch_stage"),
        ("dispatch_relay", "dispatch_relay"), ("recv_rows", "combine_send"), ("combine_conv", "combine_conv"),
        ("combine_wire", "combine_wire"))
_FIT_DIRECT = (("recv_rows", "recv_cap"), ("pair_rows", "pair_cap"))


def violations(d: Demands, c: Capacities, direct: bool = False):
    """[(capacity field, demand, capacity)] of every buffer the step would overflow."""
    return [(cf, getattr(d, df), getattr(c, cf)) for df, cf in (_FIT_DIRECT if direct else _FIT)
            if getattr(d, df) > getattr(c, cf)]


def grow(c: Capacities, d: Demands, factor: float = 1.5, direct: bool = False) -> Capacities:
    new = {f.name: getattr(c, f.name) for f in fields(c)}
    for df, cf in (_FIT_DIRECT if direct else _FIT):
        new[cf] = max(new[cf], int(math.ceil(factor * getattr(d, df))))
    new["combine_send"] = max(new["combine_send"], new["recv_cap"])
    new["dispatch_recv"] = max(new["dispatch_recv"], new["recv_cap"])
    return Capacities(**new)


class CapacityExceeded(Exception):
    def __init__(self, viol, demands: Demands):
        super().__init__("capacity exceeded: " + ", ".join(f"{f} needs {n} > {h}" for f, n, h in viol))
        self.violations = viol
        self.demands = demands

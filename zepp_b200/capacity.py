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
    """Capacities that hold `d` with headroom: every checked buffer becomes at least ceil(factor * demand) and never
    shrinks; the two buffers that alias the receive rows follow recv_cap (growth rule of the reference,
    python/zepp/capacity.py:75-82)."""
    wanted = {}
    for demand_field, cap_field in (_FIT_DIRECT if direct else _FIT):
        need = math.ceil(factor * getattr(d, demand_field))
        wanted[cap_field] = max(wanted.get(cap_field, 0), need)
    values = {f.name: max(getattr(c, f.name), wanted.get(f.name, 0)) for f in fields(c)}
    for follower in ("combine_send", "dispatch_recv"):
        values[follower] = max(values[follower], values["recv_cap"])
    return Capacities(**values)


class CapacityExceeded(Exception):
    """A step's exact demands do not fit the buffers; `.violations` lists (capacity, needed, held) and `.demands`
    holds the step's Demands (what EPMoE.resize_capacities grows from)."""

    def __init__(self, viol, demands: Demands):
        self.violations = list(viol)
        self.demands = demands
        parts = [f"{name} needs {needed} > {held}" for name, needed, held in self.violations]
        super().__init__("capacity exceeded: " + ", ".join(parts))

"""SeCoPa: selective compression and partitioning planner.

For every gradient the planner compares the modelled cost of synchronising it
uncompressed with the cost of the compressed CaSync path, over every partition
count K = 1..N, and writes one plan row ``name,size,y|n,K``.

Cost terms are ``cost(x) = slope*x + intercept`` floored at ``floor`` (x in fp32
elements), or tables of measured points.  Two kinds of profile exist:

* ``reference_profile(N)``: the coefficients the HiPress authors fitted on their
  cluster (src/SeCoPa/SeCoPa.py:25-39 of mark14wu/hipress), available for
  N in {4, 8, 16}; with them this planner reproduces the reference plans exactly.
* measured profiles written by :mod:`hipress_b200.secopa.profiler` on the B200 box
  (encode/decode kernel time, fused ring/PS time, NCCL all-reduce time), valid for
  any N >= 1.

Formulas (src/SeCoPa/SeCoPa.py:45-103): PS uncompressed = gather + broadcast;
PS compressed = gather(r x/K) + broadcast(r x/K) + min(K+1,N) encodes(x/K) +
min(N-1+K, 2(N-1)) decodes(r x/K); ring uncompressed = 2(N-1) sends(x/K); ring
compressed = 2(N-1) sends(r x/K) + N encodes(x/K) + N decodes(r x/K); merges
cost (N-1)*merge(x/K).
"""
from __future__ import annotations

import json
from dataclasses import asdict, dataclass, field
from pathlib import Path
from typing import Iterable


@dataclass(frozen=True)
class LinearCost:
    slope: float = 0.0
    intercept: float = 0.0
    floor: float = 0.0

    @property
    def knee(self) -> float:
        """Size below which the floor applies."""
        if self.slope == 0:
            return 0.0
        return max(0.0, (self.floor - self.intercept) / self.slope)

    def __call__(self, x: float) -> float:
        if x < self.knee:
            return self.floor
        return self.slope * x + self.intercept


@dataclass(frozen=True)
class TableCost:
    """Measured (elements, milliseconds) points, interpolated linearly.  Below the
    first point the first time applies (launch latency); beyond the last one the
    last segment's slope continues.  End-to-end terms are not straight lines on an
    NVSwitch box (latency floor, then a knee where the kernel fills the GPU, then
    bandwidth), and a single least-squares line misplaces the crossover."""
    points: tuple = ()

    def __post_init__(self):
        pts = tuple(sorted((float(x), float(y)) for x, y in self.points))
        if not pts:
            raise ValueError("a cost table needs at least one point")
        object.__setattr__(self, "points", pts)

    def __call__(self, x: float) -> float:
        pts = self.points
        if x <= pts[0][0] or len(pts) == 1:
            return pts[0][1]
        for (x0, y0), (x1, y1) in zip(pts, pts[1:]):
            if x <= x1:
                return y0 + (y1 - y0) * (x - x0) / (x1 - x0)
        (x0, y0), (x1, y1) = pts[-2], pts[-1]
        return y1 + max(0.0, (y1 - y0) / (x1 - x0)) * (x - x1)


@dataclass
class CostProfile:
    """All cost terms for one cluster size."""
    nodes: int
    encode: LinearCost
    decode: LinearCost
    ring_send: LinearCost
    gather: LinearCost
    broadcast: LinearCost
    merge: LinearCost = field(default_factory=LinearCost)
    comp_ratio: float = 1.0 / 16
    # measured end-to-end terms (B200 profiles); when present they replace the
    # composition of primitives above
    fused_ring: LinearCost | TableCost | None = None
    fused_ps: LinearCost | TableCost | None = None
    allreduce: LinearCost | TableCost | None = None
    # gradients smaller than this stay uncompressed whatever the costs say: a
    # rank's chunk would be under one tile, and quantising tiny tensors (biases,
    # norms) buys no time at all
    min_compress_elems: int = 0
    # compress only when it is at least this fraction cheaper: keeps decisions in the
    # launch-latency region, where both fitted lines are flat and differ by noise,
    # on the plain path (0 reproduces the reference's strict comparison)
    margin: float = 0.0
    source: str = "reference"

    def to_json(self) -> str:
        return json.dumps(asdict(self), indent=1)

    @staticmethod
    def from_json(text: str) -> "CostProfile":
        d = json.loads(text)
        def lc(v):
            if v is None:
                return None
            return TableCost(tuple(map(tuple, v["points"]))) if "points" in v else LinearCost(**v)
        keys = ("encode", "decode", "ring_send", "gather", "broadcast", "merge", "fused_ring",
                "fused_ps", "allreduce")
        return CostProfile(**{k: (lc(v) if k in keys else v) for k, v in d.items()})


_REF_COMMON = dict(
    encode=LinearCost(1.4133e-8, 5.8938e-2, 0.05408),
    decode=LinearCost(6.2041e-9, 1.3956e-1, 0.07287),
    ring_send=LinearCost(8.5005e-7, 2.0337e-1, 0.09766),
)
_REF_PS = {
    4: (LinearCost(2.7156e-6, 4.1930e-1, 0.15573), LinearCost(2.7157e-6, 2.2156e-1, 0.14820)),
    8: (LinearCost(6.1167e-6, 8.0768e-1, 0.28778), LinearCost(6.1172e-6, 2.7285e-1, 0.29666)),
    16: (LinearCost(1.2937e-5, 1.4406, 0.59503), LinearCost(1.2915e-5, 4.5538e-1, 0.58353)),
}


def reference_profile(nodes: int) -> CostProfile:
    """The reference's fitted coefficients; only N in {4, 8, 16} were measured."""
    if nodes not in _REF_PS:
        raise ValueError("the reference coefficients exist only for 4, 8 or 16 nodes; "
                         "use a measured profile for other sizes")
    g, b = _REF_PS[nodes]
    return CostProfile(nodes=nodes, gather=g, broadcast=b, **_REF_COMMON)


def _argmin_first(costs):
    best = min(costs)
    return best, costs.index(best) + 1


class Planner:
    def __init__(self, profile: CostProfile):
        self.p = profile

    # -- cost of the uncompressed path, best K ----------------------------
    def uncompressed_cost(self, size: int, topology: str):
        p, N = self.p, self.p.nodes
        if p.allreduce is not None:
            return p.allreduce(size), 1
        costs = []
        for K in range(1, N + 1):
            part = size / K
            if topology == "PS":
                c = p.gather(part) + p.broadcast(part) + (N - 1) * p.merge(part)
            else:
                c = 2 * (N - 1) * p.ring_send(part) + (N - 1) * p.merge(part)
            costs.append(c)
        return _argmin_first(costs)

    # -- cost of the compressed path, best K ------------------------------
    def compressed_cost(self, size: int, topology: str):
        p, N = self.p, self.p.nodes
        fused = p.fused_ps if topology == "PS" else p.fused_ring
        if isinstance(fused, TableCost):
            return fused(size), 1  # measured whole: partitions do not change a persistent launch
        if fused is not None:
            # one persistent launch per bucket: partitions only shorten the
            # per-hop pipeline fill, modelled as the intercept shared by K parts
            costs = [fused.slope * size + fused.intercept * (1 + 0.05 * (K - 1))
                     if size >= fused.knee else fused.floor for K in range(1, N + 1)]
            return _argmin_first(costs)
        r = p.comp_ratio
        costs = []
        for K in range(1, N + 1):
            part, cpart = size / K, size * r / K
            if topology == "PS":
                c = (p.gather(cpart) + p.broadcast(cpart)
                     + min(K + 1, N) * p.encode(part)
                     + min(N - 1 + K, 2 * (N - 1)) * p.decode(cpart)
                     + (N - 1) * p.merge(part))
            else:
                c = (2 * (N - 1) * p.ring_send(cpart) + N * p.encode(part)
                     + N * p.decode(cpart) + (N - 1) * p.merge(part))
            costs.append(c)
        return _argmin_first(costs)

    def decide(self, size: int, topology: str):
        """-> ('y'|'n', K)"""
        topology = "PS" if topology.upper() == "PS" else "RING"
        orig, k_orig = self.uncompressed_cost(size, topology)
        if size < self.p.min_compress_elems:
            return "n", k_orig
        comp, k_comp = self.compressed_cost(size, topology)
        return ("y", k_comp) if orig * (1.0 - self.p.margin) > comp else ("n", k_orig)

    def plan(self, gradients: Iterable[tuple[str, int]], topology: str):
        return [(name, size, *self.decide(size, topology)) for name, size in gradients]

    # -- joint decision for a bucketed runtime ----------------------------
    def _set_cost(self, cost, total: float, bucket_elems: float) -> float:
        """Cost of `total` elements moved in launches of at most `bucket_elems`."""
        if total <= 0:
            return 0.0
        full, rest = divmod(total, bucket_elems)
        return full * cost(bucket_elems) + (cost(rest) if rest > 0 else 0.0)

    def plan_bucketed(self, gradients: Iterable[tuple[str, int]], topology: str,
                      bucket_bytes: int = 256 << 20, plain_bucket_bytes: int = 32 << 20):
        """Plan for a runtime that batches gradients into buckets (one fused launch
        per compressed bucket, one all-reduce per plain bucket), where the
        per-gradient comparison charges every gradient a launch latency it does not
        pay.  Needs measured end-to-end terms.  Picks the size threshold T that
        minimises  fused(sum of sizes >= T) + allreduce(sum of sizes < T), both
        split into buckets; T never falls below ``min_compress_elems`` and
        compressing must beat leaving everything plain by the profile's margin."""
        p = self.p
        topology = "PS" if topology.upper() == "PS" else "RING"
        fused = p.fused_ps if topology == "PS" else p.fused_ring
        if fused is None or p.allreduce is None:
            raise ValueError("plan_bucketed needs a profile with measured fused and all-reduce terms")
        grads = list(gradients)
        sizes = sorted({s for _, s in grads if s >= max(1, p.min_compress_elems)}, reverse=True)
        fb, pb = bucket_bytes / 4.0, plain_bucket_bytes / 4.0
        total = float(sum(s for _, s in grads))
        all_plain = self._set_cost(p.allreduce, total, pb)
        best_cost, best_t = all_plain, None
        comp = 0.0
        for t in sizes:                       # thresholds from the largest size down
            comp += float(sum(s for _, s in grads if s == t))
            c = self._set_cost(fused, comp, fb) + self._set_cost(p.allreduce, total - comp, pb)
            if c < best_cost and c < all_plain * (1.0 - p.margin):
                best_cost, best_t = c, t
        return [(name, size, "y" if best_t is not None and size >= best_t else "n", 1)
                for name, size in grads]


# ------------------------------------------------------------------ plan files
def read_gradient_list(path) -> list[tuple[str, int]]:
    rows = []
    for line in Path(path).read_text().splitlines():
        if not line.strip():
            continue
        f = line.split(",")
        rows.append((f[0], int(f[1])))
    return rows


def gradient_list_of(named_parameters) -> list[tuple[str, int]]:
    """(name, element count) rows of a model, the planner's input format."""
    return [(n, p.numel()) for n, p in named_parameters]


def write_gradient_list(path, rows):
    Path(path).write_text("".join(f"{n},{s}\n" for n, s in rows))


def format_plan(rows) -> str:
    return "".join(f"{n},{s},{c},{k}\n" for n, s, c, k in rows)


def read_plan(path) -> dict[str, tuple[int, bool, int]]:
    """name -> (size, compress?, partitions)"""
    out = {}
    for line in Path(path).read_text().splitlines():
        if not line.strip():
            continue
        name, size, c, k = line.split(",")[:4]
        out[name] = (int(size), c.strip() == "y", int(k))
    return out

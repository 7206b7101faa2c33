"""Algorithm table: the five HiPress compression algorithms and their parameters.

Names follow the reference's command line spellings ``onebit``, ``tbq``,
``terngrad``, ``dgc`` (README.md:160,162,180,276 of mark14wu/hipress) plus
``graddrop`` (README.md:9).  ``none`` means "do not compress".
"""
from __future__ import annotations

from dataclasses import dataclass, replace

ONEBIT, TBQ, TERNGRAD, DGC, GRADDROP = 1, 2, 3, 4, 5


@dataclass(frozen=True)
class AlgSpec:
    name: str
    alg: int                 # id in the wire header
    bits: int = 0            # bits per element (dense algorithms)
    sparse: bool = False
    error_feedback: bool = True
    threshold: float = 0.01  # tbq
    ratio: float = 0.001     # dgc / graddrop: fraction of elements sent
    momentum: float = 0.9    # dgc momentum correction
    seed: int = 0            # terngrad stochastic rounding

    @property
    def dense(self) -> bool:
        return not self.sparse

    def state_names(self):
        """Names of the per-tensor fp32 state arrays this algorithm keeps."""
        if self.alg == DGC:
            return ("momentum_u", "accum_v")
        if self.alg == GRADDROP:
            return ("residual",)
        if self.alg in (ONEBIT, TBQ) and self.error_feedback:
            return ("residual",)
        return ()


_TABLE = {
    "onebit": AlgSpec("onebit", ONEBIT, bits=1),
    "tbq": AlgSpec("tbq", TBQ, bits=2),
    "terngrad": AlgSpec("terngrad", TERNGRAD, bits=2, error_feedback=False),
    "dgc": AlgSpec("dgc", DGC, sparse=True),
    "graddrop": AlgSpec("graddrop", GRADDROP, sparse=True),
}
ALIASES = {"2bit": "tbq", "1bit": "onebit", "topk": "graddrop"}


def get_algorithm(name: str, **overrides) -> AlgSpec:
    """Look an algorithm up by its command-line name and apply parameter overrides
    (``threshold=``, ``bitwidth=``, ``ratio=``, ``momentum=``, ``seed=``)."""
    key = ALIASES.get(name.lower(), name.lower())
    if key not in _TABLE:
        raise ValueError(f"unknown compression algorithm {name!r}; choose from {sorted(_TABLE)}")
    spec = _TABLE[key]
    if "bitwidth" in overrides:
        bw = overrides.pop("bitwidth")
        if bw is not None:
            if spec.alg != TERNGRAD:
                if bw != spec.bits:
                    raise ValueError(f"{key} has a fixed width of {spec.bits} bits")
            elif bw not in (1, 2, 4, 8):
                raise ValueError("terngrad bitwidth must be 1, 2, 4 or 8")
            spec = replace(spec, bits=bw)
    overrides = {k: v for k, v in overrides.items() if v is not None}
    return replace(spec, **overrides) if overrides else spec


def algorithm_names():
    return sorted(_TABLE)

"""String <-> integer codes of the channel merge and padding modes. The integers are the ones the
operator schemas take, identical to the reference (morphocore/functional/merge_enum.py:4-69)."""
from enum import IntEnum


class MorphoMerge(IntEnum):
    MAX = 0
    MIN = 1
    ADD = 2
    AVERAGE = 3
    SMOOTH = 4
    IDENTITY = 5


class MorphoPadding(IntEnum):
    ZERO = 0
    GEODESIC = 1
    CONSTANT = 2
    REPLICATE = 3


_MERGE_MODES = {
    "max": MorphoMerge.MAX,
    "min": MorphoMerge.MIN,
    "sum": MorphoMerge.ADD,
    "mean": MorphoMerge.AVERAGE,
    "identity": MorphoMerge.IDENTITY,
}

_PADDING_MODES = {
    "zero": MorphoPadding.ZERO,
    "geodesic": MorphoPadding.GEODESIC,
    "constant": MorphoPadding.CONSTANT,
    "replicate": MorphoPadding.REPLICATE,
}


def str_to_merge(mode: str) -> MorphoMerge:
    """"max", "min", "sum", "mean" or "identity" -> MorphoMerge; anything else raises ValueError."""
    try:
        return _MERGE_MODES[mode]
    except (KeyError, TypeError):
        raise ValueError(f"Unknown merge mode: {mode}") from None


def str_to_padding(mode: str) -> MorphoPadding:
    """"zero", "geodesic", "constant" or "replicate" -> MorphoPadding; anything else raises ValueError."""
    try:
        return _PADDING_MODES[mode]
    except (KeyError, TypeError):
        raise ValueError(f"Unknown padding mode: {mode}. Expected one of {sorted(_PADDING_MODES)}.") from None

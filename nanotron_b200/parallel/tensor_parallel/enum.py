from enum import Enum, auto


class TensorParallelLinearMode(Enum):
    """ALL_REDUCE keeps activations replicated over tp; REDUCE_SCATTER shards them on dim 0 (sequence parallel)."""

    ALL_REDUCE = auto()
    REDUCE_SCATTER = auto()

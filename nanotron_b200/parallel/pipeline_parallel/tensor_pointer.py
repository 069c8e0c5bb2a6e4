from dataclasses import dataclass


@dataclass
class TensorPointer:
    """Placeholder for a tensor living on another pipeline rank: the tensor sits on ``group_rank`` of the pp group."""

    group_rank: int

"""Import-only stand-in for the ``grouped_gemm`` package, which the reference imports at module load for its MoE layer
(dense models never call it).  Calling any op raises."""
from types import SimpleNamespace


def _missing(*a, **k):
    raise RuntimeError("grouped_gemm is not installed: MoE layers of the reference cannot run here")


ops = SimpleNamespace(gmm=_missing, permute=_missing, unpermute=_missing)

from nanotron_b200.parallel.context import ParallelContext

__all__ = ["ParallelContext"]

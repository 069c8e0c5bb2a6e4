from nanotron_b200.parallel.data_parallel.utils import average_gradients, sync_gradients_across_dp  # noqa: F401

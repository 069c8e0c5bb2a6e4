from nanotron_b200.parallel.expert_parallel.utils import is_expert_parameter, sync_dense_and_expert_gradients  # noqa: F401

from nanotron_b200.optim.base import BaseOptimizer  # noqa: F401
from nanotron_b200.optim.inherit_from_other_optimizer import InheritFromOtherOptimizer  # noqa: F401
from nanotron_b200.optim.named_optimizer import NamedOptimizer  # noqa: F401
from nanotron_b200.optim.optimizer_from_gradient_accumulator import OptimizerFromGradientAccumulator  # noqa: F401
from nanotron_b200.optim.zero import ZeroDistributedOptimizer  # noqa: F401

from nanotron_b200.models.base import DTypeInvariantTensor, NanotronModel, build_model, check_model_has_grad, init_on_device_and_dtype  # noqa: F401

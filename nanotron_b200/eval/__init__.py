from nanotron_b200.eval.one_job_runner import LightEvalRunner  # noqa: F401

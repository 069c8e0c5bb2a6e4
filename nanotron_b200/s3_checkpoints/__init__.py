from nanotron_b200.s3_checkpoints.fsspec import check_path_is_local, fs_copy, fs_open  # noqa: F401
from nanotron_b200.s3_checkpoints.s3_mover import S3Mover  # noqa: F401

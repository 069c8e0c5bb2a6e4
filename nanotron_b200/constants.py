"""Names of files inside a checkpoint directory (layout parity: reference src/nanotron/constants.py)."""
from packaging.version import Version, parse

CHECKPOINT_VERSION = Version("1.5")
CHECKPOINT_FILE_NAME = "checkpoint_metadata.json"
MODEL_CONFIG_FILE_NAME = "model_config.json"
CONFIG_FILE_NAME = "config.yaml"
LATEST_FILE_NAME = "latest.txt"


def parse_version(v: str) -> Version:
    return parse(v)

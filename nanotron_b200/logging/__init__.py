from nanotron_b200.logging.base import *  # noqa: F401,F403
from nanotron_b200.logging.base import LogItem, LoggerWriter, get_logger, human_format, log_memory, log_rank, set_ranks_logging_level, warn_once, log_libraries_versions  # noqa: F401
from nanotron_b200.logging.logmixin import LoggingCollectorMixin, LogMixin  # noqa: F401
from nanotron_b200.logging.timers import TimerRecord, Timers, TimerType, nanotron_timer  # noqa: F401

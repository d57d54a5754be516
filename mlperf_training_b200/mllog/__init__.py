"""MLPerf event logging, log filtering and run-time reports."""
from .core import *  # noqa: F401,F403
from .core import MLLogger, ThroughputTimer, check_compliance, parse_log  # noqa: F401

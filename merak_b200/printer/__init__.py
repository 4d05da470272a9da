from .logging import AccMetric, LoggerFactory, Metric, log_dist, logger
from .see_memory import see_memory_usage
from .timer import SynchronizedWallClockTimer, ThroughputTimer, set_timer_log_rank

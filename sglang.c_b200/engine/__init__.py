from .api import (generate, sched_abort, sched_get_stats, sched_nactive, sched_new, sched_poll,
                  sched_step, sched_submit_ids)
from .engine import Engine, OutOfPages, StepError
from .runtime import Runtime
from .scheduler import Request, SchedStats, Scheduler
from .step import StepEntry

__all__ = ["Engine", "OutOfPages", "StepError", "Runtime", "StepEntry", "Scheduler", "Request",
           "SchedStats", "generate", "sched_new", "sched_submit_ids", "sched_step", "sched_poll",
           "sched_nactive", "sched_abort", "sched_get_stats"]

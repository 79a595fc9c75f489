from .generator import (Op, OpKind, ScheduleSpec, backward_order, batch_block, device_program, format_table,
                        forward_order, simulate)
from .validate import ScheduleError, check_programs, steady_state_period

__all__ = ["Op", "OpKind", "ScheduleSpec", "batch_block", "device_program", "forward_order", "backward_order",
           "simulate", "format_table", "ScheduleError", "check_programs", "steady_state_period"]

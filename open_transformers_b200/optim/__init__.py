from .schedules import LRSchedule, build_schedule, rewarm_factor, schedule_lr

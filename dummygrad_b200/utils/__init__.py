"""Auxiliary subsystems: profiler, metrics log, configuration, checkpointing, watchdog."""

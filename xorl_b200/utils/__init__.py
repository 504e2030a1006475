"""Utilities: logging, metrics, FLOP counting, timers, profiler factory, seeding."""

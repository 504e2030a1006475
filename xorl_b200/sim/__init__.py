"""Analytical step-time / memory planner (cf. src/xorl/sim/): hardware and calibration packs, a
per-configuration estimate, and a search over parallel layouts."""
from .planner import Estimate, HardwareSpec, ParallelLayout, enumerate_layouts, estimate, plan  # noqa: F401

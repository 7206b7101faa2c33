"""SeCoPa planner and on-box cost profiler."""
from .planner import (CostProfile, LinearCost, Planner, format_plan, read_gradient_list,  # noqa: F401
                      read_plan, reference_profile)

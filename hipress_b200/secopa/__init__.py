"""SeCoPa planner and on-box cost profiler."""
from .planner import (CostProfile, LinearCost, Planner, TableCost, format_plan, gradient_list_of,  # noqa: F401
                      read_gradient_list, read_plan, reference_profile, write_gradient_list)

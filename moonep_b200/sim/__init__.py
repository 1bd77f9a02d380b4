"""Single-process simulator of an R-rank expert-parallel group (CPU, no GPU needed)."""
from .planner import ClusterPlan, plan_cluster, solve_allocation, layout_tables, check_invariants, dup_table_from_arrays
from . import ops

__all__ = ["ClusterPlan", "plan_cluster", "solve_allocation", "layout_tables",
           "check_invariants", "dup_table_from_arrays", "ops"]

from .pipeline import compile_graph
from .plan import EventPlan, PassOptions, Plan, TaskInst, TILE_SYMBOLS, verify_plan

__all__ = ["compile_graph", "EventPlan", "PassOptions", "Plan", "TaskInst", "TILE_SYMBOLS", "verify_plan"]

"""Planner: passes over the primitive graph, per-equation kernel plans, buffer plan, staged / sharded compile."""
from .compile import CompileOptions, Program, compile_graph
from .edit import Decline, fold_region
from .refusal import Refusal

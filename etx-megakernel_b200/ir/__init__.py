from .dims import Dim, eval_dim, eval_expr, eval_shape, free_symbols
from .edgemap import EdgeMap
from .instantiate import Instance, instantiate
from .types import ETensor, Graph, InitKind, Resource, Scope, TaskGrid, Tensor, TileBody
from .verify import Issue, VerifyError, verify

__all__ = ["Dim", "eval_dim", "eval_expr", "eval_shape", "free_symbols", "EdgeMap", "Instance", "instantiate", "ETensor",
           "Graph", "InitKind", "Resource", "Scope", "TaskGrid", "Tensor", "TileBody", "Issue", "VerifyError", "verify"]

"""B200 transformer for nGraph-Python graphs.

`import ngraph_python_b200 as ng` gives the op-building surface of the reference's `ng`
namespace for the ops the hot path uses, and `ng.transformers` the transformer factory API.
"""
from .op_graph import *  # noqa: F401,F403
from .op_graph import (sum, max, min, make_axis, make_axes, Axes, Axis, Op,  # noqa: F401,A004
                       AssignableTensorOp)
from . import transformers  # noqa: F401
from .transformers import UnsupportedTransformerException  # noqa: F401

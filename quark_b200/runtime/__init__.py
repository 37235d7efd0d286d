from .stream import Event, Graph, active_stream, capture_graph, set_stream, synchronize  # noqa: F401
from .tensor import QuarkTensor  # noqa: F401

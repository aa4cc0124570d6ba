"""B200-native neighbour-graph construction behind the torch_cluster API.

``knn``, ``knn_graph``, ``radius``, ``radius_graph``, ``nearest`` and ``fps`` keep the reference's
signatures and run hand-written sm_100a CUDA kernels through ``torch.ops.torch_cluster.*``.
Importing the package loads the in-tree native libraries and raises if they are not built.
"""
from . import _native

_native.load_ops()

from .knn import knn, knn_graph  # noqa: E402
from .radius import radius, radius_graph  # noqa: E402
from .nearest import nearest  # noqa: E402
from .fps import fps  # noqa: E402
from .host import knn_graph_host  # noqa: E402
from .sharded import (knn_sharded, radius_sharded, knn_graph_sharded, radius_graph_sharded,  # noqa: E402
                      make_plan, ShardPlan)

__version__ = '0.1.0'

__all__ = ['knn', 'knn_graph', 'radius', 'radius_graph', 'nearest', 'fps', 'knn_graph_host', 'knn_sharded', 'radius_sharded',
           'knn_graph_sharded', 'radius_graph_sharded', 'make_plan', 'ShardPlan', '__version__']

"""Drop-in import name: ``import torch_cluster`` resolves to the B200-native neighbour-graph
functions.  Only the neighbour-graph path and its two neighbours exist here (knn, knn_graph, radius,
radius_graph, nearest, fps)."""
from pytorch_cluster_b200 import __version__, fps, knn, knn_graph, nearest, radius, radius_graph  # noqa: F401

__all__ = ['knn', 'knn_graph', 'radius', 'radius_graph', 'nearest', 'fps', '__version__']

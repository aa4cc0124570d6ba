"""Drop-in import name: ``import torch_cluster`` resolves to the B200-native neighbour-graph
functions.  Only the neighbour-graph path exists here (knn, knn_graph, radius, radius_graph)."""
from pytorch_cluster_b200 import __version__, knn, knn_graph, radius, radius_graph  # noqa: F401

__all__ = ['knn', 'knn_graph', 'radius', 'radius_graph', '__version__']

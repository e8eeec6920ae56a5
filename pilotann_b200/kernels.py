"""Thin op wrappers with the names and keyword order of upstream
``pilot_ann/kernels/__init__.py:62-124`` for the GPU search stage."""
from __future__ import annotations

from . import extension


def traverse_cuda(output_I, output_D, indptr, indices, mapping, storage, query,
                  initial_I, initial_D, n_neighbors: int):
    """``pilot_ann/kernels/__init__.py:62-75``"""
    extension.traverse_cuda(output_I, output_D, indptr, indices, mapping, storage, query,
                            initial_I, initial_D, n_neighbors)


def routing_cuda(query, route_vectors, entry_nodes, entry_vectors):
    """``pilot_ann/kernels/__init__.py:97-103``"""
    return extension.routing_cuda(query, route_vectors, entry_nodes, entry_vectors)


def pipeline(graph, subgraph, subgraph_cuda, storage, storage_cuda, query, query_cuda,
             initial_I, initial_D, n_neighbors: int, k: int, ef_search: int,
             d_principle: int, chunk_size: int):
    """``pilot_ann/kernels/__init__.py:106-124``: keyword order ``k, ef_search,
    d_principle`` here, positional order ``ef_search, d_principle, k`` below, as
    upstream.  The consumer of the candidates is chosen with
    :func:`pilotann_b200.set_refine` (default: this package's GPU refinement)."""
    return extension.pipeline(graph, subgraph, subgraph_cuda, storage, storage_cuda, query,
                              query_cuda, initial_I, initial_D, n_neighbors, ef_search,
                              d_principle, k, chunk_size)

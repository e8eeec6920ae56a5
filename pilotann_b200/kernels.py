"""Thin op wrappers with the names and keyword order of upstream
``pilot_ann/kernels/__init__.py:62-124`` for the GPU search stage."""
from __future__ import annotations

import torch

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
             d_principle: int, chunk_size: int, refine=None, n_streams: int = 2):
    """``pilot_ann/kernels/__init__.py:106-124`` / ``extension/pipeline_cpu.cpp:
    32-145``: chunked GPU traversal on side streams, asynchronous copy of the
    candidate handoff into pinned buffers, CPU refinement of chunk i-2 while
    chunk i-1 runs on the GPU.

    The CPU refinement is the consumer of this stage, not part of it:
    ``refine`` must be upstream's ``extension.traverse_refine`` (or anything
    with its signature, ``extension/entry.cpp:39-46``).
    """
    if refine is None:
        raise RuntimeError("pipeline: pass refine=<upstream extension.traverse_refine>; the "
                           "CPU refinement stage is not part of this package")
    if len(graph) != 2 or len(subgraph) != 2 or len(subgraph_cuda) != 3:
        raise RuntimeError("graph / subgraph / subgraph_cuda must hold 2 / 2 / 3 tensors")
    batch = query.size(0)
    if batch % chunk_size != 0:
        raise RuntimeError("Expected batch_size % chunk_size == 0 to be true, but got false.")
    dev = query_cuda.device
    topk_I = torch.empty(batch, k, dtype=torch.int64)
    topk_D = torch.empty(batch, k, dtype=torch.float32)
    streams = _side_streams(dev, n_streams)
    torch.cuda.current_stream(dev).synchronize()
    dev_I = [torch.empty(chunk_size, 4, ef_search, dtype=torch.int64, device=dev)
             for _ in range(n_streams)]
    dev_D = [torch.empty(chunk_size, 4, ef_search, dtype=torch.float32, device=dev)
             for _ in range(n_streams)]
    host_I = [torch.empty(chunk_size, 4 * ef_search, dtype=torch.int64, pin_memory=True)
              for _ in range(n_streams)]
    host_D = [torch.empty(chunk_size, 4 * ef_search, dtype=torch.float32, pin_memory=True)
              for _ in range(n_streams)]
    n_chunks = batch // chunk_size
    for i in range(n_chunks + n_streams):
        slot = i % n_streams
        if i >= n_streams:
            streams[slot].synchronize()
            lo = (i - n_streams) * chunk_size
            hi = lo + chunk_size
            refine(topk_I[lo:hi], topk_D[lo:hi], host_I[slot], host_D[slot], host_I[slot],
                   host_D[slot], subgraph, graph, storage, query[lo:hi], ef_search, d_principle)
        if i < n_chunks:
            lo, hi = i * chunk_size, (i + 1) * chunk_size
            with torch.cuda.stream(streams[slot]):
                extension.traverse_cuda(dev_I[slot], dev_D[slot], subgraph_cuda[0],
                                        subgraph_cuda[1], subgraph_cuda[2], storage_cuda,
                                        query_cuda[lo:hi], initial_I[lo:hi], initial_D[lo:hi],
                                        n_neighbors)
                host_I[slot].copy_(dev_I[slot].view(chunk_size, -1), non_blocking=True)
                host_D[slot].copy_(dev_D[slot].view(chunk_size, -1), non_blocking=True)
    return [topk_I, topk_D]


_STREAMS: dict = {}


def _side_streams(dev: torch.device, n: int):
    """Side streams are cached per device (upstream keeps one process-wide pool
    bound to the first device used, ``pipeline_cpu.cpp:67-73``)."""
    key = (dev.index if dev.index is not None else torch.cuda.current_device(), n)
    if key not in _STREAMS:
        _STREAMS[key] = [torch.cuda.Stream(device=dev) for _ in range(n)]
    return _STREAMS[key]

"""recall@k as upstream defines it (``pilot_ann/utils/recall.py:4-23``): mean over
queries of |predicted set  ∩ target set| / |target set|."""
from __future__ import annotations

import torch


def recall(predict: torch.Tensor, target: torch.Tensor) -> float:
    if not isinstance(predict, torch.Tensor) or not isinstance(target, torch.Tensor):
        raise RuntimeError
    if predict.size() != target.size():
        raise RuntimeError
    assert target.dim() == 2
    scores = []
    for y_hat, y in zip(predict.tolist(), target.tolist()):
        y, y_hat = set(y), set(y_hat)
        scores.append(len(y & y_hat) / len(y))
    return sum(scores) / len(scores)

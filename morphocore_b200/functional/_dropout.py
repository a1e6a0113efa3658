import torch


def drop_weights(w: torch.Tensor, weight_dropout: float) -> torch.Tensor:
    """Structuring-element dropout of the training path: each weight is dropped with probability
    `weight_dropout` and replaced by -inf, and every (out, in) slice keeps at least one weight
    (reference: morphocore/functional/dilation.py:79-87)."""
    keep = torch.rand_like(w) > weight_dropout
    flat = keep.view(w.shape[0] * w.shape[1], -1)
    empty = (~flat.any(dim=1)).nonzero().flatten().tolist()
    for row in empty:
        flat[row, torch.randint(0, flat.shape[1], (1,)).item()] = True
    return torch.where(keep, w, torch.tensor(-float("inf"), device=w.device, dtype=w.dtype))

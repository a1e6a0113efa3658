"""Loader for the reference's own compiled CPU operators (oracle/_ref/_C.so, built by build_ref.py).

TEST INFRASTRUCTURE ONLY. Loading the library registers torch.ops.morphocore with the reference's
implementation, so this module must run in a process that does not import morphocore_b200. The three
functions restate the reference's thin Python layer above the operators: enum ints
(morphocore/functional/merge_enum.py:4-19), the flipped structuring element of erosion
(morphocore/functional/erosion.py:89) and the tanh re-parametrisation of smorph
(morphocore/functional/smorph.py:56-75).
"""
import os

import torch

MERGES = {"max": 0, "min": 1, "sum": 2, "mean": 3, "identity": 5}
PADDINGS = {"zero": 0, "geodesic": 1, "constant": 2, "replicate": 3}
_loaded = False


def available():
    return os.path.exists(os.path.join(os.path.dirname(os.path.abspath(__file__)), "_ref", "_C.so"))


def load():
    global _loaded
    if not _loaded:
        torch.ops.load_library(os.path.join(os.path.dirname(os.path.abspath(__file__)), "_ref", "_C.so"))
        _loaded = True
    return torch.ops.morphocore


def dilation(x, w, merge="sum", padding="replicate", padding_value=0.0, save_indices=True):
    return load().dilation(x, w, MERGES[merge], PADDINGS[padding], padding_value, save_indices, 0.0)


def erosion(x, w, merge="sum", padding="replicate", padding_value=0.0, save_indices=True):
    return load().erosion(x, w.flip((-2, -1)), MERGES[merge], PADDINGS[padding], padding_value, save_indices, 0.0)


def smorph(x, w, alpha, merge="sum"):
    t = torch.tanh(alpha)
    t = t.view(-1, 1, 1, 1) if (merge == "identity" or alpha.dim() == 1) else t.unsqueeze(-1).unsqueeze(-1)
    w_tilde = t * ((1 - t) / 2 * w.flip(dims=(-2, -1)) + (1 + t) / 2 * w)
    return load().smorph(x, w_tilde, alpha, MERGES[merge])


def smorph_scm(x, w, alpha, beta):
    """Smooth channel merge: beta holds one value per output channel (morphocore/functional/smorph.py:72-73)."""
    t = torch.tanh(alpha)
    t = t.view(-1, 1, 1, 1) if alpha.dim() == 1 else t.unsqueeze(-1).unsqueeze(-1)
    w_tilde = t * ((1 - t) / 2 * w.flip(dims=(-2, -1)) + (1 + t) / 2 * w)
    return load().smorph_scm(x, w_tilde, alpha, beta)

"""Host-side score post-processing: the reductions the reference applies after the forward."""
from __future__ import annotations

import torch


def signal_rows_from_labels(labels: torch.Tensor, num_last: int = 16) -> torch.Tensor:
    """Slot indices (B, 2) of the two signal rows the reference scores with.

    src/blockrank/losses.py:41-48: inside the last ``num_last`` slots, b = first
    slot whose label is not -100 (the "[" token that starts the completion); the
    rows are (b-1, b).  Raises ValueError where the reference's assert fails.
    """
    S = labels.shape[-1]
    h1 = min(num_last, S)
    win = labels[:, S - h1:] > -100
    idx = win.int().argmax(-1)
    if not bool(win.any(-1).all()) or bool((idx < 1).any()):
        raise ValueError("signal token not found inside the last rows (or it is the first row of the window)")
    base = S - h1
    return torch.stack([base + idx - 1, base + idx], dim=-1).to(torch.int32)


def doc_logits_from_mass(mass: torch.Tensor, temperature: float = 0.05) -> torch.Tensor:
    """(B, N, R, num_docs) per-head/per-row document mass -> (B, num_docs) logits
    (mean over heads and rows, divided by the temperature; losses.py:68-74)."""
    return mass.mean(dim=(1, 2)) / temperature


def notebook_scores(mass: torch.Tensor) -> torch.Tensor:
    """The quickstart notebook's scorer (quickstart.ipynb, cell 9): last signal row only, softmax over the
    document columns, summed per document, mean over heads.  ``mass`` (B, N, R, num_docs) already holds
    that per-row, per-head document mass, so this is its last row averaged over heads -> (B, num_docs)."""
    return mass[:, :, -1, :].mean(dim=1)


def topk_documents(logits: torch.Tensor, k: int = 10) -> torch.Tensor:
    """scripts/eval_attn.py:150-151."""
    return torch.topk(logits, k=min(k, logits.shape[-1]), dim=-1).indices

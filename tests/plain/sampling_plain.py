"""Plain restatement of the sampler (wlejon/brolm src/detail/generate.cpp:68-142),
float64, one row at a time, with a sort as the reference does it.

Where the framework departs from the reference, this oracle follows the
framework and says so:

* the uniform number comes from the framework's counter-based generator
  (passed in as ``u``), not from std::mt19937_64 (generate.cpp:134-135);
* the draw walks the kept tokens in token-id order, not in descending order
  of probability (generate.cpp:136-141); the distribution is the same;
* tokens whose probability ties with the last kept one are all kept.
"""
from __future__ import annotations

import torch


def greedy(logits: torch.Tensor) -> int:
    """First maximum (generate.cpp:38-48)."""
    return int(torch.argmax(logits))


def kept_set(logits: torch.Tensor, temperature: float, top_k: int, top_p: float):
    """(probabilities, boolean mask of the kept tokens)  (generate.cpp:78-122)."""
    z = logits.double() / temperature
    probs = torch.softmax(z, dim=0)
    order = torch.argsort(probs, descending=True, stable=True)
    keep = probs.numel()
    if top_k > 0 and top_k < keep:
        keep = top_k                                            # generate.cpp:106-109
    if top_p < 1.0:
        cum = torch.cumsum(probs[order[:keep]], dim=0)          # generate.cpp:111-122
        reached = torch.nonzero(cum >= top_p)
        nucleus = int(reached[0]) + 1 if reached.numel() else keep
        keep = max(nucleus, 1)
    threshold = probs[order[keep - 1]]
    return probs, probs >= threshold                            # ties with the last kept one stay


def sample(logits: torch.Tensor, temperature: float, top_k: int, top_p: float, u: float) -> int:
    if temperature <= 0.0 or top_k == 1:                        # generate.cpp:73-76
        return greedy(logits)
    probs, mask = kept_set(logits, temperature, top_k, top_p)
    kept = torch.where(mask, probs, torch.zeros_like(probs))
    r = u * float(kept.sum())                                   # generate.cpp:124-135
    acc = torch.cumsum(kept, dim=0)
    hit = torch.nonzero((acc > r) & mask)
    return int(hit[0]) if hit.numel() else int(torch.nonzero(mask)[-1])

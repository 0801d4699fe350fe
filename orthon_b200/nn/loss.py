"""Loss modules (reference project: python/orthon/nn/loss.py)."""
from .. import _C
from .module import Module


class NLLLoss(Module):
    def __init__(self, reduction="mean"):
        super().__init__()
        if reduction not in ("none", "mean", "sum"):
            raise ValueError("reduction must be 'none', 'mean' or 'sum'")
        self.reduction = reduction

    def forward(self, log_probs, targets):
        return _C.nll_loss(log_probs, targets, self.reduction)


class CrossEntropyLoss(Module):
    """Mean softmax cross-entropy over [N, C] logits; targets may be a device int tensor."""

    def forward(self, logits, targets):
        return _C.cross_entropy(logits, targets)

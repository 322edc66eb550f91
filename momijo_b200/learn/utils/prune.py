"""Magnitude pruning (legacy/src/momijo/learn/utils/prune.mojo:21-141)."""
import torch


def tensor_sparsity(t: torch.Tensor) -> float:
    return float((t == 0).float().mean()) if t.numel() else 0.0


class PruneState:
    def __init__(self):
        self.masks = {}

    @torch.no_grad()
    def l1_unstructured(self, layer, amount: float, name: str = "weight"):
        """Zero the ``amount`` fraction of smallest-magnitude entries and remember the mask."""
        w = getattr(layer, name)
        k = int(round(amount * w.numel()))
        mask = torch.ones_like(w, dtype=torch.bool)
        if k > 0:
            thr = w.abs().reshape(-1).float().kthvalue(k).values
            mask = w.abs().float() > thr
        w.mul_(mask.to(w.dtype))
        self.masks[(id(layer), name)] = mask
        return mask

    @torch.no_grad()
    def reapply(self, layer, name: str = "weight"):
        m = self.masks.get((id(layer), name))
        if m is not None:
            getattr(layer, name).mul_(m.to(getattr(layer, name).dtype))

    def remove(self, layer, name: str = "weight"):
        return self.masks.pop((id(layer), name), None) is not None

"""Module swap: replace the ``nn.Linear`` layers of a model by ``OrthoLinear``.

The reference never swaps modules: its model-level experiments keep ``nn.Linear`` and rewrite the dense
weight as ``w_base + alpha * w_ortho`` whenever alpha changes
(``experiments/complete_real_model_experiments.py:269-327``), so the operator is never reached from a
model.  This utility does the swap for real: every selected ``nn.Linear`` is split into base and ortho
parts by ``split_fn``, packed with ``OrthoLinear.load_from_weights`` (on the GPU when the weights are
there) and replaced in its parent; the bias moves over as an FP32 parameter and is added inside the
kernel.  ``set_alpha_all`` then flips the kill switch of every swapped layer without touching weights.
"""
from __future__ import annotations

from typing import Callable, Dict, Optional, Tuple

import torch
import torch.nn as nn

from .ortho_linear import OrthoLinear

SplitFn = Callable[[str, torch.Tensor], Tuple[torch.Tensor, torch.Tensor]]


def base_only_split(name: str, weight: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """Everything goes to the INT4 base; the ortho part stays empty."""
    return weight, torch.zeros_like(weight)


def sieve_split(h_inv_diag: Dict[str, torch.Tensor], curvature_thresh: float = 10.0,
                sparsity_target: Optional[float] = None) -> SplitFn:
    """Split by the Hessian sieve with one inverse-Hessian diagonal per layer name."""
    from .sieve import hessian_sieve

    def split(name: str, weight: torch.Tensor):
        return hessian_sieve(weight, h_inv_diag[name].to(weight.device), curvature_thresh, sparsity_target)
    return split


def swap_linear(model: nn.Module, split_fn: SplitFn = base_only_split,
                filter_fn: Optional[Callable[[str, nn.Linear], bool]] = None,
                alpha: float = 1.0) -> Dict[str, OrthoLinear]:
    """Replaces, in place, every ``nn.Linear`` of ``model`` for which ``filter_fn(name, module)`` is true
    (default: all, except low-rank adapter matrices named ``lora_A`` / ``lora_B`` as the reference skips
    them) by an ``OrthoLinear`` holding ``split_fn(name, weight_fp32)``.  Returns the new modules by name."""
    swapped: Dict[str, OrthoLinear] = {}
    targets = []
    for name, mod in model.named_modules():
        if not isinstance(mod, nn.Linear) or "lora_A" in name or "lora_B" in name:
            continue
        if filter_fn is not None and not filter_fn(name, mod):
            continue
        targets.append((name, mod))
    for name, lin in targets:
        w = lin.weight.detach().to(torch.float32)
        w_base, w_ortho = split_fn(name, w)
        ol = OrthoLinear(lin.in_features, lin.out_features, bias=lin.bias is not None, device=w.device)
        ol.load_from_weights(w_base, w_ortho)
        if lin.bias is not None:
            ol.bias.data = lin.bias.detach().to(device=w.device, dtype=torch.float32).contiguous()
        ol.set_alpha(alpha)
        parent = model
        parts = name.split(".")
        for p in parts[:-1]:
            parent = getattr(parent, p)
        if name == "":
            raise ValueError("the model itself is an nn.Linear: wrap it in a container to swap it")
        setattr(parent, parts[-1], ol)
        swapped[name] = ol
    return swapped


def set_alpha_all(model: nn.Module, alpha: float) -> int:
    """Sets the kill switch of every ``OrthoLinear`` in ``model``; returns how many there are."""
    n = 0
    for mod in model.modules():
        if isinstance(mod, OrthoLinear):
            mod.set_alpha(alpha)
            n += 1
    return n

"""Recursive get/set of attention processors on a diffusers-style module tree
(mirrors dfsattn/attn_processor.py:6-62; used to install the Wan processors)."""
from typing import Dict, Union

import torch


def get_attn_processors(module: torch.nn.Module) -> Dict[str, object]:
    found: Dict[str, object] = {}

    def visit(name: str, mod: torch.nn.Module):
        if hasattr(mod, "get_processor"):
            found[f"{name}.processor"] = mod.get_processor()
        for child_name, child in mod.named_children():
            visit(f"{name}.{child_name}", child)

    for name, child in module.named_children():
        visit(name, child)
    return found


def set_attn_processor(module: torch.nn.Module, processor: Union[object, Dict[str, object]]) -> None:
    count = len(get_attn_processors(module))
    if isinstance(processor, dict) and len(processor) != count:
        raise ValueError(f"A dict of processors was passed, but the number of processors {len(processor)} "
                         f"does not match the number of attention layers: {count}. "
                         f"Please make sure to pass {count} processor classes.")

    def visit(name: str, mod: torch.nn.Module):
        if hasattr(mod, "set_processor"):
            mod.set_processor(processor if not isinstance(processor, dict) else processor.pop(f"{name}.processor"))
        for child_name, child in mod.named_children():
            visit(f"{name}.{child_name}", child)

    for name, child in module.named_children():
        visit(name, child)

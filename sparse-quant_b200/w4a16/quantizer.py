"""Module-tree walk that swaps nn.Linear for WALinear (the only part of the reference's
quantizer classes that is on the W4A16 path: test/nvidia/quantizer/opt_quantizer.py:27-51)."""
import torch
from torch import nn

from .qlinear import WALinear


def quantize_model(model: nn.Module, w_bit: int = 4, group_size: int = 128, quant_ignore=("lm_head",)):
    """Replace every nn.Linear whose qualified name contains none of `quant_ignore` by
    WALinear.from_float (weights must be fp16 on a CUDA device).  Returns the model."""
    w_config = {"n_bit": w_bit, "group_size": group_size}
    for name, module in list(model.named_modules()):
        if isinstance(module, nn.Linear) and all(ig not in name for ig in quant_ignore):
            parent_name, _, child = name.rpartition(".")
            parent = model.get_submodule(parent_name) if parent_name else model
            setattr(parent, child, WALinear.from_float(module, w_config))
    torch.cuda.empty_cache()
    return model

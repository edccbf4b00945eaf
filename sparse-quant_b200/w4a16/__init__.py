"""Host side of the B200 W4A16 linear layer: the reference's module-level interface
(`WALinear`, `quant_lmdeploy`, the quantizer's replace loop) re-stated on top of the `quant`
C-ABI package, plus tensor-parallel sharding of the packed tensors."""
from .qlinear import WALinear
from .quant_dequant import quant_lmdeploy, generate_quant, quantize_tensor, write_4bit_tensor
from .quantizer import quantize_model

__all__ = ["WALinear", "quant_lmdeploy", "generate_quant", "quantize_tensor", "write_4bit_tensor", "quantize_model"]

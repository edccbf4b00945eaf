"""WALinear — the W4A16 linear module (plugin boundary, Python side).

Same constructor arguments, buffers and state-dict keys as the reference's WALinear
(test/nvidia/module/qlinear/qlinear.py:10-99): `weight` int32 [K, N*w_bit/32] in tile order,
`zeros_scales` fp16 [K/g, 2N], `bias` fp16 [1, N] or None — so a state dict saved by the
reference loads here and vice versa.  forward() differs only in that the bias add is fused
into the kernel epilogue (one launch instead of two) and the launch goes to the current stream.
"""
import torch
from torch import nn

from quant import gemm_awq_bias

from .quant_dequant import quant_lmdeploy


class WALinear(nn.Module):
    def __init__(self, in_features, out_features, w_config=None, a_config=None, w_bit=4, a_bit=16,
                 group_size=128, bias=True, quantize_output=False, dev="cuda", dtype=torch.int):
        super().__init__()
        if w_bit != 4:
            raise NotImplementedError("WALinear: only w_bit=4 (the W4A16 path) is built")
        self.in_features = in_features
        self.out_features = out_features
        self.w_config = w_config
        self.a_config = a_config
        self.w_bit = w_bit
        self.a_bit = a_bit
        self.group_size = group_size
        # True: the packed buffers are not being (re)written by work still in flight on the stream that runs
        # forward(), so the decode kernel may prefetch them while the previous kernel drains.  from_float()
        # leaves it False until the first synchronisation point; model builders switch it on after loading.
        self.static_weights = False
        self.register_buffer("zeros_scales", torch.zeros(in_features // group_size, out_features * 2,
                                                          dtype=torch.float16, device=dev))
        self.register_buffer("weight", torch.zeros(in_features, out_features * w_bit // 32, dtype=dtype, device=dev))
        if bias:
            self.register_buffer("bias", torch.zeros((1, out_features), dtype=torch.float16, device=dev))
        else:
            self.register_buffer("bias", None)

    @torch.no_grad()
    def forward(self, x, relu: bool = False, residual=None, silu_mul: bool = False, pre_norm=None, stats_out=None):
        """x fp16 [..., K] -> fp16 [..., N].  The reference requires 3-D input (gemm_quant.cu:73);
        2-D and >3-D inputs are viewed as [1, tokens, K] here.  Epilogues fused into the kernel: relu=True (the
        ReLU after OPT's fc1), residual (fp16 [..., N], added to the output), silu_mul=True (a fuse_gate_up linear
        at up to 32 tokens: returns silu(gate) * up, [..., N / 2]), pre_norm = (weight, bias or None, eps, rms, stats):
        x is the un-normalised input and the LayerNorm / RMSNorm in front of the linear runs inside the decode kernel,
        from the row statistics `stats` that the linear producing x left with stats_out=stats (up to 16 tokens; as its
        own launch otherwise, or when stats is None)."""
        shape = x.shape
        x3 = x if x.dim() == 3 else x.reshape(1, -1, shape[-1])
        if not x3.is_contiguous():
            x3 = x3.contiguous()
        extra = {}
        if relu:
            extra["relu"] = True
        if silu_mul:
            extra["silu_mul"] = True
        if residual is not None:
            extra["residual"] = residual if residual.is_contiguous() else residual.contiguous()
        if pre_norm is not None:
            extra["pre_norm"] = pre_norm
        if stats_out is not None:
            extra["stats_out"] = stats_out
        y = gemm_awq_bias(x3, self.weight, self.zeros_scales, self.bias, self.out_features, self.group_size,
                          static_weights=self.static_weights, **extra)
        n_out = self.out_features // 2 if silu_mul else self.out_features
        return y if x.dim() == 3 else y.reshape(*shape[:-1], n_out)

    @staticmethod
    def from_float(module, w_config, a_config=None, quantize_output=False):
        """nn.Linear (fp16, CUDA) -> WALinear; w_config = {"n_bit": 4, "group_size": g} (reference :74-89)."""
        assert isinstance(module, nn.Linear)
        new = WALinear(module.in_features, module.out_features, w_config, a_config, w_bit=w_config["n_bit"],
                       group_size=w_config["group_size"], bias=module.bias is not None,
                       quantize_output=quantize_output, dev=module.weight.device, dtype=torch.int)
        new.weight, new.zeros_scales, _ = quant_lmdeploy(module.weight.data, module.in_features, module.out_features,
                                                         group_size=w_config["group_size"], n_bit=w_config["n_bit"])
        if module.bias is not None:
            new.bias = module.bias.data.to(torch.float16).unsqueeze(0).contiguous()
        return new

    def __repr__(self):
        return "W{}A{}Linear({}, {})".format(self.w_bit, self.a_bit, self.in_features, self.out_features)

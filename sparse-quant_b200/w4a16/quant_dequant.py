"""Quantise-and-pack flow (offline, once per linear).

Mirrors test/nvidia/utils/quant_dequant_nvidia.py of the reference: same function names,
arguments and return values, so `WALinear.from_float` reads the same.  `quant_lmdeploy` runs the
whole flow as ONE sm_100a kernel (quant.quantize_pack: min/max, scale, zero point, codes and the
final tile order in a single pass over the weight); `quantize_tensor` / `generate_quant` keep the
reference's torch fp16 statements for callers that want the intermediate tensors, and
`quant_lmdeploy(..., fused=False)` runs the reference's own step sequence (torch quantizer + the
three layout kernels) - the two routes are bit-identical (tests/test_gpu_pack.py).
"""
import torch

from quant import transpose_merge_zeros_scales, convert_ours_to_awq, convert_awq_to_lmdeploy, quantize_pack


def quantize_tensor(w, n_bit, q_group_size):
    """Asymmetric min-max quantisation per group of `q_group_size` along the last dim, all in
    the dtype of `w` (fp16).  Reference: quant_dequant_nvidia.py:124-148.
    Returns (q, scales [N, K/g], zeros [N, K/g], w_dequantised)."""
    org_shape = w.shape
    if q_group_size > 0:
        assert org_shape[-1] % q_group_size == 0
        w = w.reshape(-1, q_group_size)
    assert w.dim() == 2
    max_val = w.amax(dim=1, keepdim=True)
    min_val = w.amin(dim=1, keepdim=True)
    max_int = 2 ** n_bit - 1
    scales = (max_val - min_val).clamp(min=1e-5) / max_int
    zeros = (-torch.round(min_val / scales)).clamp_(0, max_int)
    q = torch.clamp(torch.round(w / scales) + zeros, 0, max_int)
    w_deq = ((q - zeros) * scales).reshape(org_shape)
    return (q.reshape(org_shape), scales.reshape(org_shape[0], -1).contiguous(),
            zeros.reshape(org_shape[0], -1).contiguous(), w_deq)


def write_4bit_tensor(w_q):
    """[N, K] integers in 0..15 -> uint8 [N, K/2], high nibble = even k (reference :79-88)."""
    shape = w_q.shape
    pairs = w_q.type(torch.uint8).reshape(-1, 2)
    packed = (pairs[:, 0] << 4) + pairs[:, 1]
    return packed.reshape(shape[:-1] + (shape[-1] // 2,))


def generate_quant(weight_fp16, input_features, n_bit, group_size):
    """-> (qweight uint8 [N, K/2], zeros fp16 [N, K/g], scales fp16 [N, K/g], w_fp16 [N, K])
    (reference :103-122)."""
    if n_bit != 4:
        raise NotImplementedError("only n_bit=4 is packed by this build (the reference's 2-bit storage "
                                  "trick, quant_dequant_nvidia.py:34-54, is not part of the W4A16 path)")
    q, scales, zeros, w_fp16 = quantize_tensor(weight_fp16, n_bit, group_size)
    return write_4bit_tensor(q).contiguous(), zeros.half().contiguous(), scales.half().contiguous(), w_fp16


def quant_lmdeploy(weight, input_features, output_features, group_size, n_bit=4, fused=True):
    """fp16 weight [N, K] on a CUDA device -> (weight int32 [K, N/8] tile-ordered,
    zeros_scales fp16 [K/g, 2N], dequantised fp16 weight [N, K]).  Reference :5-32."""
    dev = weight.device
    if n_bit != 4:
        raise NotImplementedError("only n_bit=4 is packed by this build")
    if fused and weight.dtype == torch.float16 and weight.is_cuda:
        w = weight if weight.is_contiguous() else weight.contiguous()
        return quantize_pack(w.detach(), input_features, output_features, group_size)
    qweight, zeros, scales, w_fp16 = generate_quant(weight, input_features, n_bit, group_size)
    zeros_scales = torch.empty((input_features // group_size, output_features * 2), dtype=torch.float16, device=dev)
    transpose_merge_zeros_scales(zeros, scales, zeros_scales, input_features, output_features, group_size)
    qweight_awq = torch.empty((input_features, output_features // 2), dtype=torch.uint8, device=dev)
    convert_ours_to_awq(qweight, qweight_awq, input_features, output_features)
    qweight_lmdeploy = torch.empty((input_features, output_features // 8), dtype=torch.int, device=dev)
    convert_awq_to_lmdeploy(qweight_awq, qweight_lmdeploy, input_features, output_features)
    return qweight_lmdeploy, zeros_scales, w_fp16

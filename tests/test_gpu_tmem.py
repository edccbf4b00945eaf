"""The tcgen05 kernel writes dequantised weights into tensor memory with tcgen05.st.16x128b; this
checks on the hardware that the fragment mapping is the one the kernel assumes: thread t, register
2j+v of a store issued at (lane base L, column base C) lands at lane L + t/4 + 8v, column C + 4j + t%4."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_tmem_16x128b_fragment_mapping():
    import quant
    lib = quant.load_library()
    out = torch.zeros(128, 32, dtype=torch.int32, device="cuda")
    assert lib.w4a16_debug_tmem_layout(out.data_ptr(), torch.cuda.current_stream().cuda_stream) == 0
    torch.cuda.synchronize()
    got = out.cpu().numpy().view(np.uint32)
    exp = np.zeros((128, 32), dtype=np.uint32)
    for warp in range(4):
        for nh in range(2):
            for t in range(32):
                for j in range(16):
                    lane = warp * 32 + nh * 16 + t // 4 + 8 * (j % 2)
                    col = 4 * (j // 2) + t % 4
                    exp[lane, col] = (warp << 24) | (nh << 20) | (t << 8) | j
    if not np.array_equal(got, exp):
        bad = np.argwhere(got != exp)[:8]
        msg = "; ".join(f"[{l},{c}] got {got[l, c]:#x} exp {exp[l, c]:#x}" for l, c in bad)
        raise AssertionError("unexpected TMEM fragment mapping: " + msg)

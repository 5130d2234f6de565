"""GPU per-tensor quantiser against the oracle (bit-exact scale and codes)."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("shape,std", [((8, 8192), 1.0), ((8192, 1024), 0.02), ((3, 7), 5.0), ((1, 1), 1.0),
                                       ((4096, 4099), 1e-20), ((257, 129), 1e20)])
def test_bit_exact_against_oracle(cuda_device, oracle, shape, std):
    from rocm_dev_b200 import quant
    g = torch.Generator().manual_seed(shape[0] + shape[1])
    x = (torch.randn(shape, generator=g) * std).bfloat16()
    q, s = quant.quantize_per_tensor_device(x.to(cuda_device))
    for _ in range(2):                                       # scratch must be reusable call after call
        q, s = quant.quantize_per_tensor_device(x.to(cuda_device))
    import rocm_dev_b200 as R
    torch.cuda.synchronize()
    assert R.lib().rdb_device_status() == 0
    wq, ws = oracle.quantize_per_tensor(x.float().numpy())
    assert np.float32(s.item()).view(np.uint32) == np.float32(ws).view(np.uint32)
    assert np.array_equal(q.cpu().numpy(), wq)
    hq, hs = quant.quantize_per_tensor(x)                    # and the host (torch) quantiser
    assert torch.equal(q.cpu(), hq) and hs.item() == s.item()


def test_all_zero_tensor(cuda_device):
    from rocm_dev_b200 import quant
    q, s = quant.quantize_per_tensor_device(torch.zeros(1000, dtype=torch.bfloat16, device=cuda_device))
    assert s.item() == 1.0 and not q.any()


def test_feeds_the_gemm(cuda_device, oracle):
    """bf16 operands -> device quantiser -> skinny GEMM equals the host-quantised path."""
    import rocm_dev_b200 as R
    from rocm_dev_b200 import quant
    g = torch.Generator().manual_seed(1)
    A = torch.randn((8, 2048), generator=g).bfloat16()
    W = (torch.randn((1024, 2048), generator=g) * 0.02).bfloat16()
    dev = cuda_device
    Aq, sa = quant.quantize_per_tensor_device(A.to(dev))
    Wq, sb = quant.quantize_per_tensor_device(W.to(dev))
    out = R.skinny_gemm_fp8(Aq, Wq, sa, sb)
    hAq, hsa = quant.quantize_per_tensor(A)
    hWq, hsb = quant.quantize_per_tensor(W)
    ref = R.skinny_gemm_fp8(hAq.to(dev), hWq.to(dev), hsa.to(dev), hsb.to(dev))
    assert torch.equal(out, ref)

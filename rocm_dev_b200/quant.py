"""Host-side input preparation: seeded synthetic tensors and e4m3fn quantisers.

These produce the operands the GEMM and allreduce entry points consume.  The
conversion rule is the reference's (projects/common.cuh:103 in the reference
project: saturate to finite, round to nearest even) applied to OCP e4m3fn;
``torch``'s CPU cast does not saturate, hence the clamp.
"""
from __future__ import annotations

import torch

E4M3_MAX = 448.0


def e4m3fn_sat_rn(x: torch.Tensor) -> torch.Tensor:
    """fp32 -> e4m3fn bytes (uint8), saturating, round-to-nearest-even."""
    return x.float().clamp(-E4M3_MAX, E4M3_MAX).to(torch.float8_e4m3fn).view(torch.uint8)


def quantize_per_tensor(x: torch.Tensor):
    """(q uint8, scale fp32[1]) with scale = amax/448 (1 for an all-zero tensor)
    and q = e4m3fn_sat_rn(x / scale), the division done in fp32."""
    x = x.float()
    amax = x.abs().max()
    scale = torch.where(amax > 0, amax / E4M3_MAX, torch.ones_like(amax)).reshape(1)
    return e4m3fn_sat_rn(x / scale), scale


def quantize_blocks128(x_bf16: torch.Tensor):
    """Per-128-element blocks along the flattened tensor: (q uint8 like x,
    scales fp32 [numel/128])."""
    assert x_bf16.dtype == torch.bfloat16 and x_bf16.numel() % 128 == 0
    xb = x_bf16.float().reshape(-1, 128)
    amax = xb.abs().amax(dim=1, keepdim=True)
    scale = torch.where(amax > 0, amax / E4M3_MAX, torch.ones_like(amax))
    return e4m3fn_sat_rn(xb / scale).reshape(x_bf16.shape), scale.reshape(-1)


def synthetic_gemm_operands(M: int, N: int, K: int, seed: int = 0, w_std: float = 0.02):
    """Activations bf16 N(0,1) [M,K] and weights bf16 N(0,w_std) [N,K], each
    quantised per tensor.  Returns (Aq, Bq, scale_a, scale_b) on the CPU."""
    g = torch.Generator().manual_seed(seed)
    A = torch.randn((M, K), generator=g, dtype=torch.float32).bfloat16()
    B = (torch.randn((N, K), generator=g, dtype=torch.float32) * w_std).bfloat16()
    Aq, sa = quantize_per_tensor(A)
    Bq, sb = quantize_per_tensor(B)
    return Aq, Bq, sa, sb


def synthetic_weights_fast(N: int, K: int, seed: int, device="cpu"):
    """Weight bytes with the value distribution of quantised N(0,sigma) data,
    generated directly on ``device`` (benchmark-sized matrices; the statistical
    shape, not the exact bytes, is what matters there)."""
    g = torch.Generator(device=device).manual_seed(seed)
    w = torch.randn((N, K), generator=g, dtype=torch.float32, device=device)
    amax = w.abs().max()
    return (w * (E4M3_MAX / amax)).clamp(-E4M3_MAX, E4M3_MAX).to(torch.float8_e4m3fn).view(torch.uint8), \
        (amax / E4M3_MAX * 0.02).reshape(1)


def quantize_per_tensor_device(x: torch.Tensor):
    """The same rule on the GPU (rdb_quantize_per_tensor): x bf16 CUDA tensor ->
    (q uint8 like x, scale fp32[1]), bit-exact with ``quantize_per_tensor``."""
    from ._lib import check, lib
    assert x.is_cuda and x.dtype == torch.bfloat16 and x.is_contiguous()
    q = torch.empty(x.shape, dtype=torch.uint8, device=x.device)
    s = torch.empty(1, dtype=torch.float32, device=x.device)
    with torch.cuda.device(x.device):
        check(lib().rdb_quantize_per_tensor(x.data_ptr(), q.data_ptr(), s.data_ptr(), x.numel(),
                                            torch.cuda.current_stream(x.device).cuda_stream), "rdb_quantize_per_tensor")
    return q, s

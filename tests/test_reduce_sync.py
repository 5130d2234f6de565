"""GPU tests of tiled_sum_reduce (bit-exact against the oracle's batch-order
fp32 loop) and of the grid-barrier probe, through the C ABI."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("b,m,n", [(1, 8, 64), (3, 8, 64), (4, 16, 128), (7, 64, 256), (16, 128, 512), (5, 8, 32),
                                   (9, 3, 5), (2, 1, 1), (33, 24, 100), (0, 8, 64)])
def test_bit_exact_against_oracle(cuda_device, oracle, b, m, n):
    import rocm_dev_b200 as R
    g = torch.Generator().manual_seed(b * 1000 + m + n)
    # the reference drivers draw uniform[-0.5, 0.5)
    A = torch.rand((b, m, n), generator=g) - 0.5
    B = torch.rand((b, m, n), generator=g) - 0.5
    D = torch.full((m, n), 7.0, device=cuda_device)
    R.tiled_sum_reduce(A.to(cuda_device), B.to(cuda_device), D, b, m, n)
    want = oracle.tiled_sum_reduce(A.numpy().reshape(b, m, n), B.numpy().reshape(b, m, n)) if b else np.zeros((m, n), np.float32)
    got = D.cpu().numpy()
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))
    mx, tot = oracle.deltas(got, want)          # the reference driver's metric
    assert mx == 0.0 and tot == 0.0


def test_large_is_linear_and_matches_torch(cuda_device):
    import rocm_dev_b200 as R
    b, m, n = 8, 4096, 2048
    g = torch.Generator(device=cuda_device).manual_seed(0)
    A = torch.rand((b, m, n), generator=g, device=cuda_device) - 0.5
    B = torch.rand((b, m, n), generator=g, device=cuda_device) - 0.5
    D = torch.empty((m, n), device=cuda_device)
    R.tiled_sum_reduce(A, B, D, b, m, n)
    acc = torch.zeros((m, n), device=cuda_device)
    for i in range(b):
        acc += A[i] + B[i]
    assert torch.equal(D, acc)
    D2 = torch.empty_like(D)
    R.tiled_sum_reduce(2 * A, 2 * B, D2, b, m, n)         # power-of-two scaling commutes exactly
    assert torch.equal(D2, 2 * D)


def test_unaligned_pointers_take_the_scalar_path(cuda_device, oracle):
    import rocm_dev_b200 as R
    b, m, n = 3, 8, 64
    base = torch.rand(2 * b * m * n + 8, device=cuda_device) - 0.5
    A = base[1:1 + b * m * n]
    B = base[b * m * n + 2:2 * b * m * n + 2]
    D = torch.empty(m * n + 1, device=cuda_device)[1:]
    R.tiled_sum_reduce(A.data_ptr(), B.data_ptr(), D.data_ptr(), b, m, n)
    want = oracle.tiled_sum_reduce(A.cpu().numpy().reshape(b, m, n), B.cpu().numpy().reshape(b, m, n))
    assert np.array_equal(D.cpu().numpy().reshape(m, n), want)


def test_globs_reference_probe(cuda_device):
    import rocm_dev_b200 as R
    D = torch.full((1024,), 5, dtype=torch.int32, device=cuda_device)
    for _ in range(3):                       # the barrier words must be reusable launch after launch
        R.globs(D)
    torch.cuda.synchronize()
    assert R.lib().rdb_device_status() == 0
    # 64 threads toggle the word with atomicDec(.., 1): 0 -> 1 -> 0 ... an even count ends at 0
    assert D[:2].tolist() == [0, 0] and D[2].item() == 5


@pytest.mark.parametrize("blocks,threads,rounds", [(1, 32, 1), (148, 64, 1), (148, 128, 50), (37, 33, 7), (296, 64, 5)])
def test_globs_other_grid_sizes(cuda_device, blocks, threads, rounds):
    import rocm_dev_b200 as R
    D = torch.full((2048,), 3, dtype=torch.int32, device=cuda_device)
    R.globs_n(D, blocks, threads, rounds)
    R.globs_n(D, max(1, blocks // 2), threads, rounds)      # a different grid size right after
    torch.cuda.synchronize()
    assert R.lib().rdb_device_status() == 0
    want = (threads * rounds) % 2 if False else (threads % 2)   # each round restarts from 0
    assert set(D[:blocks].tolist()) == {want}
    assert D[blocks].item() == 3


def test_globs_rejects_oversubscribed_grid(cuda_device):
    import rocm_dev_b200 as R
    D = torch.zeros(1 << 16, dtype=torch.int32, device=cuda_device)
    assert R.lib().rdb_globs_n(D.data_ptr(), 148 * 8 + 1, 64, 1, 0) == 11
    assert R.lib().rdb_globs_n(D.data_ptr(), 0, 64, 1, 0) == 8

"""The allocation-free grid-barrier probe (rdb_globs_n_noalloc).

It exists for callers that are not allowed to allocate GPU memory once they are
running (an application that hands its plugins a fixed arena, or a loop that
cannot afford the device-wide synchronisation an allocation causes): its
barrier counters sit in a small array built into the library.  Called through
the C ABI, it must write exactly what the allocating entry point
(rdb_globs_n) writes, call after call.  This file sorts last on purpose, and
the test also passes when it is the only one run in a fresh process.
"""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("blocks,threads,rounds", [(2, 64, 1), (148, 33, 5)])
def test_same_output_as_the_allocating_entry_point_twice_in_a_row(cuda_device, blocks, threads, rounds):
    import rocm_dev_b200 as R
    L = R.lib()
    stream = torch.cuda.current_stream(cuda_device).cuda_stream
    want = torch.full((2048,), 9, dtype=torch.int32, device=cuda_device)
    assert L.rdb_globs_n(want.data_ptr(), blocks, threads, rounds, stream) == 0
    torch.cuda.synchronize()
    assert L.rdb_device_status() == 0
    for call in range(2):                                   # two calls in a row share the built-in array
        got = torch.full((2048,), 9, dtype=torch.int32, device=cuda_device)
        assert L.rdb_globs_n_noalloc(got.data_ptr(), blocks, threads, rounds, stream) == 0
        assert L.rdb_noalloc_status() == 0, f"call {call}: barrier timed out"
        assert torch.equal(got, want), f"call {call}: output differs from rdb_globs_n"
    assert want[:blocks].tolist() == [threads % 2] * blocks and want[blocks].item() == 9


def test_sizes_beyond_the_built_in_scratch_are_refused(cuda_device, capfd):
    import rocm_dev_b200 as R
    L = R.lib()
    D = torch.zeros(4096, dtype=torch.int32, device=cuda_device)
    assert L.rdb_globs_n_noalloc(D.data_ptr(), 1025, 64, 1, 0) == 11          # RDB_SIZE_ABOVE_LIMIT
    assert L.rdb_globs_n_noalloc(D.data_ptr(), 1024, 64, (1 << 20) + 1, 0) == 11
    assert "beyond what the built-in scratch supports" in capfd.readouterr().err
    assert L.rdb_globs_n_noalloc(D.data_ptr(), 0, 64, 1, 0) == 8              # RDB_BAD_SHAPE
    torch.cuda.synchronize()
    assert not D.any()

"""The skinny-GEMM tuner: candidate generation (CPU) and one short search (GPU)."""
import json

import pytest

from rocm_dev_b200 import tuner


def test_candidates_fit_one_wave_and_the_ring():
    for (M, N, K) in [(8, 4096, 4096), (32, 28672, 4096), (1, 4096, 14336), (8, 256, 512)]:
        c = tuner.candidates(M, N, K)
        assert c, (M, N, K)
        mpad = 16 if M <= 16 else 32
        for rows, sk, st in c:
            assert rows % 16 == 0 and 16 <= rows <= 256 and 1 <= sk <= 8
            assert -(-N // rows) <= tuner.MAX_CLUSTERS[sk]
            assert st * (mpad + rows) * 128 <= 200 * 1024 and st <= -(-(-(-K // 128)) // sk)
    # the automatic plan (host arithmetic only) is one of the candidates' tilings
    r, s, st = tuner.automatic_plan(8, 4096, 4096)
    assert (r, s) in {(a, b) for a, b, _ in tuner.candidates(8, 4096, 4096)}


@pytest.mark.gpu
def test_short_search_writes_resumable_results(cuda_device, tmp_path, monkeypatch):
    monkeypatch.setattr(tuner, "candidates", lambda M, N, K: [(128, 1, 2), (64, 2, 2), (256, 4, 1)])
    out = tmp_path / "t.jsonl"
    s = tuner.main(["-a", "8 1024 1024", "-o", str(out)])
    lines = [json.loads(l) for l in out.read_text().splitlines()]
    assert [l["index"] for l in lines] == [0, 1, 2] and all(l["us"] > 0 for l in lines)
    assert s["best"]["us"] == min(l["us"] for l in lines) and s["automatic_us"] > 0
    tuner.main(["-a", "8 1024 1024", "-o", str(out), "-r", "2"])           # resume: only candidate 2 is re-run
    assert len(out.read_text().splitlines()) == 4

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


def test_table_file_feeds_the_plan(tmp_path):
    """The tuner's table is what the launcher's planning consults: entries set
    directly or loaded from the file the tuner writes replace the analytic plan
    for exactly their (M bucket, N, K); a file with a bad line is refused whole."""
    from rocm_dev_b200 import lib
    L = lib()
    assert L.rdb_tuning_table_clear() == 0 and L.rdb_tuning_table_size() == 0
    auto = tuner.automatic_plan(8, 4096, 4096)
    assert L.rdb_tuning_table_set_skinny(8, 4096, 4096, 128, 4, 3) == 0
    assert tuner.automatic_plan(8, 4096, 4096) == (128, 4, 3)
    assert tuner.automatic_plan(16, 4096, 4096) == (128, 4, 3)          # same bucket (M <= 16)
    assert tuner.automatic_plan(32, 4096, 4096) != (128, 4, 3)          # other bucket: analytic plan
    assert tuner.automatic_plan(8, 4096, 14336) == tuner.automatic_plan(8, 4096, 14336)
    assert L.rdb_tuning_table_set_skinny(8, 4096, 4096, 100, 4, 3) == 6   # rows not a multiple of 16
    assert L.rdb_tuning_table_set_dense(4096, 4096, 4096, 2, 144) == 0 and L.rdb_tuning_table_size() == 2
    L.rdb_tuning_table_clear()
    assert tuner.automatic_plan(8, 4096, 4096) == auto
    path = str(tmp_path / "tuned.txt")
    tuner.write_table(path, {("skinny", 16, 6144, 4096): (208, 6, 4), ("dense", 512, 4096, 4096): (128, 0)})
    assert tuner.read_table(path) == {("skinny", 16, 6144, 4096): (208, 6, 4), ("dense", 512, 4096, 4096): (128, 0)}
    assert L.rdb_tuning_table_load(path.encode()) == 0 and L.rdb_tuning_table_size() == 2
    assert tuner.automatic_plan(1, 6144, 4096) == (208, 6, 4)
    bad = tmp_path / "bad.txt"
    bad.write_text("skinny 16 256 256 64 2 2\nsparse 1 2 3\n")
    assert L.rdb_tuning_table_load(str(bad).encode()) == 13 and L.rdb_tuning_table_size() == 2   # nothing of it was taken
    assert L.rdb_tuning_table_load(str(tmp_path / "none.txt").encode()) == 12
    L.rdb_tuning_table_clear()


def test_dense_candidates():
    c = tuner.dense_candidates(4096, 4096, 4096)
    assert (2, 0) in c and (256, 0) in c and (128, 0) in c
    assert all(tr in (2, 3, 128, 256) and 0 <= g < 148 and (tr not in (2, 3) or g % 2 == 0) for tr, g in c)
    assert all(tr not in (2, 3) for tr, _ in tuner.dense_candidates(512, 512, 272))


@pytest.mark.gpu
def test_search_writes_a_table_the_launcher_uses(cuda_device, oracle, tmp_path, monkeypatch):
    """A (forced) winner ends up in the table file; once loaded, the plain entry
    point runs that configuration and still meets the oracle."""
    import numpy as np
    import torch
    import rocm_dev_b200 as R
    from rocm_dev_b200 import quant
    from helpers import bf16_bits, check_gemm_parity
    L = R.lib()
    monkeypatch.setattr(tuner, "candidates", lambda M, N, K: [(64, 2, 2), (128, 4, 2)])
    monkeypatch.setattr(tuner, "time_config",
                        lambda M, N, K, r, sk, st, **kw: {(64, 2, 2): 5.0, (128, 4, 2): 3.0}.get((r, sk, st), 9.0))
    table = tmp_path / "tuned.txt"
    s = tuner.main(["-a", "8 1024 2048", "-o", str(tmp_path / "t.jsonl"), "--table", str(table)])
    assert s["best"]["rows"] == 128 and tuner.read_table(str(table)) == {("skinny", 16, 1024, 2048): (128, 4, 2)}
    monkeypatch.undo()
    try:
        assert L.rdb_tuning_table_load(str(table).encode()) == 0
        assert tuner.automatic_plan(8, 1024, 2048) == (128, 4, 2)
        Aq, Bq, sa, sb = quant.synthetic_gemm_operands(8, 1024, 2048, seed=3)
        out = R.skinny_gemm_fp8(Aq.to(cuda_device), Bq.to(cuda_device), sa.to(cuda_device), sb.to(cuda_device))
        torch.cuda.synchronize()
        assert L.rdb_device_status() == 0
        ref = oracle.gemm_fp8_bf16(Aq.numpy(), Bq.numpy(), sa.item(), sb.item())
        ref64, mag = oracle.gemm_fp8_f64(Aq.numpy(), Bq.numpy(), sa.item(), sb.item())
        check_gemm_parity(bf16_bits(out), ref, ref64, mag, 2048)
        d = tuner.main(["-p", "dense", "-a", "512 512 512", "-o", str(tmp_path / "d.jsonl"), "--table", str(table)])
        assert d["best"]["us"] > 0 and d["automatic_us"] > 0
    finally:
        L.rdb_tuning_table_clear()
    assert np.isfinite(s["automatic_us"])


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

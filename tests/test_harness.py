"""The reference's harness protocol (project directory, literal hipcc command,
stdout formats) driven end to end.  CPU part: parsing and bookkeeping with a
stand-in executable.  GPU part: the real drivers compiled through the hipcc
shim against librocm_dev_b200.so."""
import json
import os
import shutil
import stat

import pytest

from rocm_dev_b200 import harness

HARNESS = os.path.join(os.path.dirname(os.path.abspath(__file__)), "harness")


def test_parsers():
    assert harness.parse_test_output('{"max_delta": 0.25, "total_delta": 3}') == (0.25, 3.0)
    mx, _ = harness.parse_test_output('{"max_delta": nan, "total_delta": 1}')
    assert mx != mx
    warm, timed = harness.parse_bench_output("5.5, 4, End of warmup, 3, 2.5, 2, ")
    assert warm == [5.5, 4.0] and timed == [3.0, 2.5, 2.0]
    with pytest.raises(ValueError):
        harness.parse_bench_output("1, 2, 3, ")
    s = harness.summarise([3.0, 2.5, 2.0], [0.5, 0.25], [1.0, 2.0], "msg")
    assert s["mean"] == 2.5 and s["median"] == 2.5 and s["message"] == "msg"
    assert s["max_deltas"].startswith("0.5000 <- [0.5000, 0.2500]")


def test_project_flow_with_a_stand_in_compiler(tmp_path, monkeypatch):
    root = tmp_path
    (root / "projects" / "demo").mkdir(parents=True)
    (root / "projects" / "demo" / "test.cu").write_text("// test")
    (root / "projects" / "demo" / "bench.cu").write_text("// bench")
    bindir = root / "bin"
    bindir.mkdir()
    # a fake hipcc: "compiles" to a shell script that prints the protocol
    fake = bindir / "hipcc"
    fake.write_text('#!/bin/bash\nout="${@: -1}"\n'
                    'if [[ "$2" == *test.cu ]]; then printf \'#!/bin/bash\\nprintf "{\\\\"max_delta\\\\": 0.5, \\\\"total_delta\\\\": 2}"\\n\' > "$out";\n'
                    'else printf \'#!/bin/bash\\nprintf "9, 8, End of warmup, 4, 2, "\\n\' > "$out"; fi\nchmod +x "$out"\n')
    fake.chmod(fake.stat().st_mode | stat.S_IEXEC)
    monkeypatch.setenv("PATH", f"{bindir}:{os.environ['PATH']}")
    monkeypatch.chdir(root)
    data = harness.main(["-p", "demo", "-a", "1 2 3", "-t", "2", "-m", "hello"])
    assert data["mean"] == 3.0 and data["median"] == 3.0 and data["message"] == "hello"
    assert data["max_deltas"].startswith("0.5000")
    recs = list((root / "data" / "demo").glob("*.json"))
    assert len(recs) == 1 and json.loads(recs[0].read_text())["1 2 3"][0]["mean"] == 3.0
    assert len(list((root / "backups" / "demo").glob("*.zip"))) == 1
    with pytest.raises(FileNotFoundError):
        harness.Project("missing", str(root))


@pytest.mark.gpu
@pytest.mark.parametrize("project,args,tol", [("skinny_gemm", "8 1024 1024", 0.01), ("async_gemm_16x16x64", "64 64 256", 1e-3),
                                              ("async_gemm_blanes", "32 96 128", 1e-3), ("async_gemm_sparse", "8 64 64", 1e-3),
                                              ("tiled_sum_reduce", "4 8 64", 0.0), ("tiled_sum_reduce_async", "3 16 96", 0.0),
                                              ("global_sync", "", 0.0)])
def test_reference_protocol_end_to_end(cuda_device, oracle, tmp_path, monkeypatch, project, args, tol):
    if shutil.which("nvcc") is None:
        pytest.skip("nvcc not on PATH")
    monkeypatch.setenv("PATH", f"{os.path.join(HARNESS, 'bin')}:{os.environ['PATH']}")
    root = tmp_path
    shutil.copytree(os.path.join(HARNESS, "projects"), root / "projects")
    (root / "build").mkdir()
    monkeypatch.chdir(root)
    data = harness.main(["-p", project, "-a", args, "-t", "1"])
    assert data["mean"] > 0 and data["median"] > 0
    assert float(data["max_deltas"].split(" ")[0]) <= tol

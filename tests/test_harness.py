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


def _driver_formats():
    """The printf formats the real drivers use (tests/harness/common.cuh), so
    that the stand-in executables below print exactly what they print."""
    import re
    src = open(os.path.join(HARNESS, "common.cuh")).read()
    sample = re.search(r'printf\("(%[.0-9a-z]+, )", ms \* 1000.0f\)', src).group(1)
    warm = re.search(r'printf\("(End of warmup, )"\)', src).group(1)
    deltas = re.search(r'printf\("(\{.*?\})", mx, tot\)', src).group(1).replace('\\"', '"')
    return sample, warm, deltas


def test_the_reference_harness_itself_accepts_the_drivers_output(tmp_path):
    """The reference's OWN bench.py and class_project.py, unmodified (located
    through RDB_REFERENCE_ROOT, copied next to a projects/ directory, never
    committed), run against executables that print what this repository's
    drivers print: its test parser (bench.py:31-44) and its time parser
    `time_string[2:-3].split(", ")[3:]` (bench.py:49-56) accept the output and
    the summary and the record come out right."""
    import subprocess
    import sys
    ref = os.environ.get("RDB_REFERENCE_ROOT", "/root/reference")
    if not (os.path.isfile(os.path.join(ref, "bench.py")) and os.path.isfile(os.path.join(ref, "class_project.py"))):
        pytest.skip("reference harness not available on this machine")
    sample_fmt, warm_token, delta_fmt = _driver_formats()
    root = tmp_path
    for f in ("bench.py", "class_project.py"):
        shutil.copy(os.path.join(ref, f), root / f)
    (root / "projects" / "demo").mkdir(parents=True)
    (root / "projects" / "demo" / "test.cu").write_text("// test")
    (root / "projects" / "demo" / "bench.cu").write_text("// bench")
    (root / "build").mkdir()
    warm, timed = [31.5, 20.25, 19.0, 18.5, 18.25], [12.5, 12.25, 12.75, 12.0]
    bench_out = "".join(sample_fmt % v for v in warm) + warm_token + "".join(sample_fmt % v for v in timed)
    test_out = delta_fmt % (0.0625, 1.5)
    (root / "expected_test.txt").write_text(test_out)
    (root / "expected_bench.txt").write_text(bench_out)
    bindir = root / "bin"
    bindir.mkdir()
    fake = bindir / "hipcc"             # "compiles" <file> to a script that prints the recorded driver output
    fake.write_text('#!/bin/bash\nout="${@: -1}"\nsrc="$2"\nkind=test; [[ "$src" == *bench.cu ]] && kind=bench\n'
                    f'printf \'#!/bin/bash\\ncat "{root}/expected_%s.txt"\\n\' "$kind" > "$out"\nchmod +x "$out"\n')
    fake.chmod(fake.stat().st_mode | stat.S_IEXEC)
    env = dict(os.environ, PATH=f"{bindir}:{os.environ['PATH']}")
    res = subprocess.run([sys.executable, "bench.py", "-p", "demo", "-a", "8 64 64", "-t", "2", "-m", "drop-in"], cwd=root, env=env,
                         capture_output=True, text=True, timeout=120)
    assert res.returncode == 0, res.stdout + res.stderr
    data = json.loads(res.stdout[res.stdout.index("{"):])
    # the reference's parser drops the last character of the last sample (12.0000 -> 12.000): same value
    assert data["median"] == pytest.approx(12.375) and data["mean"] == pytest.approx(12.375) and data["message"] == "drop-in"
    assert data["max_deltas"].startswith("0.0625 <- [0.0625, 0.0625]")
    recs = list((root / "data" / "demo").glob("*.json"))
    assert len(recs) == 1 and json.loads(recs[0].read_text())["8 64 64"][0]["median"] == pytest.approx(12.375)
    # and this repository's mirror of the harness reads the same output the same way
    w, t = harness.parse_bench_output(bench_out)
    assert t == timed and w == warm
    assert harness.parse_test_output(test_out) == (0.0625, 1.5)


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

"""Experiment harness with the reference's command line and stdout protocol.

Mirrors the reference's ``bench.py`` / ``class_project.py`` (paths within the
reference project): a project is a directory ``projects/<name>/`` holding
``test.cu`` and ``bench.cu``; each is compiled with the literal command
``hipcc -O3 <file> -save-temps -o <name>.out`` (class_project.py:56), moved to
``./build`` and run with the argument string; ``test`` prints one JSON object
with ``max_delta`` / ``total_delta`` (bench.py:37-39); ``bench`` prints
", "-separated microsecond samples with the token ``End of warmup`` between
warm-up and timed samples (bench.py:49-56).  Results are summarised as
mean / std / median (bench.py:58-62), the project directory is archived under
its md5 (class_project.py:71-86) and the record appended to
``data/<project>/<md5>.json`` (class_project.py:88-103).

On a CUDA machine ``hipcc`` is the small shim in tests/harness/bin, which
forwards to nvcc and links librocm_dev_b200.so.

    python -m rocm_dev_b200.harness -p skinny_gemm -a "8 8192 8192" -t 3
"""
from __future__ import annotations

import argparse
import hashlib
import json
import os
import shutil
import statistics
import subprocess
from typing import Any

TEMP_SUFFIXES = (".bc", ".hipi", ".hipfb", ".o", ".s", ".out", "out.resolution.txt", ".ii", ".cubin", ".ptx",
                 ".fatbin", ".fatbin.c", ".module_id", ".reg.c", ".stub.c", ".cudafe1.cpp", ".cudafe1.c", ".gpu")


class Project:
    def __init__(self, name: str, root: str | None = None):
        self.name = name
        self.root = os.path.abspath(root or os.getcwd())
        self.project_dir = os.path.join(self.root, "projects", name)
        if not os.path.isdir(self.project_dir):
            raise FileNotFoundError(f"Directory {self.project_dir} does not exist")
        self.backup_dir = os.path.join(self.root, "backups", name)
        os.makedirs(self.backup_dir, exist_ok=True)

    # -- compile + run ------------------------------------------------------
    def compile_and_run(self, c_file: str, arguments: str = "", timeout: float | None = None) -> str:
        stem = c_file.split(".")[0]
        src = os.path.join(self.project_dir, c_file)
        subprocess.check_call(f"hipcc -O3 {src} -save-temps -o {stem}.out".split(), cwd=self.root)
        build = os.path.join(self.root, "build")
        shutil.rmtree(build, ignore_errors=True)
        os.mkdir(build)
        for f in os.listdir(self.root):
            if os.path.isfile(os.path.join(self.root, f)) and f.endswith(TEMP_SUFFIXES):
                shutil.move(os.path.join(self.root, f), os.path.join(build, f))
        return self.run(c_file, arguments, timeout)

    def run(self, c_file: str, arguments: str = "", timeout: float | None = None) -> str:
        stem = c_file.split(".")[0]
        out = subprocess.check_output([os.path.join(self.root, "build", f"{stem}.out"), *arguments.split()],
                                      timeout=timeout, cwd=self.root)
        return out.decode()

    # -- bookkeeping --------------------------------------------------------
    def backup(self) -> str:
        tmp = os.path.join(self.backup_dir, "tmp")
        shutil.make_archive(tmp, "zip", self.project_dir)
        with open(tmp + ".zip", "rb") as f:
            digest = hashlib.md5(f.read()).hexdigest()
        final = os.path.join(self.backup_dir, digest + ".zip")
        if os.path.exists(final):
            os.remove(tmp + ".zip")
        else:
            os.rename(tmp + ".zip", final)
        return digest

    def record(self, digest: str, arguments: str, data: dict[str, Any]) -> str:
        d = os.path.join(self.root, "data", self.name)
        os.makedirs(d, exist_ok=True)
        path = os.path.join(d, f"{digest}.json")
        rec = {}
        if os.path.exists(path):
            with open(path) as f:
                rec = json.load(f)
        rec.setdefault(arguments, []).append(data)
        with open(path, "w") as f:
            json.dump(rec, f)
        return path


def parse_test_output(text: str) -> tuple[float, float]:
    """``{"max_delta": x, "total_delta": y}`` -> (x, y); nan is tolerated."""
    parsed = json.loads(text.replace("nan", '"nan"'))
    return float(parsed["max_delta"]), float(parsed["total_delta"])


def parse_bench_output(text: str) -> tuple[list[float], list[float]]:
    """(warm-up samples, timed samples) in microseconds."""
    toks = [t.strip() for t in text.split(",") if t.strip()]
    if "End of warmup" not in toks:
        raise ValueError("bench output has no 'End of warmup' marker")
    i = toks.index("End of warmup")
    return [float(t) for t in toks[:i]], [float(t) for t in toks[i + 1:]]


def summarise(times: list[float], max_deltas: list[float], sum_deltas: list[float], message: str) -> dict[str, Any]:
    fmt = lambda xs: f"{max(xs):.4f} <- [" + ", ".join(f"{x:.4f}" for x in xs) + "]"  # noqa: E731
    return {
        "mean": statistics.fmean(times) if times else 0.0,
        "std": statistics.pstdev(times) if len(times) > 1 else 0.0,
        "median": statistics.median(times) if times else 0.0,
        "message": message,
        "max_deltas": fmt(max_deltas),
        "sum_deltas": fmt(sum_deltas),
    }


def main(argv=None) -> dict[str, Any]:
    ap = argparse.ArgumentParser()
    ap.add_argument("--project", "-p", required=True)
    ap.add_argument("--message", "-m", default="")
    ap.add_argument("--arguments", "-a", default="")
    ap.add_argument("--test-runs", "-t", type=int, default=1)
    ap.add_argument("--skip-bench", "-sb", action="store_true")
    ap.add_argument("--root", default=None, help="directory holding projects/ (default: cwd)")
    a = ap.parse_args(argv)
    proj = Project(a.project, a.root)
    max_d, sum_d = ([], []) if a.test_runs > 0 else ([-1.0], [-1.0])
    for i in range(a.test_runs):
        out = proj.compile_and_run("test.cu", a.arguments) if i == 0 else proj.run("test.cu", a.arguments)
        mx, tot = parse_test_output(out)
        max_d.append(mx)
        sum_d.append(tot)
    times = [0.0]
    if not a.skip_bench:
        _, times = parse_bench_output(proj.compile_and_run("bench.cu", a.arguments))
    data = summarise(times, max_d, sum_d, a.message)
    print(json.dumps(data, indent=4))
    proj.record(proj.backup(), a.arguments, data)
    return data


if __name__ == "__main__":
    main()

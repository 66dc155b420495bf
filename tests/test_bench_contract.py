"""The parts of bench.py's contract that need no GPU: more than one GPU is refused with one line and
exit code 2; without a GPU the reference arm says why it is unavailable and exits 0; the peaks come from
MEASURED_PEAKS.json when it is there, else the fallback figures."""

import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _run(*args):
    return subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), *args], capture_output=True, text=True, cwd=ROOT,
                          timeout=300)


def test_more_than_one_gpu_is_one_line_and_exit_2():
    r = _run("--gpus", "2", "--steps", "4", "--warmup", "3")
    assert r.returncode == 2
    lines = [ln for ln in r.stdout.splitlines() if ln.strip()]
    assert len(lines) == 1 and "one GPU" in lines[0]


def test_reference_arm_without_a_gpu_is_unavailable_with_a_reason():
    r = _run("--impl", "reference", "--gpus", "1", "--steps", "4", "--warmup", "3")
    assert r.returncode == 0
    out = json.loads(r.stdout.strip().splitlines()[-1])
    assert out["impl"] == "reference" and isinstance(out["unavailable"], str) and out["unavailable"]


def test_peaks_fall_back_when_the_measured_file_is_absent():
    sys.path.insert(0, ROOT)
    import bench

    hbm, tflops, src = bench.peaks()
    assert hbm > 0 and tflops > 0 and src in ("measured", "fallback")
    if not os.path.exists(os.path.join(ROOT, "MEASURED_PEAKS.json")):
        assert (hbm, tflops, src) == (6650.0, 1590.0, "fallback")

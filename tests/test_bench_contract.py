"""The measurement script's contract as far as it can be checked without a GPU, and its record on one."""

import json
import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
BENCH = os.path.join(ROOT, "bench.py")


def test_more_than_one_gpu_is_refused_with_one_line_and_exit_code_2():
    done = subprocess.run([sys.executable, BENCH, "--gpus", "2", "--steps", "1", "--warmup", "1"], capture_output=True, text=True,
                          timeout=300)
    assert done.returncode == 2
    assert len(done.stdout.strip().splitlines()) == 1 and "--gpus 2" in done.stdout


def test_peaks_come_from_the_measured_file_or_the_stated_fallback(tmp_path, monkeypatch):
    sys.path.insert(0, ROOT)
    import bench
    values, kind = bench.peaks()
    assert kind in ("measured", "fallback") and values["hbm_gbs"] > 1000 and values["bf16_tflops"] > 100


def test_both_arms_print_the_same_metric_unit_and_direction():
    """The driver divides one arm's value by the other's only if these agree; the reference arm's record is built without running it."""
    sys.path.insert(0, ROOT)
    import inspect

    import bench
    ref = bench.reference_record(1000.0, 20, 5, 0.16, 16, {"sm_mhz": 1900})
    assert ref["metric"] == bench.METRIC and ref["unit"] == bench.UNIT and ref["higher_is_better"] is True
    assert ref["impl"] == "reference" and ref["e2e"]["unit"] == bench.UNIT
    assert ref["e2e"]["h2d_bytes_per_step"] > 0 and ref["e2e"]["d2h_bytes_per_step"] > 0
    assert len(ref["config"]) <= 20 and all(not isinstance(v, (dict, list)) for v in ref["config"].values())
    ours = inspect.getsource(bench.run_ours)
    assert '"metric": METRIC' in ours and '"unit": UNIT' in ours and '"higher_is_better": True' in ours
    shared = bench.size_config(bench.MODEL, "Llama-3.2-1B", 16, 16)
    assert all(ref["config"][k] == v for k, v in shared.items())


@pytest.mark.gpu
def test_a_short_run_prints_one_record_with_the_contract_keys():
    done = subprocess.run([sys.executable, BENCH, "--layers", "2", "--steps", "5", "--warmup", "3"], capture_output=True, text=True,
                          timeout=900)
    assert done.returncode == 0, done.stderr[-2000:]
    lines = [line for line in done.stdout.splitlines() if line.startswith("{")]
    assert len(lines) == 1
    record = json.loads(lines[0])
    for key in ("metric", "value", "unit", "n_gpus", "steps", "warmup", "ms_per_step", "higher_is_better", "scaling", "vs_baseline",
                "dtype", "data", "config", "prefill", "roofline", "points", "e2e", "gpu_launches", "clocks"):
        assert key in record, key
    sys.path.insert(0, ROOT)
    import bench
    assert record["metric"] == bench.METRIC and record["unit"] == bench.UNIT and record["higher_is_better"] is True
    assert record["n_gpus"] == 1 and record["steps"] == 5 and record["gpu_launches"] > 0
    assert len(record["config"]) <= 20 and all(not isinstance(v, (dict, list)) for v in record["config"].values())
    assert record["config"]["layers"] == 2 and record["config"]["layers_of_model"] == 16
    assert set(record["prefill"]) >= {"value", "tokens", "ms", "frac"} and record["prefill"]["tokens"] == 2048
    assert set(record["roofline"]) >= {"bound", "achieved", "peak", "unit", "frac"}
    assert set(record["points"]) >= {"decode_b1", "decode_b64"}
    assert record["e2e"]["h2d_bytes_per_step"] > 0 and record["e2e"]["d2h_bytes_per_step"] > 0

"""Host logic of bench.py that needs no GPU: the deadline that lets a multi-rank run report its headline line when one of
its extra measurements never returns (made on the host: the guarded part simply sleeps)."""
import json
import os
import subprocess
import sys
import textwrap

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _child(rank: int, cancel: bool):
    code = textwrap.dedent(f"""
        import os, sys, time
        sys.path.insert(0, {ROOT!r})
        import bench
        t = bench.start_exit_timer(0.5, {rank}, 1, lambda: {{"metric": "m", "value": 1.0, "decode": {{"error": "left out"}}}},
                                   lambda: "decode")
        if {cancel!r}:
            t.cancel()
            print("finished")
            sys.exit(0)
        time.sleep(60)  # the extra that never returns
        print("not reached")
    """)
    return subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, timeout=30)


def test_deadline_reports_the_line_on_rank_0_and_leaves_with_exit_code_0():
    res = _child(0, cancel=False)
    assert res.returncode == 0
    lines = [l for l in res.stdout.splitlines() if l.strip()]
    assert len(lines) == 1 and "not reached" not in res.stdout
    line = json.loads(lines[0])
    assert line["value"] == 1.0 and "error" in line["decode"]
    assert "deadline" in res.stderr and "decode" in res.stderr


def test_deadline_on_other_ranks_prints_nothing():
    res = _child(3, cancel=False)
    assert res.returncode == 0 and res.stdout.strip() == ""


def test_cancelled_deadline_does_nothing():
    res = _child(0, cancel=True)
    assert res.returncode == 0 and res.stdout.strip() == "finished"


def test_reference_arm_line_and_independence_from_the_product():
    """`bench.py --impl reference` on CPU: one JSON line with the keys of the contract, the same `config` object the GPU arm
    prints for that workload, and a process that never imported the product package (so it maps no CUDA library)."""
    code = textwrap.dedent(f"""
        import runpy, sys
        sys.argv = ["bench.py", "--impl", "reference", "--steps", "1", "--warmup", "1"]
        sys.path.insert(0, {ROOT!r})
        runpy.run_path({os.path.join(ROOT, "bench.py")!r}, run_name="__main__")
        sys.stderr.write("PRODUCT_IMPORTED=" + str(any(m == "floneum_b200" or m.startswith("floneum_b200.") for m in sys.modules)) + "\\n")
    """)
    res = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, timeout=600)
    assert res.returncode == 0, res.stderr[-2000:]
    lines = [l for l in res.stdout.splitlines() if l.strip()]
    assert len(lines) == 1
    line = json.loads(lines[0])
    assert line["impl"] == "reference" and line["higher_is_better"] is True and line["unit"] == "TFLOP/s"
    assert line["steps"] == 1 and line["n_gpus"] == 1 and line["value"] > 0
    cb = line["cpu_baseline"]
    assert cb["kind"] == "port" and cb["cores"] >= 1 and cb["value"] == line["value"] and cb["sample"]
    assert line["e2e"] == {"value": line["value"], "unit": line["unit"], "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}
    sys.path.insert(0, ROOT)
    import bench
    assert line["config"] == bench.workload_config("cfg2", 1) and line["metric"] == bench.METRIC
    assert "PRODUCT_IMPORTED=False" in res.stderr


def test_reference_arm_other_ranks_do_nothing():
    env = dict(os.environ, RANK="1", WORLD_SIZE="2", LOCAL_RANK="1")
    res = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--gpus", "2", "--steps", "1",
                          "--warmup", "1"], capture_output=True, text=True, timeout=120, env=env)
    assert res.returncode == 0 and res.stdout.strip() == ""

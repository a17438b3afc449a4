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

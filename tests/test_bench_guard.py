"""The benchmark's guard around its side measurements: the JSON line comes out exactly once - from the normal
path, or from the timer when the main thread is stuck - and the process then ends with status 0."""
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

STUCK = r'''
import sys, time
sys.path.insert(0, sys.argv[1])
import bench
extras = {"first": 1}
guard = bench.LineGuard(sys.argv[2] == "printer", lambda: {"metric": "m", "extras": dict(extras)}, extras, 0.5)
guard.start()
time.sleep(30)          # a collective that never returns
print("not reached")
'''

NORMAL = r'''
import sys
sys.path.insert(0, sys.argv[1])
import bench
extras = {}
guard = bench.LineGuard(True, lambda: {"metric": "m", "extras": dict(extras)}, extras, 30.0)
guard.start()
extras["done"] = True
guard.finish()
guard.finish()          # a second call prints nothing
'''


def _run(code, *args):
    return subprocess.run([sys.executable, "-c", code, ROOT, *args], capture_output=True, text=True, timeout=20)


def test_a_stuck_main_thread_still_yields_the_line_and_a_clean_exit():
    r = _run(STUCK, "printer")
    assert r.returncode == 0 and "not reached" not in r.stdout
    lines = [l for l in r.stdout.splitlines() if l.strip()]
    assert len(lines) == 1
    d = json.loads(lines[0])
    assert d["extras"]["first"] == 1 and "did not finish" in d["extras"]["watchdog"]


def test_ranks_that_do_not_print_only_exit():
    r = _run(STUCK, "silent")
    assert r.returncode == 0 and r.stdout.strip() == ""


def test_the_normal_path_prints_once_and_cancels_the_timer():
    r = _run(NORMAL)
    assert r.returncode == 0
    lines = [l for l in r.stdout.splitlines() if l.strip()]
    assert len(lines) == 1 and json.loads(lines[0])["extras"] == {"done": True}

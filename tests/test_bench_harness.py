"""Host-side pieces of bench.py that decide whether the headline number survives a slow or stuck extra workload:
child processes with a time limit (the whole process group is ended at the limit), the JSON line taken from a child's
output, and the time budget that skips an extra workload instead of cutting into the headline run."""
import os
import sys
import time
import types

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import bench  # noqa: E402


def test_child_result_is_the_last_json_line(monkeypatch):
    monkeypatch.setattr(bench, "MIN_CHILD_S", 0.1)
    r = bench.run_child(["-c", "print('noise'); print('{\"value\": 1}'); print('{\"value\": 2}'); print('tail')"], dict(os.environ), 30.0)
    assert r == {"value": 2}
    assert bench.run_child(["-c", "print('no json here')"], dict(os.environ), 30.0) is None
    r = bench.run_child(["-c", "import sys; sys.stderr.write('boom'); sys.exit(3)"], dict(os.environ), 30.0)
    assert "exit code 3" in r["unavailable"] and "boom" in r["unavailable"]


def test_child_that_hangs_is_ended_with_its_own_children(monkeypatch, tmp_path):
    monkeypatch.setattr(bench, "MIN_CHILD_S", 0.1)
    pid_file = tmp_path / "grandchild.pid"
    code = ("import subprocess, sys, time\n"
            "p = subprocess.Popen([sys.executable, '-c', 'import time; time.sleep(60)'])\n"
            f"open({str(pid_file)!r}, 'w').write(str(p.pid))\n"
            "time.sleep(60)\n")
    t0 = time.monotonic()
    r = bench.run_child(["-c", code], dict(os.environ), 2.0)
    assert "did not finish" in r["unavailable"]
    assert time.monotonic() - t0 < 20
    pid = int(pid_file.read_text())
    for _ in range(50):                      # the grandchild belongs to the child's process group and goes with it
        try:
            os.kill(pid, 0)
        except ProcessLookupError:
            break
        time.sleep(0.1)
    else:
        raise AssertionError("the hung child's own child process survived the time limit")


def test_extras_without_time_left_are_skipped_not_started(monkeypatch):
    started = []
    monkeypatch.setattr(bench, "T_START", time.monotonic() - 10_000.0)         # the budget is long gone
    real = bench.run_child

    def spy(cmd, env, timeout_s):
        started.append((cmd[0], timeout_s))
        return real(cmd, env, timeout_s)
    monkeypatch.setattr(bench, "run_child", spy)
    args = types.SimpleNamespace(gpus=1, impl="ours", comm="fused", steps=2, warmup=3, extras_timeout=600.0, time_budget=800.0)
    out = bench.run_extras(args)
    assert started and all(t < bench.MIN_CHILD_S for _, t in started)
    assert "skipped" in out["config3_qwen3_8b_tp1"]["unavailable"]

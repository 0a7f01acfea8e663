"""Host-side pieces of bench.py that need no GPU: the clock record and the result-line plumbing."""
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_clock_record_reports_only_the_timed_region():
    import bench
    s = bench.ClockSampler(0)

    class Done:                      # stands in for the sampling process
        def terminate(self):
            pass
    s.proc = Done()
    # rows as the sampler stores them: fields of the query, then the arrival time
    s.rows = [["1200", "1965", "Not Active", "Not Active", "Not Active", "Active", 1.0],     # before the region: ignored
              ["1965", "1965", "Not Active", "Not Active", "Not Active", "Not Active", 5.0],
              ["1950", "1965", "Not Active", "Not Active", "Not Active", "Active", 6.0],
              ["1965", "1965", "Not Active", "Not Active", "Not Active", "Not Active", 7.0],
              ["garbage", 8.0]]
    s.t_begin = 4.0
    rec = s.stop()
    assert rec == {"sm_mhz": 1965, "sm_max_mhz": 1965, "reasons": ["sw_power_cap"], "samples": 3}
    s.rows[2][2] = "Active"
    assert s.stop()["reasons"] == ["hw_slowdown", "sw_power_cap"]


def test_only_the_result_line_reaches_stdout():
    """Whatever is written to file descriptor 1 after divert_stdout() lands on stderr; emit() writes the line."""
    code = ("import os, sys; sys.path.insert(0, %r); import bench; bench.divert_stdout(); "
            "os.write(1, b'library chatter\\n'); print('more chatter'); bench.emit('{\"ok\": 1}')" % ROOT)
    r = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, timeout=120)
    assert r.returncode == 0, r.stderr
    assert r.stdout.strip().splitlines() == ['{"ok": 1}'] and json.loads(r.stdout)["ok"] == 1
    assert "library chatter" in r.stderr and "more chatter" in r.stderr

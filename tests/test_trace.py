"""Stage stamps (XSCHED_TRACE_FILE) and the bench's timeline arithmetic, without a GPU: the host lane under the
in-process scheduler must leave ready / decision / operation / suspend / resume records in one file per process,
and bench.timeline_stages must turn records of three processes into the per-stage durations they encode."""
import importlib.util
import os
import subprocess
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent
DRIVER = ROOT / "oracle" / "lane_driver_new"


def load_bench():
    spec = importlib.util.spec_from_file_location("bench_module", ROOT / "bench.py")
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def test_stamps_are_written_per_process_and_ordered(tmp_path):
    prefix = str(tmp_path / "trace")
    env = dict(os.environ, XLOG_LEVEL="ERRO", XSCHED_TRACE_FILE=prefix)
    r = subprocess.run([str(DRIVER), "config0", "2", "200", "1000", "2000", "20", "42", "16", "8", "LCL"], env=env, capture_output=True, text=True, timeout=120)
    assert r.returncode == 0, r.stderr[-500:]
    bench = load_bench()
    traces = bench.load_traces(prefix)
    assert len(traces) == 1
    rows = next(iter(traces.values()))
    kinds = [k for _, k, _, _ in rows]
    for k in ("ready_sent", "decision", "op_sent", "op_recv", "suspend_begin", "suspend_end", "resume_begin", "resume_end"):
        assert k in kinds, k
    assert [t for t, *_ in rows] == sorted(t for t, *_ in rows)
    # every suspension that began also ended, and a resume follows it
    assert kinds.count("suspend_begin") == kinds.count("suspend_end") >= 1
    assert abs(kinds.count("resume_begin") - kinds.count("suspend_begin")) <= 1


def test_no_file_without_the_variable(tmp_path):
    env = {k: v for k, v in os.environ.items() if k != "XSCHED_TRACE_FILE"}
    env["XLOG_LEVEL"] = "ERRO"
    r = subprocess.run([str(DRIVER), "config0", "1", "50", "500", "1000", "50", "1", "4", "2", "LCL"], env=env, capture_output=True, text=True, timeout=120, cwd=tmp_path)
    assert r.returncode == 0
    assert list(tmp_path.iterdir()) == []


def test_timeline_arithmetic_on_synthetic_records():
    bench = load_bench()
    HP, LP, SRV = 100, 200, 300
    # host - device clock in ns: one device clock, so one true offset, drifting by 40 us per second against the host;
    # each process records it twice (start and end) and the reader interpolates
    def off(t):
        return 5_000_000 + (t * 40) // 1_000_000
    off_hp = off_lp = None
    hp = [(10, "gpu_clock_offset", off(10), 1000), (5_000_000, "gpu_clock_offset", off(5_000_000), 1000)]
    lp = [(11, "gpu_clock_offset", off(11), 1000), (6_000_000, "gpu_clock_offset", off(6_000_000), 1000)]
    srv = []
    for i in range(1, 4):
        t0 = 1_000_000 * i
        hp += [(t0, "app_submit", i, 0), (t0 + 2_000, "ready_sent", 7, 0)]
        srv += [(t0 + 12_000, "event_recv", 7, HP), (t0 + 13_000, "decision", 1, 0), (t0 + 14_000, "op_sent", LP, i)]
        lp += [(t0 + 24_000, "op_recv", i, 1), (t0 + 25_000, "suspend_begin", 9, 0), (t0 + 31_000, "deactivate_issued", 9, 0)]
        lp_exit_host = t0 + 61_000
        hp_start_host, hp_end_host = t0 + 191_000, t0 + 351_000
        # the LP stamps are written later, at Reactivate, with device-clock values
        lp += [(t0 + 500_000, "task_gpu_times", lp_exit_host - 700_000 - off(lp_exit_host), lp_exit_host - off(lp_exit_host))]
        hp += [(t0 + 360_000, "app_done", i, 0), (t0 + 360_100, "app_gpu_times", hp_start_host - off(hp_start_host), hp_end_host - off(hp_end_host))]
    out = bench.timeline_stages({HP: sorted(hp), LP: sorted(lp), SRV: sorted(srv)})
    assert out["requests_matched"] == 3
    st = {k: round(v["p50"]) for k, v in out["stages_us"].items()}        # whole microseconds: the interpolation is read at the record's time
    assert st == {"submit_to_ready_sent": 2.0, "ready_sent_to_server_recv": 10.0, "server_recv_to_op_sent": 2.0, "op_sent_to_lp_recv": 10.0,
                  "lp_recv_to_flag_write_issued": 7.0, "flag_write_to_lp_last_cta_exit": 30.0, "lp_last_cta_exit_to_hp_first_cta": 130.0,
                  "hp_kernel": 160.0, "hp_kernel_end_to_host_done": 9.0, "total": 360.0}
    # a request that found the GPU idle (no flag write before it completed) is left out
    hp += [(9_000_000, "app_submit", 9, 0), (9_002_000, "ready_sent", 7, 0), (9_200_000, "app_done", 9, 0), (9_200_100, "app_gpu_times", 1, 2)]
    srv += [(9_012_000, "event_recv", 7, HP)]
    assert bench.timeline_stages({HP: sorted(hp), LP: sorted(lp), SRV: sorted(srv)})["requests_matched"] == 3

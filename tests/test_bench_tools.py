"""Host-side pieces of the benchmark that need no GPU: the ncu-log -> profiles/traffic.json summary step and its reader."""
import importlib.util
import json
import os

from conftest import ROOT

HEAD = '"ID","Process ID","Process Name","Host Name","Kernel Name","Context","Stream","Block Size","Grid Size","Device","CC","Section Name","Metric Name","Metric Unit","Metric Value"'


def _bench():
    spec = importlib.util.spec_from_file_location("bench_mod", os.path.join(ROOT, "bench.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def _row(i, kernel, metric, unit, value):
    return f'"{i}","1","python","h","{kernel}","1","7","(256, 1, 1)","(12, 8, 5)","0","10.0","Command line profiler metrics","{metric}","{unit}","{value}"'


def test_traffic_is_recorded_per_launch_and_dropped_when_the_source_changes(tmp_path, capsys):
    b = _bench()
    log = tmp_path / "ncu.csv"
    lines = ["==PROF== Connected to process 1", HEAD]
    for i, (rd, wr) in enumerate([(16.0, 0.0), (15.0, 1.0)]):
        lines += [_row(2 * i, "void gemv_kernel<2, 1>(GemvArgs)", "dram__bytes_read.sum", "Mbyte", rd),
                  _row(2 * i, "void gemv_kernel<2, 1>(GemvArgs)", "dram__bytes_write.sum", "Mbyte", wr),
                  _row(2 * i, "void gemv_kernel<2, 1>(GemvArgs)", "gpu__time_duration.sum", "ns", 20000),
                  _row(2 * i + 1, "void gemv_kernel<1, 1>(GemvArgs)", "dram__bytes_read.sum", "byte", "7,900,000"),
                  _row(2 * i + 1, "void gemv_kernel<1, 1>(GemvArgs)", "dram__bytes_write.sum", "byte", 0)]
    log.write_text("\n".join(lines) + "\n")
    out = tmp_path / "traffic.json"
    b.record_traffic(str(log), "gemv_gateup_rows1", r"gemv_kernel<\(?(int\))?2", "ncu ... bench.py", out=str(out))
    rec = json.loads(out.read_text())["gemv_gateup_rows1"]
    assert rec["launches"] == 2 and rec["traffic_bytes"] == 16_000_000 and rec["dram_write_bytes"] == 500_000
    assert rec["source"].endswith("gemv.cuh") and rec["command"] == "ncu ... bench.py"
    assert b.recorded_traffic("gemv_gateup_rows1", str(out)) == 16_000_000.0
    assert b.recorded_traffic("no_such_key", str(out)) is None
    table = json.loads(out.read_text())
    table["gemv_gateup_rows1"]["source_sha256"] = "0" * 64           # the kernel source changed after the capture
    out.write_text(json.dumps(table))
    assert b.recorded_traffic("gemv_gateup_rows1", str(out)) is None


def test_the_tracked_traffic_file_names_existing_sources():
    p = os.path.join(ROOT, "profiles", "traffic.json")
    if not os.path.exists(p):
        return
    for key, rec in json.load(open(p)).items():
        assert os.path.exists(os.path.join(ROOT, rec["source"])), key
        assert rec["traffic_bytes"] > 0 and "ncu" in rec["command"] and "--clock-control none" in rec["command"], key

"""The slot policy of the persistent kernels' work-item counters (csrc/sched_slots.h) on the host: a
counter is never shared by two launches that may run at the same time, however many launches overlap."""
import os
import subprocess

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_slot_ring_policy(tmp_path):
    exe = tmp_path / "sched_slots_test"
    src = os.path.join(ROOT, "tests", "cpp", "sched_slots_test.cpp")
    inc = os.path.join(ROOT, "pku-aiprogramming_b200", "csrc")
    subprocess.run(["g++", "-std=c++17", "-O1", "-pthread", "-I" + inc, src, "-o", str(exe)], check=True)
    r = subprocess.run([str(exe)], capture_output=True, text=True, timeout=120)
    assert r.returncode == 0 and r.stdout.strip().endswith("ok"), r.stdout + r.stderr

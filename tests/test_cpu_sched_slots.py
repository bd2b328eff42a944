"""The slot policy of the persistent kernels' work-item counters (csrc/sched_slots.h) on the host: a
counter is never shared by two launches that may run at the same time, however many launches overlap."""
import os
import subprocess

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


import pytest


@pytest.mark.parametrize("sanitizer", ["none", "address,undefined", "thread"])
def test_slot_ring_policy(tmp_path, sanitizer):
    """Plain, and under the address/undefined-behaviour and thread sanitizers (the allocator is the one piece of
    host logic that several launching threads share)."""
    exe = tmp_path / "sched_slots_test"
    src = os.path.join(ROOT, "tests", "cpp", "sched_slots_test.cpp")
    inc = os.path.join(ROOT, "pku-aiprogramming_b200", "csrc")
    flags = [] if sanitizer == "none" else ["-fsanitize=" + sanitizer, "-fno-omit-frame-pointer", "-g"]
    c = subprocess.run(["g++", "-std=c++17", "-O1", "-pthread", *flags, "-I" + inc, src, "-o", str(exe)],
                       capture_output=True, text=True)
    if c.returncode != 0 and sanitizer != "none":
        pytest.skip("this toolchain cannot link -fsanitize=" + sanitizer)
    assert c.returncode == 0, c.stderr
    r = subprocess.run([str(exe)], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0 and r.stdout.strip().endswith("ok"), r.stdout + r.stderr

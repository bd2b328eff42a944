"""CPU tests of the boundary and the host logic: the C-ABI library loads and exports every
symbol the header declares, rejects bad arguments with status codes (no compute is attempted
without a GPU), the slice partition is a partition, and the sharder's gather logic works on
two gloo ranks."""
import ctypes
import os
import re
import subprocess
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "tt_attn.h")


def _declared_functions():
    src = open(HEADER).read()
    src = re.sub(r"/\*.*?\*/", "", src, flags=re.S)
    return sorted(set(re.findall(r"\b(tt_[a-z0-9_]+)\s*\(", src)))


def test_header_and_library_agree(tt):
    declared = _declared_functions()
    assert len(declared) >= 20
    lib = ctypes.CDLL(tt.capi.LIB_PATH)
    for name in declared:
        assert hasattr(lib, name), f"{name} declared in include/tt_attn.h but not exported"
    # and the Python binding covers the same set
    assert sorted(tt.capi.SIGNATURES) == declared


def test_no_cpu_fallback_without_gpu(tt):
    torch = pytest.importorskip("torch")
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    d = tt.capi.make_desc(1, 1, 8, 8, 64, tt.capi.TT_BF16, False, None)
    buf = (ctypes.c_char * 4096)()
    p = ctypes.cast(buf, ctypes.c_void_p)
    rc = tt.capi.lib.tt_attn_fwd(ctypes.byref(d), p, p, p, p, None, None)
    assert rc == tt.capi.TT_ERR_BAD_DEVICE and tt.capi.last_error()
    with pytest.raises(ValueError):
        x = torch.zeros((1, 1, 8, 64), dtype=torch.bfloat16)
        tt.attention_forward(x, x, x)


def test_argument_validation_codes(tt):
    lib, c = tt.capi.lib, tt.capi
    buf = (ctypes.c_char * 64)()
    p = ctypes.cast(buf, ctypes.c_void_p)
    assert lib.tt_attn_fwd(None, p, p, p, p, None, None) == c.TT_ERR_NULL
    d = c.make_desc(1, 1, 0, 8, 64, c.TT_BF16)
    assert lib.tt_attn_fwd(ctypes.byref(d), p, p, p, p, None, None) == c.TT_ERR_BAD_SHAPE
    d = c.make_desc(1, 1, 8, 8, 300, c.TT_F32)
    assert lib.tt_attn_fwd(ctypes.byref(d), p, p, p, p, None, None) == c.TT_ERR_BAD_SHAPE
    d = c.make_desc(1, 1, 8, 8, 64, 7)
    assert lib.tt_attn_fwd(ctypes.byref(d), p, p, p, p, None, None) == c.TT_ERR_BAD_DTYPE
    d = c.make_desc(1, 1, 8, 4, 64, c.TT_BF16, causal=True)
    assert lib.tt_attn_fwd(ctypes.byref(d), p, p, p, p, None, None) == c.TT_ERR_BAD_SHAPE
    assert "causal" in c.last_error()
    d = c.make_desc(1, 1, 8, 8, 64, c.TT_BF16)
    assert lib.tt_attn_fwd(ctypes.byref(d), None, p, p, p, None, None) == c.TT_ERR_NULL
    assert lib.tt_attn_decode(ctypes.byref(d), p, p, p, p, None, None, 0, None) == c.TT_ERR_BAD_SHAPE  # S != 1
    assert lib.tt_attn_bwd(ctypes.byref(d), p, p, p, p, p, p, p, p, p, None, 0, None) == c.TT_ERR_WORKSPACE
    assert lib.tt_attn_bwd_workspace_bytes(ctypes.byref(d)) >= 2 * 8 * 4
    assert lib.tt_attn_fwd_path(ctypes.byref(d)) == b"tcgen05"
    assert lib.tt_attn_fwd_path(ctypes.byref(c.make_desc(1, 1, 8, 8, 32, c.TT_F32))) == b"simt"
    assert lib.tt_attn_bwd_path(ctypes.byref(d)) == b"tcgen05"


def test_shard_range_is_a_partition(tt):
    for n in (0, 1, 7, 64, 128, 2048, 2049):
        for world in (1, 2, 3, 4, 8):
            nxt = 0
            sizes = []
            for r in range(world):
                b, c = tt.shard_range(n, world, r)
                assert b == nxt and c >= 0
                nxt += c
                sizes.append(c)
            assert nxt == n and max(sizes) - min(sizes) <= 1
    with pytest.raises(ValueError):
        tt.shard_range(8, 2, 2)


_GLOO_WORKER = r"""
import importlib, os, sys
import numpy as np, torch, torch.distributed as dist
sys.path.insert(0, sys.argv[1])
rank, world, n_slices = int(sys.argv[2]), int(sys.argv[3]), int(sys.argv[4])
os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=sys.argv[5], RANK=str(rank), WORLD_SIZE=str(world))
dist.init_process_group("gloo", rank=rank, world_size=world)
tt = importlib.import_module("pku-aiprogramming_b200")
from oracle import attention_oracle as orc
sh = importlib.import_module("pku-aiprogramming_b200.sharder").SliceSharder(n_slices)
S, D = 12, 8
q, k, v, _ = orc.make_inputs(5, 1, n_slices, S, S, D, with_do=False)
full = [torch.from_numpy(x) for x in (q, k, v)]
mine = [sh.shard_of(x).contiguous() for x in full]
def cpu_fwd(q_, k_, v_, causal=False, scale=None):      # stands in for the CUDA kernels on CPU ranks
    o, lse = orc.attention_forward(q_.numpy(), k_.numpy(), v_.numpy(), causal)
    return torch.from_numpy(o), torch.from_numpy(lse)
out, lse, gathered = sh.forward(*mine, causal=True, fwd=cpu_fwd)
want, _ = orc.attention_forward(q, k, v, True)
assert gathered.shape == (n_slices, S, D)
assert np.array_equal(gathered.numpy(), want.reshape(n_slices, S, D)), "gathered O differs from the unsharded result"
assert out.shape[1] == sh.count
dist.barrier(); dist.destroy_process_group()
print("ok", rank)
"""


@pytest.mark.parametrize("n_slices", [8, 7])
def test_sharder_two_gloo_ranks(tmp_path, n_slices):
    """world_size 2 on CPU: each rank computes its contiguous slice range and the all-gather
    rebuilds the full [B*H,S,D] output in place (even split) or via padding (uneven)."""
    script = tmp_path / "worker.py"
    script.write_text(_GLOO_WORKER)
    port = str(29500 + (os.getpid() % 2000) + n_slices)
    procs = [subprocess.Popen([sys.executable, str(script), ROOT, str(r), "2", str(n_slices), port],
                              stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True) for r in range(2)]
    outs = [p.communicate(timeout=240)[0] for p in procs]
    for p, o in zip(procs, outs):
        assert p.returncode == 0, o
        assert "ok" in o


def test_reference_arm_prints_contract_line():
    import json
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--steps", "1",
                        "--warmup", "0", "--workload", "cfg2"], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stderr
    line = json.loads(r.stdout.strip().splitlines()[-1])
    assert line["impl"] == "reference" and line["unit"] == "TFLOP/s" and line["value"] > 0
    assert line["cpu_baseline"]["kind"] == "port" and line["e2e"]["h2d_bytes_per_step"] == 0

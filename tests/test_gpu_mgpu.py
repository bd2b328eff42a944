"""The library's multi-GPU entry points (tt_mgpu_*) on real GPUs with the real NCCL library.

One rank on one GPU exercises every call (NCCL bound by dlopen, communicator, side stream, all-gather
into the full tensor, stream-ordered wait).  With two or more GPUs two ranks run as child processes
(NCCL_NVLS_ENABLE=0; ranks only ever leave between steps, after a barrier), each on its own half of
the slices, and every rank's gathered output and gradients must equal the one-GPU result."""
import os
import subprocess
import sys

import numpy as np
import pytest

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _np(t):
    return t.detach().float().cpu().numpy()


def test_single_rank_through_nccl(tt, oracle):
    import importlib
    sharder = importlib.import_module("pku-aiprogramming_b200.sharder")
    B, H, Hkv, S, D = 2, 4, 2, 200, 128
    q, _, _, do = oracle.make_inputs(5, B, H, S, S, D, sigma=0.6)
    _, k, v, _ = oracle.make_inputs(6, B, Hkv, S, S, D, sigma=0.6, with_do=False)
    qn, kn, vn, don = (oracle.bf16_round(x) for x in (q, k, v, do))
    dev = lambda x, h: torch.from_numpy(x).to("cuda", dtype=torch.bfloat16).reshape(1, B * h, S, D).contiguous()
    tq, tk, tv, tdo = dev(qn, H), dev(kn, Hkv), dev(vn, Hkv), dev(don, H)
    sa = sharder.ShardedAttention(1, 0, sharder.ShardedAttention.unique_id())
    try:
        out, lse, out_full = sa.forward(tq, tk, tv, B, H, causal=True)
        res = sa.backward(tq, tk, tv, out, lse, tdo, B, H, causal=True, gather_grads=True)
        sa.wait()
        tt.check_device_status()
    finally:
        sa.close()
    dq, dk, dv, dq_f, dk_f, dv_f = res
    assert torch.equal(out_full, out.reshape(B * H, S, D))
    assert torch.equal(dq_f, dq.reshape(B * H, S, D)) and torch.equal(dk_f, dk.reshape(B * Hkv, S, D)) and torch.equal(dv_f, dv.reshape(B * Hkv, S, D))
    o_r, _, dq_r, dk_r, dv_r = oracle.attention_backward_grouped(qn, kn, vn, don, True)
    assert oracle.max_abs_err(_np(out_full).reshape(B, H, S, D), o_r) <= 2e-2
    for got, ref in ((dq_f, dq_r), (dk_f, dk_r), (dv_f, dv_r)):
        assert oracle.max_abs_err(_np(got).reshape(ref.shape), ref) <= oracle.bf16_grad_tol(ref)


_WORKER = r"""
import importlib, os, sys, time
import numpy as np, torch
root, rank, world, idfile = sys.argv[1], int(sys.argv[2]), int(sys.argv[3]), sys.argv[4]
sys.path.insert(0, root)
torch.cuda.set_device(rank)
tt = importlib.import_module("pku-aiprogramming_b200")
sharder = importlib.import_module("pku-aiprogramming_b200.sharder")
from oracle import attention_oracle as orc
if rank == 0:
    with open(idfile + ".tmp", "wb") as f:
        f.write(sharder.ShardedAttention.unique_id())
    os.replace(idfile + ".tmp", idfile)
t0 = time.time()
while not os.path.exists(idfile):
    assert time.time() - t0 < 60, "no NCCL id arrived"
    time.sleep(0.05)
ident = open(idfile, "rb").read()
B, H, S, D = 2, 8, 384, 128
q, k, v, do = (orc.bf16_round(x) for x in orc.make_inputs(9, B, H, S, S, D, sigma=0.6))
full = [torch.from_numpy(x).to("cuda", dtype=torch.bfloat16) for x in (q, k, v, do)]
n = B * H // world
mine = [x.reshape(B * H, S, D)[rank * n:(rank + 1) * n].unsqueeze(0).contiguous() for x in full]
sa = sharder.ShardedAttention(world, rank, ident)
tt.set_backward_deterministic(True)
for _ in range(2):                               # second step reuses the communicator and its events
    out, lse, out_full = sa.forward(mine[0], mine[1], mine[2], B, H, causal=True)
    dq, dk, dv, dq_f, dk_f, dv_f = sa.backward(mine[0], mine[1], mine[2], out, lse, mine[3], B, H, causal=True, gather_grads=True)
    sa.wait()
torch.cuda.synchronize(); tt.check_device_status()
o1, l1 = tt.attention_forward(*full[:3], causal=True)
g1 = tt.attention_backward(full[0], full[1], full[2], o1, l1, full[3], causal=True)
torch.cuda.synchronize()
assert torch.equal(out_full, o1.reshape(B * H, S, D)), "gathered out differs from the one-GPU result"
for a, b in zip((dq_f, dk_f, dv_f), g1):
    assert torch.equal(a, b.reshape(B * H, S, D)), "gathered gradient differs from the one-GPU result"
sa.close()                                       # collective: every rank reaches it, nothing is in flight
print("ok", rank)
"""


def test_two_ranks_gather_equals_one_gpu(tmp_path):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    script = tmp_path / "worker.py"
    script.write_text(_WORKER)
    idfile = str(tmp_path / "nccl_id")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    procs = [subprocess.Popen([sys.executable, str(script), ROOT, str(r), "2", idfile], env=env,
                              stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True) for r in range(2)]
    outs = [p.communicate(timeout=300)[0] for p in procs]
    for p, o in zip(procs, outs):
        assert p.returncode == 0 and "ok" in o, o

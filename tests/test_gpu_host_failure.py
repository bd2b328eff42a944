"""Error exits of the host-buffer calls (tt_attn_fwd_host, tt_attn_bwd_host, tt_attn_fwd_bwd_host).

The failure is made on the host: a countdown in the library reports one CUDA runtime result as an error
although the runtime call was made and succeeded, so the entry point returns in the middle of its
sequence with copies and kernels still queued on its non-blocking streams.  Nothing fails on the
device.  What is checked: the call reports TT_ERR_CUDA, it synchronises its streams before its pooled
device buffers go back to the pool (so the next owner of those blocks is not written over), and the
library works as before afterwards.
"""
import ctypes

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

B, H, S, D = 2, 8, 512, 128


@pytest.fixture(scope="module")
def problem(tt):
    g = torch.Generator().manual_seed(11)
    q, k, v, do = (torch.randn(B, H, S, D, generator=g).bfloat16().pin_memory() for _ in range(4))
    tt.functional.set_backward_deterministic(True)
    out, lse, dq, dk, dv = tt.functional.attention_step_host(q, k, v, do, causal=True)
    yield dict(q=q, k=k, v=v, do=do, out=out.clone(), lse=lse.clone(), dq=dq.clone(), dk=dk.clone(), dv=dv.clone())
    tt.capi.lib.tt_debug_fail_host_call_after(-1)
    tt.functional.set_backward_deterministic(False)


def _take_pool_blocks(tt, nbytes, count):
    """Takes `count` blocks of the size the failed call just released and fills them with a pattern."""
    blocks = []
    for _ in range(count):
        p = ctypes.c_void_p()
        tt.capi.check(tt.capi.lib.tt_alloc(nbytes, ctypes.byref(p)))
        blocks.append(p)
    views = []
    for p in blocks:
        view = torch.as_tensor(_RawBlock(p.value, nbytes), device="cuda")   # a view; the pool keeps ownership
        view.fill_(0x5A)
        views.append(view)
    torch.cuda.synchronize()
    return blocks, views


class _RawBlock:
    """Minimal __cuda_array_interface__ carrier so torch can view a pool block without owning it."""
    def __init__(self, ptr, nbytes):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 2}


def _run(tt, which, p):
    f = tt.functional
    if which == "fwd":
        return f.attention_forward_host(p["q"], p["k"], p["v"], causal=True)
    if which == "bwd":
        return f.attention_backward_host(p["q"], p["k"], p["v"], p["out"], p["lse"], p["do"], causal=True)
    return f.attention_step_host(p["q"], p["k"], p["v"], p["do"], causal=True)


def _expected(which, p):
    if which == "fwd":
        return p["out"], p["lse"]
    if which == "bwd":
        return p["dq"], p["dk"], p["dv"]
    return p["out"], p["lse"], p["dq"], p["dk"], p["dv"]


@pytest.mark.parametrize("which", ["fwd", "bwd", "step"])
def test_failed_host_call_leaves_pool_and_library_usable(tt, problem, which):
    lib = tt.capi.lib
    nbytes = B * H * S * D * 2
    fired = 0
    for n in range(0, 600):
        before = lib.tt_debug_guard_syncs()
        lib.tt_debug_fail_host_call_after(n)
        try:
            res = _run(tt, which, problem)
        except tt.capi.TTError as e:
            fired += 1
            assert e.code == tt.capi.TT_ERR_CUDA and "cudaErrorUnknown" in str(e), str(e)
            assert lib.tt_debug_guard_syncs() == before + 1, "the error exit did not synchronise its streams"
            # whoever gets the released blocks next must not be written over by the abandoned sequence
            blocks, views = _take_pool_blocks(tt, nbytes, 4)
            torch.cuda.synchronize()
            for view in views:
                assert bool((view == 0x5A).all())
            del views
            for blk in blocks:
                tt.capi.check(lib.tt_free(blk))
            continue
        finally:
            lib.tt_debug_fail_host_call_after(-1)
        # the countdown outlived the call: every check of the sequence has been failed once
        for got, want in zip(res, _expected(which, problem)):
            assert torch.equal(got, want)
        break
    else:
        pytest.fail("the call never completed")
    assert fired >= 5, fired
    # and a clean call after all those failures still gives the same bits
    for got, want in zip(_run(tt, which, problem), _expected(which, problem)):
        assert torch.equal(got, want)
    assert np.isfinite(problem["out"].float().numpy()).all()

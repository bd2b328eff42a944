"""Host-side tests of the multi-GPU entry points (tt_mgpu_*): sharding rules, error mapping of failing
collective calls, and communicator life cycle, with stand-ins for the NCCL calls.  No GPU is touched
and no rank is killed: a failing collective is an error code from the stand-in."""
import ctypes
from ctypes import CFUNCTYPE, POINTER, c_int, c_size_t, c_void_p

import pytest


class _Table(ctypes.Structure):
    _fields_ = [("get_unique_id", CFUNCTYPE(c_int, c_void_p)),
                ("comm_init_rank", CFUNCTYPE(c_int, POINTER(c_void_p), c_int, c_void_p, c_int)),
                ("comm_destroy", CFUNCTYPE(c_int, c_void_p)),
                ("all_gather", CFUNCTYPE(c_int, c_void_p, c_void_p, c_size_t, c_int, c_void_p, c_void_p)),
                ("error_string", CFUNCTYPE(c_void_p, c_int))]      # returns a char* that outlives the call


class _Stub:
    """Stand-in collectives; `fail_at` names the call that returns ncclSystemError (2)."""

    def __init__(self, fail_at=None):
        self.fail_at = fail_at
        self.log = []
        self._msgs = (ctypes.create_string_buffer(b"ok"), ctypes.create_string_buffer(b"stand-in: unhandled system error"))
        self.table = _Table(
            _Table._fields_[0][1](self._uid), _Table._fields_[1][1](self._init), _Table._fields_[2][1](self._destroy),
            _Table._fields_[3][1](self._gather),
            _Table._fields_[4][1](lambda r: ctypes.addressof(self._msgs[1 if r == 2 else 0])))

    def _rc(self, name):
        self.log.append(name)
        return 2 if self.fail_at == name else 0

    def _uid(self, p):
        ctypes.memset(p, 0x5A, 128)
        return self._rc("unique_id")

    def _init(self, comm_out, world, idp, rank):
        comm_out[0] = 0x1234
        self.world, self.rank = world, rank
        return self._rc("init")

    def _destroy(self, comm):
        assert comm == 0x1234
        return self._rc("destroy")

    def _gather(self, send, recv, count, dtype, comm, stream):
        return self._rc("gather")


@pytest.fixture
def stub(tt):
    made = []

    def install(fail_at=None):
        s = _Stub(fail_at)
        made.append(s)
        tt.capi.check(tt.capi.lib.tt_mgpu_set_collectives(ctypes.byref(s.table)))
        return s
    yield install
    tt.capi.lib.tt_mgpu_set_collectives(None)


def test_unique_id_and_failure_mapping(tt, stub):
    lib, c = tt.capi.lib, tt.capi
    s = stub()
    buf = (ctypes.c_char * 128)()
    assert lib.tt_mgpu_unique_id(buf) == c.TT_OK and bytes(buf) == b"\x5a" * 128
    assert lib.tt_mgpu_unique_id(None) == c.TT_ERR_NULL
    s = stub("unique_id")
    assert lib.tt_mgpu_unique_id(buf) == c.TT_ERR_NCCL
    assert "NCCL result 2" in c.last_error() and "system error" in c.last_error()


def test_init_failure_leaves_no_communicator(tt, stub):
    lib, c = tt.capi.lib, tt.capi
    stub("init")
    buf = (ctypes.c_char * 128)()
    comm = c_void_p(0xdead)
    assert lib.tt_mgpu_init(ctypes.byref(comm), 2, 1, buf) == c.TT_ERR_NCCL
    assert comm.value is None
    assert lib.tt_mgpu_init(ctypes.byref(comm), 2, 2, buf) == c.TT_ERR_BAD_SHAPE      # rank outside the world
    assert lib.tt_mgpu_init(None, 2, 0, buf) == c.TT_ERR_NULL


def test_shard_rules(tt, stub):
    """Contiguous equal ranges; uneven splits and shards that would cut a group of query heads sharing
    key/value heads are refused."""
    lib, c = tt.capi.lib, tt.capi
    s = stub()
    buf = (ctypes.c_char * 128)()
    comms = []
    for rank in range(4):
        comm = c_void_p()
        c.check(lib.tt_mgpu_init(ctypes.byref(comm), 4, rank, buf))
        comms.append(comm)
    assert (s.world, s.rank) == (4, 3)
    first, cnt = ctypes.c_int64(), ctypes.c_int64()
    d = c.make_desc(1, 64, 32768, 32768, 128, c.TT_BF16, True)             # configuration 5: 16 heads per rank
    nxt = 0
    for rank, comm in enumerate(comms):
        c.check(lib.tt_mgpu_shard(comm, ctypes.byref(d), ctypes.byref(first), ctypes.byref(cnt)))
        assert (first.value, cnt.value) == (nxt, 16)
        b, n = tt.shard_range(64, 4, rank)
        assert (b, n) == (first.value, cnt.value)                           # same partition as tt_shard_range
        nxt += cnt.value
    d = c.make_desc(1, 6, 128, 128, 128, c.TT_BF16)                         # 6 slices over 4 ranks
    assert lib.tt_mgpu_shard(comms[0], ctypes.byref(d), ctypes.byref(first), ctypes.byref(cnt)) == c.TT_ERR_UNSUPPORTED
    d = c.make_desc(1, 8, 128, 128, 128, c.TT_BF16, Hkv=2)                  # groups of 4, shards of 2 heads
    assert lib.tt_mgpu_shard(comms[0], ctypes.byref(d), ctypes.byref(first), ctypes.byref(cnt)) == c.TT_ERR_UNSUPPORTED
    assert "group" in c.last_error()
    d = c.make_desc(2, 8, 128, 128, 128, c.TT_BF16, Hkv=2)                  # 16 slices: shards of 4 = one group each
    c.check(lib.tt_mgpu_shard(comms[2], ctypes.byref(d), ctypes.byref(first), ctypes.byref(cnt)))
    assert (first.value, cnt.value) == (8, 4)
    assert lib.tt_mgpu_bwd_workspace_bytes(comms[0], ctypes.byref(d)) > 0
    for comm in comms:
        c.check(lib.tt_mgpu_destroy(comm))
    assert s.log.count("destroy") == 4
    assert lib.tt_mgpu_destroy(None) == c.TT_OK


def test_attention_calls_need_a_device(tt, stub):
    torch = pytest.importorskip("torch")
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    lib, c = tt.capi.lib, tt.capi
    stub()
    buf = (ctypes.c_char * 4096)()
    comm = c_void_p()
    c.check(lib.tt_mgpu_init(ctypes.byref(comm), 1, 0, buf))
    d = c.make_desc(1, 2, 8, 8, 64, c.TT_BF16)
    p = ctypes.cast(buf, c_void_p)
    assert lib.tt_mgpu_attn_fwd(comm, ctypes.byref(d), p, p, p, p, None, p, None) == c.TT_ERR_BAD_DEVICE
    assert lib.tt_mgpu_wait(comm, None) == c.TT_OK          # nothing pending
    c.check(lib.tt_mgpu_destroy(comm))


def test_destroy_reports_a_failing_collective(tt, stub):
    lib, c = tt.capi.lib, tt.capi
    stub("destroy")
    buf = (ctypes.c_char * 128)()
    comm = c_void_p()
    c.check(lib.tt_mgpu_init(ctypes.byref(comm), 1, 0, buf))
    assert lib.tt_mgpu_destroy(comm) == c.TT_ERR_NCCL

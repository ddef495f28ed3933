"""Bounded device-side waits really run out, report, and leave the GPU usable: a message that is
never sent (a dropped ring stage; a peer word that nobody writes, with the "peer" tables pointing at
local memory), never a fault or an endless loop. The kernels return normally, the status word names
the cause, and the next launch is clean."""
import ctypes

import pytest
import torch

from rmlx_b200 import _lib
from rmlx_b200.ops import decode as D
from rmlx_b200.ops.weights import LinearWeight

pytestmark = pytest.mark.gpu

STATUS_MBAR_TIMEOUT, STATUS_PEER_TIMEOUT = 1, 2


@pytest.mark.parametrize("quant", [None, "q4"])
def test_dropped_ring_stage_expires_and_next_launch_is_clean(dev, quant):
    torch.manual_seed(0)
    n, k = 4096, 1024
    w = LinearWeight.from_dense(torch.randn(n, k) * 0.02, quant, device=dev)
    x = torch.randn(1, k, device=dev).to(torch.bfloat16)
    D.set_stream(True, ops="all")
    want = x.float() @ w.dequantized().t()
    assert D.stream_status() == 0
    _lib.cuda().rmlx_sg_debug_drop_stage(0)           # block 0 never receives its first stage
    got = D.rms_gemv(x, w)
    torch.cuda.synchronize()                          # the kernel returns by itself
    st = D.stream_status()
    assert st & 0xff == STATUS_MBAR_TIMEOUT and (st >> 8) & 0xf == 2, hex(st)   # a consumer's stage wait
    assert D.stream_status() == 0                     # reading clears it
    got = D.rms_gemv(x, w)                            # the next launch is unaffected
    torch.cuda.synchronize()
    assert D.stream_status() == 0
    assert (got.float() - want).abs().max().item() <= 2e-2 * want.abs().max().item()
    D.set_stream(True)                                # back to the default selection of operations


def test_peer_word_that_is_never_written_expires(dev):
    """One-shot all-reduce with world = 2 whose 'peer' is local memory nobody writes: the poll runs
    out, the status word says peer timeout, the kernel returns and a world-1 call works after."""
    from rmlx_b200.parallel import comm as C   # registers the signatures
    lib = _lib.cuda()
    n = 256
    recv0 = torch.zeros(2 * 2 * n, dtype=torch.int64, device=dev)     # 2 slots x world 2 x n words
    recv1 = torch.zeros_like(recv0)
    ctr0 = torch.zeros(8, dtype=torch.int32, device=dev)
    ctr1 = torch.zeros(8, dtype=torch.int32, device=dev)
    recv = (ctypes.c_void_p * 2)(recv0.data_ptr(), recv1.data_ptr())
    ctr = (ctypes.c_void_p * 2)(ctr0.data_ptr(), ctr1.data_ptr())
    x = torch.randn(n, device=dev)
    out = torch.empty(n, device=dev)
    assert lib.rmlx_tp_status() == 0
    rc = lib.rmlx_tp_allreduce(x.data_ptr(), None, out.data_ptr(), 1, n, recv, ctr, 0, 2, 2 * n, 0,
                               _lib.stream_ptr())
    assert rc == 0
    torch.cuda.synchronize()
    assert lib.rmlx_tp_status() == STATUS_PEER_TIMEOUT
    # rank 0's words did reach the "peer" buffer, tagged with call number 1
    assert int(recv1[:n].view(torch.int32).view(-1, 2)[:, 1].min()) == 1
    # a single-rank call on the same counters afterwards is clean (the sequence number advanced)
    rc = lib.rmlx_tp_allreduce(x.data_ptr(), None, out.data_ptr(), 1, n, recv, ctr, 0, 1, 2 * n, 0,
                               _lib.stream_ptr())
    assert rc == 0
    torch.cuda.synchronize()
    assert lib.rmlx_tp_status() == 0
    assert torch.equal(out, x)
    assert int(ctr0[0]) == 2

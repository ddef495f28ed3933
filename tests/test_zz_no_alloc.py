"""The allocation-free flash-decode entry point, called through its exported C symbol.

Who needs it: code that embeds this library in a place where it may not allocate device memory
(an engine that has already carved up the whole GPU, a real-time loop, a plug-in boundary that
passes only inputs and outputs). The test calls ``rmlx_flash_decode_paged_noalloc`` twice in a row
and checks both results against the regular entry point, which takes its scratch from the caller.
The file name sorts last on purpose, so a failing run has already exercised every other test.
"""
import ctypes
import math

import pytest
import torch

pytestmark = pytest.mark.gpu


def _setup(dev, b, hq, hkv, hd, lens):
    g = torch.Generator().manual_seed(0)
    nblk = 1 + sum((l + 15) // 16 for l in lens)
    kc = torch.randn(nblk, hkv, 16, hd, generator=g).to(torch.bfloat16).to(dev)
    vc = torch.randn(nblk, hkv, 16, hd, generator=g).to(torch.bfloat16).to(dev)
    bt = torch.zeros(b, max((l + 15) // 16 for l in lens) + 1, dtype=torch.int32)
    nxt = 1
    for i, l in enumerate(lens):
        n = (l + 15) // 16
        bt[i, :n] = torch.arange(nxt, nxt + n, dtype=torch.int32)
        nxt += n
    q = torch.randn(b, hq, hd, generator=g).to(torch.bfloat16).to(dev)
    return q, kc, vc, bt.to(dev), torch.tensor(lens, dtype=torch.int32, device=dev)


def test_noalloc_entry_matches_regular_entry_twice():
    from rmlx_b200 import _build
    from rmlx_b200.ops import decode as D

    dev = torch.device("cuda:0")
    lib = ctypes.CDLL(str(_build.CUDA_LIB))          # the exported C symbol, not a Python wrapper
    fn = lib.rmlx_flash_decode_paged_noalloc
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.c_void_p] * 6 + [ctypes.c_int] * 7 + [ctypes.c_float, ctypes.c_void_p]
    err = lib.rmlx_flash_decode_noalloc_error
    err.restype = ctypes.c_char_p
    err.argtypes = [ctypes.c_int]

    b, hq, hkv, hd, splits = 3, 32, 2, 128, 8
    scale = 1.0 / math.sqrt(hd)
    for call, lens in enumerate(([700, 33, 1500], [64, 2048, 5])):   # two calls in a row
        q, kc, vc, bt, sl = _setup(dev, b, hq, hkv, hd, lens)
        want = D.flash_decode_paged(q, kc, vc, bt, sl, scale, splits=splits)
        out = torch.empty_like(q)
        before = torch.cuda.memory_allocated()
        rc = fn(q.data_ptr(), kc.data_ptr(), vc.data_ptr(), bt.data_ptr(), sl.data_ptr(), out.data_ptr(),
                b, hq, hkv, hd, bt.stride(0), splits, 0, scale, torch.cuda.current_stream().cuda_stream)
        assert rc == 0, (rc, err(rc))
        torch.cuda.synchronize()
        assert torch.cuda.memory_allocated() == before
        diff = (out.float() - want.float()).abs().max().item()
        assert diff <= 2e-2 * max(want.float().abs().max().item(), 1e-6), (call, diff)

    # beyond the built-in scratch: a clear refusal, nothing launched
    q, kc, vc, bt, sl = _setup(dev, 3, 32, 2, 128, [64, 64, 64])
    rc = fn(q.data_ptr(), kc.data_ptr(), vc.data_ptr(), bt.data_ptr(), sl.data_ptr(), q.data_ptr(),
            3, 32, 2, 128, bt.stride(0), 17, 0, scale, torch.cuda.current_stream().cuda_stream)
    assert rc == -5 and b"exceeds the built-in scratch" in err(rc)
    rc = fn(q.data_ptr(), kc.data_ptr(), vc.data_ptr(), bt.data_ptr(), sl.data_ptr(), q.data_ptr(),
            65, 32, 2, 128, bt.stride(0), 2, 0, scale, torch.cuda.current_stream().cuda_stream)
    assert rc == -5

"""The bounds-checked build of the kernels (-DRMLX_BOUNDS): an index that leaves its table is
recorded (source file, line, index, limit) and the access is skipped or redirected to the reserved
page, so the launch returns normally. The library is chosen per process (RMLX_BOUNDS=1), hence the
child process. Stands in for a memory checker (the reference relies on Metal's validation layer and
its ``tracked_hazards`` feature, crates/rmlx-metal/src/device.rs:23-32)."""
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu

CHILD = r'''
import torch
from rmlx_b200 import _lib
from rmlx_b200.ops import decode as D
from rmlx_b200.ops.weights import LinearWeight

dev = torch.device("cuda:0")
hq, hkv, hd, K, page, max_blocks = 4, 2, 64, 256, 16, 4
g = torch.Generator(device=dev).manual_seed(0)
w = LinearWeight.random((hq + 2 * hkv) * hd, K, None, dev, generator=g)
x = torch.randn(1, K, device=dev, generator=g).to(torch.bfloat16)
norm = torch.ones(K, dtype=torch.bfloat16, device=dev)
kc = torch.zeros(8, hkv, page, hd, dtype=torch.bfloat16, device=dev)
vc = torch.zeros_like(kc)
bt = torch.tensor([[1, 2, 3, 4]], dtype=torch.int32, device=dev)
ang = torch.arange(256, device=dev, dtype=torch.float32)[:, None] * torch.arange(hd // 2, device=dev)[None, :] * 0.01
cos, sin = ang.cos().contiguous(), ang.sin().contiguous()
q = torch.empty(1, hq, hd, dtype=torch.bfloat16, device=dev)
pos_ok = torch.tensor([5], dtype=torch.int32, device=dev)
pos_bad = torch.tensor([70], dtype=torch.int32, device=dev)      # block column 4 of a 4-column table

D.set_stream(True, ops="all")
assert _lib.cuda().rmlx_bounds_build() == 1
assert _lib.bounds_status() is None

def qkv(pos):
    D.rms_qkv_rope(x, w, norm, 1e-6, q, kc, vc, bt, pos, cos, sin, hq, hkv)
    torch.cuda.synchronize()

qkv(pos_ok)
assert _lib.bounds_status() is None and float(kc[1, :, 5].abs().sum()) > 0
kc.zero_(); vc.zero_()
qkv(pos_bad)
rec = _lib.bounds_status()
assert rec is not None and rec[0] == "decode_stream.cu" and rec[2:] == (4, 4), rec
assert float(kc.abs().sum()) == 0 and float(vc.abs().sum()) == 0      # the append was skipped
assert _lib.bounds_status() is None                                   # reading clears the record
D.set_stream(False)
qkv(pos_bad)
rec = _lib.bounds_status()
assert rec is not None and rec[0] == "decode_qkv_rope.cu" and rec[2:] == (4, 4), rec
assert float(kc.abs().sum()) == 0
D.set_stream(True, ops="all")

flat = torch.randn(1, (hq + 2 * hkv) * hd, device=dev, generator=g).to(torch.bfloat16)
D.rope_kv_write(flat, q, kc, vc, bt, pos_bad, cos, sin, hq, hkv)
torch.cuda.synchronize()
rec = _lib.bounds_status()
assert rec is not None and rec[0] == "rope_kv.cu" and rec[2:] == (4, 4), rec
assert float(kc.abs().sum()) == 0

# attention over 80 tokens with a 64-token table: the fifth page is read from the reserved page 0
lens = torch.tensor([80], dtype=torch.int32, device=dev)
out = D.flash_decode_paged(q, kc, vc, bt, lens)
torch.cuda.synchronize()
rec = _lib.bounds_status()
assert rec is not None and rec[0] in ("flash_decode.cu", "flash_decode_cluster.cu") and rec[2:] == (4, 4), rec
assert torch.isfinite(out.float()).all()

table = torch.randn(32, 64, device=dev, generator=g).to(torch.bfloat16)
D.embedding(table, torch.tensor([40], dtype=torch.int32, device=dev))
torch.cuda.synchronize()
rec = _lib.bounds_status()
assert rec is not None and rec[0] == "misc.cu" and rec[2:] == (40, 32), rec

# and a clean call leaves no record
qkv(pos_ok)
assert _lib.bounds_status() is None
print("BOUNDS-OK")
'''


def test_bounds_checked_build_records_and_skips(dev):
    from rmlx_b200 import _build
    if not _build.CUDA_BOUNDS_LIB.exists():
        _build.build(kinds=("cuda_bounds",))
    env = dict(os.environ, RMLX_BOUNDS="1")
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    proc = subprocess.run([sys.executable, "-c", CHILD], env=env, cwd=root, capture_output=True,
                          text=True, timeout=300)
    assert proc.returncode == 0 and "BOUNDS-OK" in proc.stdout, proc.stdout + proc.stderr


def test_normal_build_has_no_bounds_records(dev):
    from rmlx_b200 import _lib
    assert _lib.cuda().rmlx_bounds_build() == 0
    with pytest.raises(_lib.NativeError):
        _lib.bounds_status()

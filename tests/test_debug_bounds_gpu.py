"""The ``-DOSLO_DEBUG_BOUNDS`` build (``_C_bounds.so``): data-dependent indices that fall outside their buffer are
skipped or clamped in every build - nothing faults - and the debug build additionally reports them through the device
error word. Each case runs in a child process, because one process can load only one of the two libraries."""
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

_CHILD = r'''
import sys, math, torch
sys.path.insert(0, %(root)r)
import oslo_b200 as ob
from oslo_b200 import ops
from oslo_b200.ops import cuda_ops as co
ext = ops.load_ext(required=True)
assert ops.ext_path().endswith(%(lib)r), ops.ext_path()
dev = "cuda"
codes = []
def code():
    torch.cuda.synchronize()
    c = int(ext.error_word(torch.zeros(1, device=dev)).item())
    co.reset_device_error(torch.zeros(1, device=dev))
    return c
# 1. n-gram blocking with a generated token outside the vocabulary: the in-range bans still happen
vocab = 32
toks = torch.tensor([[5, 7, 5, 7, 5], [3, 40, 3, 40, 3]], device=dev)        # row 1 would ban token 40 >= vocab
lp = torch.zeros(2, vocab, device=dev)
ops.ban_repeated_ngrams(toks, lp, 2)
torch.cuda.synchronize()
assert lp[0, 7] == -math.inf and torch.isfinite(lp[1]).all()
codes.append(code())
# 2. decode attention with a length beyond the cache: clamped to the cache, result finite and equal to the full-cache answer
B, H, T, D = 2, 2, 64, 64
q = torch.randn(B, H, D, device=dev).to(torch.bfloat16)
kc = torch.randn(B, H, T, D, device=dev).to(torch.bfloat16)
vc = torch.randn(B, H, T, D, device=dev).to(torch.bfloat16)
o_bad = ops.decode_attention(q, kc, vc, torch.tensor([T + 9, 10], device=dev, dtype=torch.int32), 0.125, None)
codes.append(code())
o_ok = ops.decode_attention(q, kc, vc, torch.tensor([T, 10], device=dev, dtype=torch.int32), 0.125, None)
assert torch.isfinite(o_bad.float()).all() and torch.equal(o_bad, o_ok)
codes.append(code())
# 3. cache append at a position past the cache: skipped, the cache is untouched
k = torch.randn(B, H * D, device=dev).to(torch.bfloat16)
before = kc.clone()
co.rotary_append(k.clone(), k, k, kc, vc, torch.tensor([3, 3], device=dev, dtype=torch.int32),
                 torch.tensor([T], device=dev), 16)
torch.cuda.synchronize()
assert torch.equal(kc, before)
codes.append(code())
print("CODES", codes)
'''


def _run(debug: bool):
    env = dict(os.environ, OSLO_B200_DEBUG_BOUNDS="1" if debug else "0")
    src = _CHILD % {"root": ROOT, "lib": "_C_bounds.so" if debug else "_C.so"}
    r = subprocess.run([sys.executable, "-c", src], capture_output=True, text=True, timeout=300, env=env)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-3000:]
    line = [l for l in r.stdout.splitlines() if l.startswith("CODES")][-1]
    return eval(line[len("CODES"):])


def test_debug_build_reports_skipped_indices():
    if not os.path.exists(os.path.join(ROOT, "oslo_b200", "_C_bounds.so")):
        pytest.skip("debug build not present (python -m oslo_b200.build --debug-bounds)")
    assert _run(True) == [6, 6, 0, 6]          # ERR_BOUNDS for the three bad inputs, nothing for the good one


def test_release_build_skips_silently():
    assert _run(False) == [0, 0, 0, 0]

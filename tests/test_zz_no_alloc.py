"""The allocation-free column-statistics entry point (`oc_colstats_static`).

Some users of the library cannot give it a workspace and cannot let it allocate:
a serving process that reserved the whole GPU for its own arena at start-up, or a
plugin that is handed raw device pointers and nothing else.  For them the
per-block partial sums live in a fixed array inside the library.  This test calls
that entry point through the C ABI twice in a row (the second call finds the first
call's partials still in the array) and checks both results against the regular
`oc_colstats`, which takes a caller-provided workspace.  It is collected last so
that a failure here cannot hide another test's result.
"""
import numpy as np
import pytest
import torch

import ocnn_pytorch_b200 as b200

pytestmark = pytest.mark.gpu
L = b200._lib


def _regular(a, b):
  n, C = a.shape
  s1 = torch.empty(C, dtype=torch.float32, device=a.device)
  s2 = torch.empty(C, dtype=torch.float32, device=a.device)
  ws = L.workspace(L.lib().oc_colstats_workspace_bytes(n, C), a.device)
  L.call('oc_colstats', L.ptr(a), L.ptr(b), n, C, L.dtype_code(a.dtype), L.ptr(s1), L.ptr(s2), L.ptr(ws),
         ws.numel(), L.stream(a.device))
  return s1, s2


def _static(a, b):
  n, C = a.shape
  s1 = torch.full((C,), float('nan'), dtype=torch.float32, device=a.device)
  s2 = torch.full((C,), float('nan'), dtype=torch.float32, device=a.device)
  L.call('oc_colstats_static', L.ptr(a), L.ptr(b), n, C, L.dtype_code(a.dtype), L.ptr(s1), L.ptr(s2),
         L.stream(a.device))
  return s1, s2


def _close(x, y):
  # same tolerance as the fp32 parity tests: 1e-4 relative (L2 and max-norm)
  x, y = x.double().cpu().numpy(), y.double().cpu().numpy()
  return (np.linalg.norm(x - y) <= 1e-4 * max(np.linalg.norm(y), 1e-30) and
          np.abs(x - y).max() <= 1e-4 * max(np.abs(y).max(), 1e-30))


def test_static_scratch_matches_workspace_variant_twice_in_a_row():
  dev = torch.device('cuda', 0)
  g = torch.Generator(device=dev).manual_seed(11)
  cases = [(200000, 64, torch.float32), (50001, 96, torch.float16), (3000, 4096, torch.bfloat16), (7, 5, torch.float32)]
  for n, C, dtype in cases:
    a1 = (torch.randn(n, C, device=dev, generator=g) * 2 + 0.5).to(dtype)
    b1 = torch.randn(n, C, device=dev, generator=g).to(dtype)
    a2 = (torch.randn(n, C, device=dev, generator=g) * 3 - 1.0).to(dtype)
    # first call: sum a, sum a*b
    e1, e2 = _regular(a1, b1)
    s1, s2 = _static(a1, b1)
    # second call right behind it, other data and b omitted (sum a, sum a*a)
    f1, f2 = _regular(a2, None)
    t1, t2 = _static(a2, None)
    torch.cuda.synchronize()
    assert _close(s1, e1) and _close(s2, e2), (n, C, dtype, 'first call')
    assert _close(t1, f1) and _close(t2, f2), (n, C, dtype, 'second call')
  # empty input gives zeros, a channel count past the limit is refused with a clear message
  z1, z2 = _static(torch.empty(0, 8, device=dev), None)
  assert float(z1.abs().sum()) == 0.0 and float(z2.abs().sum()) == 0.0
  big = torch.zeros(2, 4097, device=dev)
  with pytest.raises(L.OctConvError, match='4096'):
    _static(big, None)

"""Morton ("shuffled") keys: same functions and conventions as the reference's
ocnn/octree/shuffled_key.py:60-115, computed by the `oc_xyz2key` / `oc_key2xyz`
kernels (bit arithmetic, no look-up tables)."""
from typing import Optional, Union

import torch

from .. import _lib

_COORD_CODES = {torch.int64: _lib.OC_I64, torch.int32: _lib.OC_I32, torch.int16: _lib.OC_I16,
                torch.float32: _lib.OC_COORD_F32, torch.float64: _lib.OC_COORD_F64}


def xyz2key(x: torch.Tensor, y: torch.Tensor, z: torch.Tensor,
            b: Optional[Union[torch.Tensor, int]] = None, depth: int = 16):
  r''' Encodes :attr:`x`, :attr:`y`, :attr:`z` (and the batch index :attr:`b`)
  into int64 shuffled keys, ``key = (b << 48) | interleave(x, y, z)``.

  Values are truncated toward zero like ``.long()`` and masked to
  :attr:`depth` bits, exactly as the reference does (shuffled_key.py:76-90).
  '''
  _lib.require_cuda(x, y, z)
  if x.dtype not in _COORD_CODES:
    x, y, z = x.long(), y.long(), z.long()
  x, y, z = x.contiguous(), y.contiguous(), z.contiguous()
  assert x.shape == y.shape == z.shape and y.dtype == x.dtype and z.dtype == x.dtype
  bt = None
  if isinstance(b, torch.Tensor):
    bt = b.to(x.dtype).contiguous()
    assert bt.shape == x.shape
  key = torch.empty(x.shape, dtype=torch.int64, device=x.device)
  _lib.call('oc_xyz2key', _lib.ptr(x), _lib.ptr(y), _lib.ptr(z), _lib.ptr(bt),
            _COORD_CODES[x.dtype], x.numel(), depth, _lib.ptr(key), _lib.stream(x.device))
  if b is not None and bt is None:
    key = (int(b) << 48) | key
  return key


def key2xyz(key: torch.Tensor, depth: int = 16):
  r''' Decodes shuffled keys into ``(x, y, z, b)`` int64 tensors
  (shuffled_key.py:93-115). '''
  _lib.require_cuda(key)
  key = key.contiguous()
  assert key.dtype == torch.int64
  x, y, z, b = (torch.empty_like(key) for _ in range(4))
  _lib.call('oc_key2xyz', _lib.ptr(key), key.numel(), depth, _lib.ptr(x), _lib.ptr(y), _lib.ptr(z),
            _lib.ptr(b), _lib.stream(key.device))
  return x, y, z, b

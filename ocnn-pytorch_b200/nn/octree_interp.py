"""Nearest-neighbour octree upsampling (ocnn/nn/octree_interp.py:140-200):
depad -> repeat x8 -> depad fused into one gather kernel, with its gradient.
Point interpolation (octree_nearest_pts / octree_linear_pts) is not part of
this package."""
from typing import Optional

import torch
from torch.autograd import Function

from .. import _lib


class _UpsampleFunction(Function):

  @staticmethod
  def forward(ctx, data, octree, depth, nempty):
    data = data.contiguous()
    C = data.shape[1]
    if nempty:
      idx_c, idx_f = None, octree.nempty_index(depth + 1)
      n_out = int(octree.nnum_nempty[depth + 1])
    else:
      idx_c, idx_f = octree.nempty_index(depth), None
      n_out = int(octree.nnum[depth + 1])
    out = torch.empty(n_out, C, dtype=data.dtype, device=data.device)
    _lib.call('oc_upsample_fwd', _lib.ptr(data), _lib.ptr(idx_c), _lib.ptr(idx_f), n_out, C,
              _lib.dtype_code(data.dtype), _lib.ptr(out), _lib.stream(data.device))
    ctx.conf = (octree, depth, nempty, data.shape[0])
    return out

  @staticmethod
  def backward(ctx, grad):
    octree, depth, nempty, n_in = ctx.conf
    grad = grad.contiguous()
    C = grad.shape[1]
    ch_c = None if nempty else octree.children[depth]
    ch_f = octree.children[depth + 1] if nempty else None
    gin = torch.empty(n_in, C, dtype=grad.dtype, device=grad.device)
    _lib.call('oc_upsample_bwd', _lib.ptr(grad), _lib.ptr(ch_c), _lib.ptr(ch_f), n_in, C,
              _lib.dtype_code(grad.dtype), _lib.ptr(gin), _lib.stream(grad.device))
    return gin, None, None, None


def octree_nearest_upsample(data: torch.Tensor, octree, depth: int, nempty: bool = False):
  r''' Copies the feature of every node of :attr:`depth` to its 8 children. '''
  _lib.require_cuda(data)
  nnum = octree.nnum_nempty[depth] if nempty else octree.nnum[depth]
  assert data.shape[0] == nnum, 'The shape of input data is wrong.'
  return _UpsampleFunction.apply(data, octree, depth, nempty)


class OctreeUpsample(torch.nn.Module):
  r''' Upsamples node features from :attr:`depth` to ``depth + 1``.  Only
  ``method='nearest'`` with ``target_depth == depth + 1`` is provided here. '''

  def __init__(self, method: str = 'linear', nempty: bool = False):
    super().__init__()
    self.method = method
    self.nempty = nempty

  def forward(self, data: torch.Tensor, octree, depth: int, target_depth: Optional[int] = None):
    if target_depth is None:
      target_depth = depth + 1
    if target_depth == depth:
      return data
    assert target_depth >= depth, 'target_depth must be larger than depth'
    if target_depth == depth + 1 and self.method == 'nearest':
      return octree_nearest_upsample(data, octree, depth, self.nempty)
    raise NotImplementedError(
        'OctreeUpsample: only method="nearest" to depth+1 is available in this package')

  def extra_repr(self) -> str:
    return 'method={}, nempty={}'.format(self.method, self.nempty)

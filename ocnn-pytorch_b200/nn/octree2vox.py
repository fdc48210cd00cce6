"""octree2voxel / Octree2Voxel (ocnn/nn/octree2vox.py:13-48): node features scattered into a dense
``(batch, 2^d, 2^d, 2^d, C)`` grid, zeros elsewhere.  Reuses the pad / depad row kernels."""
import torch
from torch.autograd import Function

from .. import _lib


class _ToVoxelFunction(Function):

  @staticmethod
  def forward(ctx, data, index, n_vox):
    data = data.contiguous()
    n, C = data.shape
    out = torch.empty(n_vox, C, dtype=data.dtype, device=data.device)
    _lib.call('oc_pad', _lib.ptr(data), _lib.ptr(index), n, n_vox, C, _lib.dtype_code(data.dtype), 0.0,
              _lib.ptr(out), _lib.stream(data.device))
    ctx.save_for_backward(index)
    return out

  @staticmethod
  def backward(ctx, grad):
    index, = ctx.saved_tensors
    grad = grad.contiguous()
    n, C = index.numel(), grad.shape[1]
    gin = torch.empty(n, C, dtype=grad.dtype, device=grad.device)
    _lib.call('oc_depad', _lib.ptr(grad), _lib.ptr(index), n, C, _lib.dtype_code(grad.dtype), _lib.ptr(gin),
              _lib.stream(grad.device))
    return gin, None, None


def octree2voxel(data: torch.Tensor, octree, depth: int, nempty: bool = False):
  r''' Converts node features at `depth` to the full-voxel representation. '''
  _lib.require_cuda(data)
  x, y, z, b = octree.xyzb(depth, nempty)
  assert data.shape[0] == x.numel(), 'The shape of input data is wrong.'
  num = 1 << depth
  index = (((b * num + x) * num + y) * num + z).contiguous()
  vox = _ToVoxelFunction.apply(data, index, octree.batch_size * num ** 3)
  return vox.view(octree.batch_size, num, num, num, data.shape[1])


class Octree2Voxel(torch.nn.Module):
  r''' See :func:`octree2voxel`. '''

  def __init__(self, nempty: bool = False):
    super().__init__()
    self.nempty = nempty

  def forward(self, data: torch.Tensor, octree, depth: int):
    return octree2voxel(data, octree, depth, self.nempty)

  def extra_repr(self) -> str:
    return 'nempty={}'.format(self.nempty)

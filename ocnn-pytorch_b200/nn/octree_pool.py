"""octree_max_pool / OctreeMaxPool (ocnn/nn/octree_pool.py:17-38, 143-156) and
octree_max_unpool / OctreeMaxUnpool (41-65, 159-171) as fused kernels: the
reference's pad(-inf) -> view(-1,8,C).max -> pad(0) chain is one pass."""
import torch
from torch.autograd import Function

from .. import _lib
from .octree_pad import octree_pad, octree_depad


class _MaxPoolFunction(Function):

  @staticmethod
  def forward(ctx, data, octree, depth, nempty):
    data = data.contiguous()
    C = data.shape[1]
    child_in = octree.children[depth] if nempty else None
    child_out = None if nempty else octree.children[depth - 1]
    n_ne = int(octree.nnum_nempty[depth - 1])
    n_out = n_ne if nempty else int(octree.nnum[depth - 1])
    n_in = int(octree.nnum_nempty[depth] if nempty else octree.nnum[depth])
    assert data.shape[0] == n_in, 'The shape of input data is wrong.'
    out = torch.empty(n_out, C, dtype=data.dtype, device=data.device)
    argmax = torch.empty(n_ne, C, dtype=torch.int64, device=data.device)
    _lib.call('oc_maxpool_fwd', _lib.ptr(data), _lib.ptr(child_in), _lib.ptr(child_out), n_out, C,
              _lib.dtype_code(data.dtype), _lib.ptr(out), _lib.ptr(argmax),
              _lib.stream(data.device))
    ctx.save_for_backward(argmax)
    ctx.conf = (child_in, child_out, n_out, n_in)
    ctx.mark_non_differentiable(argmax)
    return out, argmax

  @staticmethod
  def backward(ctx, grad, _):
    argmax, = ctx.saved_tensors
    child_in, child_out, n_out, n_in = ctx.conf
    grad = grad.contiguous()
    C = grad.shape[1]
    gin = torch.empty(n_in, C, dtype=grad.dtype, device=grad.device)
    _lib.call('oc_maxpool_bwd', _lib.ptr(grad), _lib.ptr(argmax), _lib.ptr(child_in),
              _lib.ptr(child_out), n_out, n_in, C, _lib.dtype_code(grad.dtype), _lib.ptr(gin),
              _lib.stream(grad.device))
    return gin, None, None, None


def octree_max_pool(data: torch.Tensor, octree, depth: int, nempty: bool = False,
                    return_indices: bool = False):
  r''' Max pooling over the 8 siblings (kernel 2, stride 2): depth -> depth-1.
  ``indices`` (int64) is the sibling number of the maximum per non-empty parent. '''
  _lib.require_cuda(data)
  out, indices = _MaxPoolFunction.apply(data, octree, depth, nempty)
  return (out, indices) if return_indices else out


def octree_max_unpool(data: torch.Tensor, indices: torch.Tensor, octree, depth: int,
                      nempty: bool = False):
  r''' Inverse of max pooling (depth -> depth+1): each value goes to the sibling
  recorded in :attr:`indices`, the other siblings are zero. '''
  _lib.require_cuda(data, indices)
  if not nempty:
    data = octree_depad(data, octree, depth)
  num, channel = data.shape
  sib = torch.arange(8, device=data.device, dtype=indices.dtype).view(1, 8, 1)
  out = torch.where(indices.unsqueeze(1) == sib, data.unsqueeze(1), data.new_zeros(()))
  out = out.reshape(num * 8, channel)
  if nempty:
    out = octree_depad(out, octree, depth + 1)
  return out


class OctreeMaxPool(torch.nn.Module):
  r''' Module form of :func:`octree_max_pool`. '''

  def __init__(self, nempty: bool = False, return_indices: bool = False):
    super().__init__()
    self.nempty = nempty
    self.return_indices = return_indices

  def forward(self, data: torch.Tensor, octree, depth: int):
    return octree_max_pool(data, octree, depth, self.nempty, self.return_indices)

  def extra_repr(self) -> str:
    return 'nempty={}'.format(self.nempty)


class OctreeMaxUnpool(torch.nn.Module):
  r''' Module form of :func:`octree_max_unpool`. '''

  def __init__(self, nempty: bool = False):
    super().__init__()
    self.nempty = nempty

  def forward(self, data: torch.Tensor, indices: torch.Tensor, octree, depth: int):
    return octree_max_unpool(data, indices, octree, depth, self.nempty)

  def extra_repr(self) -> str:
    return 'nempty={}'.format(self.nempty)

"""octree_pad / octree_depad with the reference's signatures
(ocnn/nn/octree_pad.py:13-39), as single scatter / gather kernels with autograd."""
import torch
from torch.autograd import Function

from .. import _lib


def _pad(data, index, n_all, val):
  data = data.contiguous()
  out = torch.empty(n_all, data.shape[1], dtype=data.dtype, device=data.device)
  _lib.call('oc_pad', _lib.ptr(data), _lib.ptr(index), data.shape[0], n_all, data.shape[1],
            _lib.dtype_code(data.dtype), float(val), _lib.ptr(out), _lib.stream(data.device))
  return out


def _depad(data, index):
  data = data.contiguous()
  out = torch.empty(index.numel(), data.shape[1], dtype=data.dtype, device=data.device)
  _lib.call('oc_depad', _lib.ptr(data), _lib.ptr(index), index.numel(), data.shape[1],
            _lib.dtype_code(data.dtype), _lib.ptr(out), _lib.stream(data.device))
  return out


class _PadFunction(Function):

  @staticmethod
  def forward(ctx, data, index, n_all, val):
    ctx.save_for_backward(index)
    return _pad(data, index, n_all, val)

  @staticmethod
  def backward(ctx, grad):
    index, = ctx.saved_tensors
    return _depad(grad, index), None, None, None


class _DepadFunction(Function):

  @staticmethod
  def forward(ctx, data, index):
    ctx.save_for_backward(index)
    ctx.n_all = data.shape[0]
    return _depad(data, index)

  @staticmethod
  def backward(ctx, grad):
    index, = ctx.saved_tensors
    return _pad(grad, index, ctx.n_all, 0.0), None


def octree_pad(data: torch.Tensor, octree, depth: int, val: float = 0.0):
  r''' Expands features of the non-empty nodes to all nodes of :attr:`depth`,
  filling the empty ones with :attr:`val`. '''
  _lib.require_cuda(data)
  assert data.dim() == 2
  index = octree.nempty_index(depth)
  assert data.shape[0] == index.numel(), 'The shape of input data is wrong.'
  return _PadFunction.apply(data, index, int(octree.nnum[depth]), val)


def octree_depad(data: torch.Tensor, octree, depth: int):
  r''' Keeps only the rows of the non-empty nodes of :attr:`depth`. '''
  _lib.require_cuda(data)
  assert data.dim() == 2
  assert data.shape[0] == int(octree.nnum[depth]), 'The shape of input data is wrong.'
  return _DepadFunction.apply(data, octree.nempty_index(depth))

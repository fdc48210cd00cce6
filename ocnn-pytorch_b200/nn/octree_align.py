"""search_value / octree_align (ocnn/nn/octree_align.py:13-48): features of one octree looked up
at the nodes of another by shuffled key; zeros where the other octree has no such node."""
import torch
from torch.autograd import Function

from .. import _lib


class _AlignFunction(Function):

  @staticmethod
  def forward(ctx, value, idx):
    value = value.contiguous()
    m, C = idx.numel(), value.shape[1]
    out = torch.empty(m, C, dtype=value.dtype, device=value.device)
    _lib.call('oc_rows_gather', _lib.ptr(value), _lib.ptr(idx), m, C, _lib.dtype_code(value.dtype),
              _lib.ptr(out), _lib.stream(value.device))
    ctx.save_for_backward(idx)
    ctx.conf = (value.shape[0], value.dtype)
    return out.float()                       # the reference fills a float32 tensor

  @staticmethod
  def backward(ctx, grad):
    idx, = ctx.saved_tensors
    n, dtype = ctx.conf
    grad = grad.contiguous()
    C = grad.shape[1]
    acc = torch.zeros(n, C, dtype=torch.float32, device=grad.device)
    _lib.call('oc_rows_scatter_add', _lib.ptr(grad), _lib.ptr(idx), idx.numel(), C,
              _lib.dtype_code(grad.dtype), _lib.ptr(acc), _lib.stream(grad.device))
    return acc.to(dtype), None


def search_value(value: torch.Tensor, key: torch.Tensor, query: torch.Tensor):
  r''' Rows of `value` (one per sorted shuffled key in `key`) at the keys `query`. '''
  _lib.require_cuda(value, key, query)
  key = key.contiguous()
  query = query.long().contiguous()
  idx = torch.empty_like(query)
  _lib.call('oc_search_key', _lib.ptr(key), key.numel(), _lib.ptr(query), query.numel(), _lib.ptr(idx),
            _lib.stream(value.device))
  return _AlignFunction.apply(value, idx)


def octree_align(value: torch.Tensor, octree, octree_query, depth: int, nempty: bool = False):
  r''' :func:`search_value` with the keys of two octrees at `depth`. '''
  key = octree.key(depth, nempty)
  query = octree_query.key(depth, nempty)
  assert key.shape[0] == value.shape[0]
  return search_value(value, key, query)

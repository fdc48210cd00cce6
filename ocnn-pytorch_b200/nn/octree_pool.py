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


def _idx_bytes(table):
  return 8 if table.dtype == torch.int64 else 4


class _AvgPoolFunction(Function):
  r''' Mean over the existing entries of each row of a neighbour table
  (ocnn/nn/octree_pool.py:68-103), gradient through the table of the scatter direction. '''

  @staticmethod
  def forward(ctx, data, octree, depth, kernel, stride, nempty):
    data = data.contiguous()
    table, taps = octree.conv_table(depth, kernel, stride, nempty)
    n_out, C = table.shape[0], data.shape[1]
    out = torch.empty(n_out, C, dtype=data.dtype, device=data.device)
    val = torch.empty(n_out, dtype=torch.float32, device=data.device)
    _lib.call('oc_avgpool_fwd', _lib.ptr(data), _lib.ptr(table), _idx_bytes(table), table.shape[1],
              _lib.int_array(taps), len(taps), n_out, C, _lib.dtype_code(data.dtype), _lib.ptr(out),
              _lib.ptr(val), _lib.stream(data.device))
    ctx.save_for_backward(val)
    ctx.conf = (octree, depth, kernel, stride, nempty, data.shape[0])
    return out

  @staticmethod
  def backward(ctx, grad):
    val, = ctx.saved_tensors
    octree, depth, kernel, stride, nempty, n_in = ctx.conf
    grad = grad.contiguous()
    C = grad.shape[1]
    table_t, taps_t = octree.conv_table_transposed(depth, kernel, stride, nempty)
    assert table_t.shape[0] == n_in
    gin = torch.empty(n_in, C, dtype=grad.dtype, device=grad.device)
    _lib.call('oc_avgpool_bwd', _lib.ptr(grad), _lib.ptr(val), _lib.ptr(table_t), _idx_bytes(table_t),
              table_t.shape[1], _lib.int_array(taps_t), len(taps_t), n_in, C,
              _lib.dtype_code(grad.dtype), _lib.ptr(gin), _lib.stream(grad.device))
    return gin, None, None, None, None, None


def octree_avg_pool(data: torch.Tensor, octree, depth: int, kernel: str, stride: int = 2,
                    nempty: bool = False):
  r''' Octree average pooling over the `kernel` neighbourhood with `stride`. '''
  _lib.require_cuda(data)
  nnum = octree.nnum_nempty[depth] if nempty else octree.nnum[depth]
  assert data.shape[0] == nnum, 'The shape of input data is wrong.'
  return _AvgPoolFunction.apply(data, octree, depth, kernel, stride, nempty)


class _GlobalPoolFunction(Function):
  r''' Per-octree mean of the rows (ocnn/nn/octree_pool.py:106-124). '''

  @staticmethod
  def forward(ctx, data, octree, depth, nempty):
    import ctypes
    data = data.contiguous()
    offs = octree.batch_offsets(depth, nempty)
    B, C = octree.batch_size, data.shape[1]
    mean = torch.empty(B, C, dtype=torch.float32, device=data.device)
    L = _lib.lib()
    ws = _lib.workspace(L.oc_global_pool_workspace_bytes(data.shape[0], B, C), data.device)
    h = (ctypes.c_int64 * (B + 1))(*offs)
    _lib.call('oc_global_pool_fwd', _lib.ptr(data), h, B, C, _lib.dtype_code(data.dtype), _lib.ptr(mean),
              _lib.ptr(ws), ws.numel(), _lib.stream(data.device))
    ctx.conf = (offs, data.shape[0], data.dtype)
    return mean.to(data.dtype)

  @staticmethod
  def backward(ctx, grad):
    import ctypes
    offs, n, dtype = ctx.conf
    B, C = grad.shape
    # grad_in[r] = grad[b(r)] / max(count_b, 1): broadcast each octree's row, then scale its segment
    cnt = torch.tensor([max(offs[b + 1] - offs[b], 1) for b in range(B)], dtype=torch.float32)
    inv = (1.0 / cnt).to(grad.device)
    bid = torch.repeat_interleave(torch.arange(B, device=grad.device),
                                  torch.tensor([offs[b + 1] - offs[b] for b in range(B)], device=grad.device))
    rows = torch.empty(n, C, dtype=grad.dtype, device=grad.device)
    g = grad.contiguous()
    _lib.call('oc_rows_gather', _lib.ptr(g), _lib.ptr(bid), n, C, _lib.dtype_code(g.dtype), _lib.ptr(rows),
              _lib.stream(grad.device))
    h = (ctypes.c_int64 * (B + 1))(*offs)
    out = torch.empty_like(rows)
    _lib.call('oc_scale_segments', _lib.ptr(rows), h, B, _lib.ptr(inv), C, _lib.dtype_code(rows.dtype),
              _lib.ptr(out), _lib.stream(grad.device))
    return out.to(dtype), None, None, None


def octree_global_pool(data: torch.Tensor, octree, depth: int, nempty: bool = False):
  r''' Octree global average pooling: one row per octree of the batch. '''
  _lib.require_cuda(data)
  nnum = octree.nnum_nempty[depth] if nempty else octree.nnum[depth]
  assert data.shape[0] == nnum, 'The shape of input data is wrong.'
  return _GlobalPoolFunction.apply(data, octree, depth, nempty)


class OctreeGlobalPool(torch.nn.Module):
  r''' See :func:`octree_global_pool`. '''

  def __init__(self, nempty: bool = False):
    super().__init__()
    self.nempty = nempty

  def forward(self, data: torch.Tensor, octree, depth: int):
    return octree_global_pool(data, octree, depth, self.nempty)

  def extra_repr(self) -> str:
    return 'nempty={}'.format(self.nempty)


class OctreeAvgPool(torch.nn.Module):
  r''' See :func:`octree_avg_pool`. '''

  def __init__(self, kernel_size, stride: int, nempty: bool = False):
    super().__init__()
    from ..utils import resize_with_last_val, list2str
    self.kernel_size = resize_with_last_val(kernel_size)
    self.kernel = list2str(self.kernel_size)
    self.stride = stride
    self.nempty = nempty

  def forward(self, data: torch.Tensor, octree, depth: int):
    return octree_avg_pool(data, octree, depth, self.kernel, self.stride, self.nempty)

  def extra_repr(self) -> str:
    return 'kernel_size={}, stride={}, nempty={}'.format(self.kernel_size, self.stride, self.nempty)

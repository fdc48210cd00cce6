"""Point interpolation on an octree level (ocnn/nn/octree_interp.py:16-137:
octree_nearest_pts, octree_linear_pts, OctreeInterp) and nearest-neighbour octree
upsampling (:140-200, depad -> repeat x8 -> depad fused into one gather kernel), with
their gradients with respect to the features."""
from typing import Optional, Union

import torch
from torch.autograd import Function

from .. import _lib


def _search_xyzb(octree, pts, depth, nempty):
  return octree.search_xyzb(pts, depth, nempty)


class _NearestPtsFunction(Function):
  r''' out[p] = data[idx[p]] (0 where idx < 0); the gradient is accumulated in fp32. '''

  @staticmethod
  def forward(ctx, data, idx):
    data = data.contiguous()
    m, C = idx.numel(), data.shape[1]
    out = torch.empty(m, C, dtype=data.dtype, device=data.device)
    _lib.call('oc_rows_gather', _lib.ptr(data), _lib.ptr(idx), m, C, _lib.dtype_code(data.dtype),
              _lib.ptr(out), _lib.stream(data.device))
    ctx.save_for_backward(idx)
    ctx.conf = (data.shape[0], data.dtype)
    return out

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


class _LinearPtsFunction(Function):
  r''' Weighted mean of the existing corners (idx8, w8 from ``oc_interp_corners``). '''

  @staticmethod
  def forward(ctx, data, idx8, w8):
    data = data.contiguous()
    m, C = idx8.shape[0], data.shape[1]
    out = torch.empty(m, C, dtype=data.dtype, device=data.device)
    _lib.call('oc_interp_linear_fwd', _lib.ptr(data), _lib.ptr(idx8), _lib.ptr(w8), m, C,
              _lib.dtype_code(data.dtype), _lib.ptr(out), _lib.stream(data.device))
    ctx.save_for_backward(idx8, w8)
    ctx.conf = (data.shape[0], data.dtype)
    return out

  @staticmethod
  def backward(ctx, grad):
    idx8, w8 = ctx.saved_tensors
    n, dtype = ctx.conf
    grad = grad.contiguous()
    C = grad.shape[1]
    acc = torch.zeros(n, C, dtype=torch.float32, device=grad.device)
    _lib.call('oc_interp_linear_bwd', _lib.ptr(grad), _lib.ptr(idx8), _lib.ptr(w8), idx8.shape[0], C,
              _lib.dtype_code(grad.dtype), _lib.ptr(acc), _lib.stream(grad.device))
    return acc.to(dtype), None, None


def octree_nearest_pts(data: torch.Tensor, octree, depth: int, pts: torch.Tensor,
                       nempty: bool = False, bound_check: bool = False):
  r''' Nearest-neighbour interpolation: the feature of the node that contains each point
  ``pts (N, 4) = (x, y, z, batch)``, coordinates scaled to ``[0, 2^depth)``; zero where there
  is no such node (octree_interp.py:16-48). '''
  _lib.require_cuda(data, pts)
  nnum = octree.nnum_nempty[depth] if nempty else octree.nnum[depth]
  assert data.shape[0] == nnum, 'The shape of input data is wrong.'
  idx = _search_xyzb(octree, pts, depth, nempty)
  if bound_check:
    bound = torch.logical_and(pts[:, :3] >= 0, pts[:, :3] < 2 ** depth).all(1)
    idx = torch.where(bound, idx, torch.full_like(idx, -1))
  return _NearestPtsFunction.apply(data, idx)


def octree_linear_pts(data: torch.Tensor, octree, depth: int, pts: torch.Tensor,
                      nempty: bool = False, bound_check: bool = False):
  r''' Linear interpolation between the 8 cell centres around each point, normalised by the
  weights of the cells that exist (octree_interp.py:51-98).  Differentiable in `data` only. '''
  _lib.require_cuda(data, pts)
  nnum = octree.nnum_nempty[depth] if nempty else octree.nnum[depth]
  assert data.shape[0] == nnum, 'The shape of input data is wrong.'
  key = octree.key(depth, nempty).contiguous()
  p = pts.detach().float().contiguous()
  m = p.shape[0]
  idx8 = torch.empty(m, 8, dtype=torch.int64, device=data.device)
  w8 = torch.empty(m, 8, dtype=torch.float32, device=data.device)
  _lib.call('oc_interp_corners', _lib.ptr(key), key.numel(), _lib.ptr(p), m, depth, int(bound_check),
            _lib.ptr(idx8), _lib.ptr(w8), _lib.stream(data.device))
  return _LinearPtsFunction.apply(data, idx8, w8)


class OctreeInterp(torch.nn.Module):
  r''' Interpolates octree features at points (octree_interp.py:101-137).  With
  `rescale_pts` the points are mapped from ``[bbmin, bbmax]`` to ``[0, 2^depth]`` in place,
  as the reference does. '''

  def __init__(self, method: str = 'linear', nempty: bool = False, bound_check: bool = False,
               rescale_pts: bool = True):
    super().__init__()
    self.method = method
    self.nempty = nempty
    self.bound_check = bound_check
    self.rescale_pts = rescale_pts
    self.func = octree_linear_pts if method == 'linear' else octree_nearest_pts

  def forward(self, data: torch.Tensor, octree, depth: int, pts: torch.Tensor,
              bbmin: Union[torch.Tensor, float] = -1, bbmax: Union[torch.Tensor, float] = 1):
    if self.rescale_pts:
      box_size = bbmax - bbmin
      if type(box_size) is torch.Tensor:
        box_size = box_size.max().item()
      assert box_size > 0, 'The bounding box size must be greater than 0.'
      pts[:, :3] = (pts[:, :3] - bbmin) * (2 ** depth / box_size)
    return self.func(data, octree, depth, pts, self.nempty, self.bound_check)

  def extra_repr(self) -> str:
    return 'method={}, nempty={}, bound_check={}, rescale_pts={}'.format(
        self.method, self.nempty, self.bound_check, self.rescale_pts)


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

"""OctreeDropPath (ocnn/nn/octree_drop.py:14-60): stochastic depth per octree of the batch."""
import ctypes
from typing import Optional

import torch
from torch.autograd import Function

from .. import _lib


class _ScaleSegments(Function):
  r''' out[r] = data[r] * scale[octree of r]; the gradient is the same map. '''

  @staticmethod
  def forward(ctx, data, scale, offsets):
    data = data.contiguous()
    B, C = len(offsets) - 1, data.shape[1]
    out = torch.empty_like(data)
    h = (ctypes.c_int64 * (B + 1))(*offsets)
    _lib.call('oc_scale_segments', _lib.ptr(data), h, B, _lib.ptr(scale), C, _lib.dtype_code(data.dtype),
              _lib.ptr(out), _lib.stream(data.device))
    ctx.save_for_backward(scale)
    ctx.offsets = offsets
    return out

  @staticmethod
  def backward(ctx, grad):
    scale, = ctx.saved_tensors
    return _ScaleSegments.apply(grad, scale, ctx.offsets), None, None


class OctreeDropPath(torch.nn.Module):
  r''' Drops the whole residual branch of an octree with probability `drop_prob` (training only)
  and, with `scale_by_keep`, divides the kept ones by the keep probability.  The mask is drawn
  with the same call as the reference (``bernoulli_`` on a ``(batch_size, 1)`` tensor).  The
  optional `batch_id` argument of the reference is accepted and ignored: rows of one octree are
  contiguous, the row ranges come from the octree. '''

  def __init__(self, drop_prob: float = 0.0, nempty: bool = False, scale_by_keep: bool = True):
    super().__init__()
    self.drop_prob = drop_prob
    self.nempty = nempty
    self.scale_by_keep = scale_by_keep

  def forward(self, data: torch.Tensor, octree, depth: int, batch_id: Optional[torch.Tensor] = None):
    if self.drop_prob <= 0.0 or not self.training:
      return data
    _lib.require_cuda(data)
    keep_prob = 1 - self.drop_prob
    rnd = data.new_empty(octree.batch_size, 1).bernoulli_(keep_prob)
    if keep_prob > 0.0 and self.scale_by_keep:
      rnd.div_(keep_prob)
    self.last_mask = rnd                      # kept for inspection (tests)
    scale = rnd.float().view(-1).contiguous()
    return _ScaleSegments.apply(data, scale, octree.batch_offsets(depth, self.nempty))

  def extra_repr(self) -> str:
    return 'drop_prob={:.4f}, nempty={}, scale_by_keep={}'.format(self.drop_prob, self.nempty, self.scale_by_keep)


DropPath = OctreeDropPath

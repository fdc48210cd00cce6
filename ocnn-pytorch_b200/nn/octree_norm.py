"""OctreeBatchNorm / OctreeGroupNorm / OctreeInstanceNorm / OctreeNorm with the
reference's signatures (ocnn/nn/octree_norm.py:16-126).

BatchNorm follows torch.nn.BatchNorm1d semantics (biased variance for the
normalisation, unbiased for the running estimate, momentum 0.1, eps 1e-5) on
liboctconv column-statistics kernels.  With ``process_group`` set (or after
`convert_sync_batchnorm`) the per-channel sums are all-reduced across ranks, the
only cross-GPU exchange of a data-parallel octree network."""
from typing import Optional

import torch
import torch.distributed as dist
from torch.autograd import Function

from .. import _lib


def col_stats(a: torch.Tensor, b: Optional[torch.Tensor] = None):
  r''' fp32 ``(sum_n a[n,c], sum_n a[n,c]*b[n,c])`` (``b = a`` when omitted). '''
  _lib.require_cuda(a)
  a = a.contiguous()
  if b is not None:
    b = b.contiguous()
  n, C = a.shape
  s1 = torch.empty(C, dtype=torch.float32, device=a.device)
  s2 = torch.empty(C, dtype=torch.float32, device=a.device)
  ws = _lib.workspace(_lib.lib().oc_colstats_workspace_bytes(n, C), a.device)
  _lib.call('oc_colstats', _lib.ptr(a), _lib.ptr(b), n, C, _lib.dtype_code(a.dtype), _lib.ptr(s1),
            _lib.ptr(s2), _lib.ptr(ws), ws.numel(), _lib.stream(a.device))
  return s1, s2


def _affine(x, scale, shift):
  out = torch.empty_like(x)
  _lib.call('oc_affine_cols', _lib.ptr(x), _lib.ptr(scale), _lib.ptr(shift), x.shape[0],
            x.shape[1], _lib.dtype_code(x.dtype), _lib.ptr(out), _lib.stream(x.device))
  return out


def _all_reduce(t, group):
  if group is not None and dist.is_available() and dist.is_initialized() and \
      dist.get_world_size(group) > 1:
    dist.all_reduce(t, op=dist.ReduceOp.SUM, group=group)
  return t


class _BatchNormTrain(Function):

  @staticmethod
  def forward(ctx, x, weight, bias, eps, group):
    x = x.contiguous()
    C = x.shape[1]
    s1, s2 = col_stats(x)
    packed = torch.cat([s1, s2, s1.new_tensor([float(x.shape[0])])])
    packed = _all_reduce(packed, group)
    count = packed[2 * C]
    mean = packed[:C] / count
    var = (packed[C:2 * C] / count - mean * mean).clamp_(min=0)
    invstd = torch.rsqrt(var + eps)
    w = weight.float() if weight is not None else torch.ones_like(mean)
    b = bias.float() if bias is not None else torch.zeros_like(mean)
    scale = (w * invstd).contiguous()
    shift = (b - mean * scale).contiguous()
    out = _affine(x, scale, shift)
    ctx.save_for_backward(x, w, mean, invstd, count)
    ctx.group = group
    ctx.has_affine = (weight is not None, bias is not None)
    ctx.mark_non_differentiable(mean, var, count)
    return out, mean, var, count

  @staticmethod
  def backward(ctx, grad, _gm, _gv, _gc):
    x, w, mean, invstd, count = ctx.saved_tensors
    grad = grad.contiguous()
    C = x.shape[1]
    sg, sgx = col_stats(grad, x)
    packed = _all_reduce(torch.cat([sg, sgx]), ctx.group)
    sg_all, sgx_all = packed[:C], packed[C:]
    # xhat = (x - mean) * invstd;  dx = w*invstd * (g - mean_g - xhat * mean_gxhat)
    sum_gxhat = (sgx_all - mean * sg_all) * invstd
    k = w * invstd
    ka = k.contiguous()
    kb = (-k * invstd * sum_gxhat / count).contiguous()
    kc = (-k * sg_all / count - kb * mean).contiguous()
    gin = None
    if ctx.needs_input_grad[0]:
      gin = torch.empty_like(x)
      _lib.call('oc_bn_bwd_apply', _lib.ptr(grad), _lib.ptr(x), _lib.ptr(ka), _lib.ptr(kb),
                _lib.ptr(kc), x.shape[0], C, _lib.dtype_code(x.dtype), _lib.ptr(gin),
                _lib.stream(x.device))
    # parameter gradients are local sums; DDP averages them like any other parameter
    gw = ((sgx - mean * sg) * invstd) if ctx.has_affine[0] else None
    gb = sg.clone() if ctx.has_affine[1] else None
    return gin, gw, gb, None, None


class OctreeBatchNorm(torch.nn.Module):
  r''' Batch normalisation over the rows of ``(N, C)`` octree features, with the
  parameters, buffers and state_dict keys of ``torch.nn.BatchNorm1d``. '''

  def __init__(self, num_features: int, eps: float = 1e-5, momentum: float = 0.1,
               affine: bool = True, track_running_stats: bool = True, process_group=None):
    super().__init__()
    self.num_features = num_features
    self.eps = eps
    self.momentum = momentum
    self.affine = affine
    self.track_running_stats = track_running_stats
    self.process_group = process_group
    if affine:
      self.weight = torch.nn.Parameter(torch.ones(num_features))
      self.bias = torch.nn.Parameter(torch.zeros(num_features))
    else:
      self.register_parameter('weight', None)
      self.register_parameter('bias', None)
    if track_running_stats:
      self.register_buffer('running_mean', torch.zeros(num_features))
      self.register_buffer('running_var', torch.ones(num_features))
      self.register_buffer('num_batches_tracked', torch.tensor(0, dtype=torch.long))
    else:
      self.register_buffer('running_mean', None)
      self.register_buffer('running_var', None)
      self.register_buffer('num_batches_tracked', None)

  def forward(self, x: torch.Tensor, octree=None, depth=None):
    _lib.require_cuda(x)
    assert x.dim() == 2 and x.shape[1] == self.num_features
    use_batch = self.training or not self.track_running_stats
    if use_batch:
      out, mean, var, count = _BatchNormTrain.apply(x, self.weight, self.bias, self.eps,
                                                    self.process_group)
      if self.training and self.track_running_stats:
        with torch.no_grad():
          self.num_batches_tracked += 1
          m = self.momentum if self.momentum is not None else 1.0 / float(self.num_batches_tracked)
          unbiased = var * (count / (count - 1).clamp(min=1))
          self.running_mean.mul_(1 - m).add_(mean.to(self.running_mean.dtype), alpha=m)
          self.running_var.mul_(1 - m).add_(unbiased.to(self.running_var.dtype), alpha=m)
      return out
    invstd = torch.rsqrt(self.running_var.float() + self.eps)
    w = self.weight.float() if self.weight is not None else torch.ones_like(invstd)
    b = self.bias.float() if self.bias is not None else torch.zeros_like(invstd)
    scale = (w * invstd).contiguous()
    shift = (b - self.running_mean.float() * scale).contiguous()
    return _EvalAffine.apply(x.contiguous(), scale, shift)


class _EvalAffine(Function):

  @staticmethod
  def forward(ctx, x, scale, shift):
    ctx.save_for_backward(scale)
    return _affine(x, scale, shift)

  @staticmethod
  def backward(ctx, grad):
    scale, = ctx.saved_tensors
    return _affine(grad.contiguous(), scale, torch.zeros_like(scale)), None, None


def convert_sync_batchnorm(module: torch.nn.Module, process_group=None):
  r''' Sets ``process_group`` on every OctreeBatchNorm of :attr:`module` so their
  statistics are reduced over the data-parallel ranks. '''
  group = process_group if process_group is not None else dist.group.WORLD
  for m in module.modules():
    if isinstance(m, OctreeBatchNorm):
      m.process_group = group
  return module


class _GroupNormFunction(Function):

  @staticmethod
  def forward(ctx, x, weight, bias, offsets, groups, eps):
    x = x.contiguous()
    B, C = len(offsets) - 1, x.shape[1]
    w = weight.float().contiguous().view(-1)
    b = bias.float().contiguous().view(-1)
    out = torch.empty_like(x)
    mean = torch.empty(B * groups, dtype=torch.float32, device=x.device)
    inv_std = torch.empty(B * groups, dtype=torch.float32, device=x.device)
    ws = _lib.workspace(_lib.lib().oc_gn_workspace_bytes(B, C), x.device)
    _lib.call('oc_gn_fwd', _lib.ptr(x), _lib.i64_array(offsets), B, C, groups, eps, _lib.ptr(w),
              _lib.ptr(b), _lib.dtype_code(x.dtype), _lib.ptr(out), _lib.ptr(mean),
              _lib.ptr(inv_std), _lib.ptr(ws), ws.numel(), _lib.stream(x.device))
    ctx.save_for_backward(x, w, mean, inv_std)
    ctx.conf = (offsets, groups, eps, weight.shape, bias.shape, weight.dtype, bias.dtype)
    return out

  @staticmethod
  def backward(ctx, grad):
    x, w, mean, inv_std = ctx.saved_tensors
    offsets, groups, eps, wshape, bshape, wdt, bdt = ctx.conf
    grad = grad.contiguous()
    B, C = len(offsets) - 1, x.shape[1]
    gin = torch.empty_like(x) if ctx.needs_input_grad[0] else None
    gw = torch.empty(C, dtype=torch.float32, device=x.device)
    gb = torch.empty(C, dtype=torch.float32, device=x.device)
    ws = _lib.workspace(_lib.lib().oc_gn_workspace_bytes(B, C), x.device)
    _lib.call('oc_gn_bwd', _lib.ptr(grad), _lib.ptr(x), _lib.i64_array(offsets), B, C, groups, eps,
              _lib.ptr(w), _lib.ptr(mean), _lib.ptr(inv_std), _lib.dtype_code(x.dtype),
              _lib.ptr(gin), _lib.ptr(gw), _lib.ptr(gb), _lib.ptr(ws), ws.numel(),
              _lib.stream(x.device))
    return gin, gw.view(wshape).to(wdt), gb.view(bshape).to(bdt), None, None, None


class OctreeGroupNorm(torch.nn.Module):
  r''' Group normalisation per octree of the batch (octree_norm.py:19-80),
  including the reference's eps placement (added to the element count and to the
  variance). '''

  def __init__(self, in_channels: int, group: int, nempty: bool = False,
               min_group_channels: int = 4):
    super().__init__()
    self.eps = 1e-5
    self.nempty = nempty
    self.group = group
    self.in_channels = in_channels
    self.min_group_channels = min_group_channels
    if self.min_group_channels * self.group > in_channels:
      self.group = in_channels // self.min_group_channels
    assert in_channels % self.group == 0
    self.channels_per_group = in_channels // self.group
    self.weights = torch.nn.Parameter(torch.Tensor(1, in_channels))
    self.bias = torch.nn.Parameter(torch.Tensor(1, in_channels))
    self.reset_parameters()

  def reset_parameters(self):
    torch.nn.init.ones_(self.weights)
    torch.nn.init.zeros_(self.bias)

  def forward(self, data: torch.Tensor, octree, depth: int):
    _lib.require_cuda(data)
    offsets = octree.batch_offsets(depth, bool(self.nempty))
    assert data.shape[0] == offsets[-1], 'The shape of input data is wrong.'
    return _GroupNormFunction.apply(data, self.weights, self.bias, offsets, self.group, self.eps)

  def extra_repr(self) -> str:
    return ('in_channels={}, group={}, nempty={}, min_group_channels={}').format(
        self.in_channels, self.group, self.nempty, self.min_group_channels)


class OctreeInstanceNorm(OctreeGroupNorm):
  r''' Instance normalisation = group normalisation with one channel per group. '''

  def __init__(self, in_channels: int, nempty: bool = False):
    super().__init__(in_channels=in_channels, group=in_channels, nempty=nempty,
                     min_group_channels=1)

  def extra_repr(self) -> str:
    return ('in_channels={}, nempty={}').format(self.in_channels, self.nempty)


class OctreeNorm(torch.nn.Module):
  r''' Wrapper choosing batch / group / instance normalisation (octree_norm.py:95-126).
  Like the reference, ``min_group_channels`` is passed positionally into
  OctreeGroupNorm's third parameter (``nempty``). '''

  def __init__(self, in_channels: int, norm_type: str = 'batch_norm', group: int = 32,
               min_group_channels: int = 4):
    super().__init__()
    self.in_channels = in_channels
    self.norm_type = norm_type
    self.group = group
    self.min_group_channels = min_group_channels
    if self.norm_type == 'batch_norm':
      self.norm = OctreeBatchNorm(in_channels)
    elif self.norm_type == 'group_norm':
      self.norm = OctreeGroupNorm(in_channels, group, min_group_channels)
    elif self.norm_type == 'instance_norm':
      self.norm = OctreeInstanceNorm(in_channels)
    else:
      raise ValueError

  def forward(self, x: torch.Tensor, octree=None, depth: Optional[int] = None):
    if self.norm_type == 'batch_norm':
      return self.norm(x)
    elif self.norm_type in ('group_norm', 'instance_norm'):
      return self.norm(x, octree, depth)
    raise ValueError

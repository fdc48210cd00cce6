"""Module-tree swapper modelled on the reference's `convert_conv_triton`
(ocnn/nn/octree_conv_t.py:139-160): replaces reference `ocnn` operator modules
inside a model by this package's modules, sharing the Parameter objects, so a
model built from `ocnn.models` runs on liboctconv kernels with its weights."""
import torch

from . import nn as _nn


def _swap_one(m: torch.nn.Module):
  name = type(m).__name__
  mod = type(m).__module__
  if not (mod.startswith('ocnn.') or mod.startswith('torch.nn.modules.batchnorm')):
    return None
  if name in ('OctreeConv', 'OctreeConvTriton', 'OctreeDeconv'):
    cls = _nn.OctreeDeconv if name == 'OctreeDeconv' else _nn.OctreeConv
    new = cls(m.in_channels, m.out_channels, m.kernel_size, m.stride, m.nempty,
              use_bias=m.use_bias)
    new.weights = m.weights
    new.bias = m.bias
    return new
  if name == 'OctreeDWConv':
    new = _nn.OctreeDWConv(m.in_channels, m.kernel_size, m.stride, m.nempty, m.use_bias)
    new.weights = m.weights
    if m.use_bias:
      new.bias = m.bias
    return new
  if name == 'BatchNorm1d':
    new = _nn.OctreeBatchNorm(m.num_features, m.eps, m.momentum, m.affine, m.track_running_stats)
    if m.affine:
      new.weight, new.bias = m.weight, m.bias
    if m.track_running_stats:
      new.running_mean, new.running_var = m.running_mean, m.running_var
      new.num_batches_tracked = m.num_batches_tracked
    return new
  if name in ('OctreeGroupNorm', 'OctreeInstanceNorm'):
    new = _nn.OctreeGroupNorm(m.in_channels, m.group, m.nempty, 1)
    new.group, new.channels_per_group = m.group, m.channels_per_group
    new.weights, new.bias = m.weights, m.bias
    return new
  if name == 'OctreeMaxPool':
    return _nn.OctreeMaxPool(m.nempty, m.return_indices)
  if name == 'OctreeUpsample' and getattr(m, 'method', None) == 'nearest':
    return _nn.OctreeUpsample('nearest', m.nempty)
  if name == 'OctreeMaxUnpool':
    return _nn.OctreeMaxUnpool(m.nempty)
  if name == 'OctreeGlobalPool':
    return _nn.OctreeGlobalPool(m.nempty)
  if name == 'OctreeAvgPool':
    return _nn.OctreeAvgPool(m.kernel_size, m.stride, m.nempty)
  if name == 'OctreeInterp':
    return _nn.OctreeInterp(m.method, m.nempty, m.bound_check, m.rescale_pts)
  if name == 'Octree2Voxel':
    return _nn.Octree2Voxel(m.nempty)
  if name in ('OctreeDropPath', 'DropPath'):
    return _nn.OctreeDropPath(m.drop_prob, m.nempty, m.scale_by_keep)
  return None


def convert_octree_ops(module: torch.nn.Module, batchnorm: bool = True) -> torch.nn.Module:
  r''' Recursively replaces reference operator modules in :attr:`module` (in
  place) and returns it.  Parameters and buffers are shared, not copied. '''
  for child_name, child in list(module.named_children()):
    new = _swap_one(child)
    if new is not None and (batchnorm or type(child).__name__ != 'BatchNorm1d'):
      new.train(child.training)
      setattr(module, child_name, new)
    else:
      convert_octree_ops(child, batchnorm)
  return module

"""OctreeDWConv with the reference's signature (ocnn/nn/octree_dwconv.py:162-205)
on the `oc_dwconv_*` kernels: no (N, K, C) buffer, no einsum."""
from typing import List

import torch
from torch.autograd import Function

from .. import _lib
from ..octree import Octree
from ..utils import xavier_uniform_
from .octree_conv import OctreeConvBase, _idx_bytes, _autocast
from .octree_pad import octree_pad


def dwconv_gather(data, weights, table, taps):
  r''' ``out[r, c] = sum_k data[table[r, taps[k]], c] * weights[k, c]``. '''
  _lib.require_cuda(data, weights, table)
  data = data.contiguous()
  K, C = len(taps), data.shape[1]
  w = weights.reshape(K, C).float().contiguous()
  n_out = table.shape[0]
  out = torch.empty(n_out, C, dtype=data.dtype, device=data.device)
  _lib.call('oc_dwconv_fwd', _lib.ptr(data), data.shape[0], _lib.ptr(w), _lib.ptr(table),
            _idx_bytes(table), table.shape[1], _lib.int_array(taps), K, n_out, C,
            _lib.dtype_code(data.dtype), _lib.ptr(out), _lib.stream(data.device))
  return out


def dwconv_wgrad(data, grad_out, table, taps):
  r''' ``gw[k, c] = sum_r data[table[r, taps[k]], c] * grad_out[r, c]`` (fp32). '''
  data, grad_out = data.contiguous(), grad_out.contiguous()
  K, C = len(taps), data.shape[1]
  n_out = table.shape[0]
  gw = torch.empty(K, C, dtype=torch.float32, device=data.device)
  ws = _lib.workspace(_lib.lib().oc_dwconv_wgrad_workspace_bytes(K, C, n_out), data.device)
  _lib.call('oc_dwconv_wgrad', _lib.ptr(data), data.shape[0], _lib.ptr(grad_out), n_out,
            _lib.ptr(table), _idx_bytes(table), table.shape[1], _lib.int_array(taps), K, C,
            _lib.dtype_code(data.dtype), _lib.ptr(gw), _lib.ptr(ws), ws.numel(),
            _lib.stream(data.device))
  return gw


class OctreeDWConvBase(OctreeConvBase):

  def __init__(self, in_channels: int, kernel_size: List[int] = [3], stride: int = 1,
               nempty: bool = False, max_buffer: int = int(2e8)):
    super().__init__(in_channels, in_channels, kernel_size, stride, nempty, max_buffer)
    self.weights_shape = (self.kdim, 1, self.out_channels)

  def is_conv_layer(self): return True


class OctreeDWConvFunction(Function):
  r''' Depth-wise octree convolution with autograd (octree_dwconv.py:121-155). '''

  @staticmethod
  def forward(ctx, data, weights, octree, depth, in_channels, kernel_size=[3, 3, 3], stride=1,
              nempty=False):
    conv = OctreeDWConvBase(in_channels, kernel_size, stride, nempty)
    conv.setup(octree, depth)
    conv.check(data)
    table, taps = octree.conv_table(depth, conv.kernel, stride, nempty)
    out = dwconv_gather(data, weights, table, taps)
    ctx.save_for_backward(data, weights)
    ctx.conf = (octree, depth, conv.kernel, stride, nempty)
    return out

  @staticmethod
  def backward(ctx, grad):
    data, weights = ctx.saved_tensors
    octree, depth, kernel, stride, nempty = ctx.conf
    grad = grad.contiguous()
    grad_in = grad_w = None
    if ctx.needs_input_grad[0]:
      table_t, taps_t = octree.conv_table_transposed(depth, kernel, stride, nempty)
      grad_in = dwconv_gather(grad, weights, table_t, taps_t)
    if ctx.needs_input_grad[1]:
      table, taps = octree.conv_table(depth, kernel, stride, nempty)
      grad_w = dwconv_wgrad(data, grad, table, taps).view(weights.shape).to(weights.dtype)
    return (grad_in, grad_w) + (None,) * 6


def octree_dwconv(data, weights, octree, depth, in_channels, kernel_size=[3, 3, 3], stride=1,
                  nempty=False, max_buffer=int(2e8)):
  return OctreeDWConvFunction.apply(data, weights, octree, depth, in_channels, kernel_size,
                                    stride, nempty)


class OctreeDWConv(OctreeDWConvBase, torch.nn.Module):
  r''' Depth-wise octree convolution; weights ``(K, 1, C)``.  See
  :class:`OctreeConv` for the arguments. '''

  def __init__(self, in_channels: int, kernel_size: List[int] = [3], stride: int = 1,
               nempty: bool = False, use_bias: bool = False, max_buffer: int = int(2e8)):
    super().__init__(in_channels, kernel_size, stride, nempty, max_buffer)
    self.use_bias = use_bias
    self.weights = torch.nn.Parameter(torch.Tensor(*self.weights_shape))
    if self.use_bias:
      self.bias = torch.nn.Parameter(torch.Tensor(in_channels))
    self.reset_parameters()

  def reset_parameters(self):
    xavier_uniform_(self.weights)
    if self.use_bias:
      torch.nn.init.zeros_(self.bias)

  def forward(self, data: torch.Tensor, octree: Octree, depth: int):
    data = _autocast(data)
    out = OctreeDWConvFunction.apply(data, self.weights, octree, depth, self.in_channels,
                                     self.kernel_size, self.stride, self.nempty)
    if self.use_bias:
      out = out + self.bias.to(out.dtype)
    if self.stride == 2 and not self.nempty:
      out = octree_pad(out, octree, depth - 1)
    return out

  def extra_repr(self) -> str:
    return ('in_channels={}, out_channels={}, kernel_size={}, stride={}, '
            'nempty={}, bias={}').format(self.in_channels, self.out_channels, self.kernel_size,
                                         self.stride, self.nempty, self.use_bias)

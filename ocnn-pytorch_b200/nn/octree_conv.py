"""OctreeConv / OctreeDeconv with the reference's module signatures
(ocnn/nn/octree_conv.py:300-466).  Every variant — all kernel shapes, stride 1
and 2, nempty on and off, forward, input gradient and weight gradient — runs on
two liboctconv kernels: a gather implicit GEMM (`oc_conv_fwd`) and a weight
gradient (`oc_conv_wgrad`).  The scatter direction (conv input gradient, deconv
forward) is turned into a gather through mirrored taps (stride 1) or a cached
inverse table (stride 2), so there are no atomics and no im2col buffer."""
from typing import List

import torch
from torch.autograd import Function

from .. import _lib
from ..octree import Octree
from ..utils import xavier_uniform_, resize_with_last_val, list2str
from .octree_pad import octree_pad, octree_depad


def _idx_bytes(table):
  return 8 if table.dtype == torch.int64 else 4


def tiled_supported(K, c_in, c_out, dtype):
  r''' True where the convolution runs on the tensor-core kernel, which can take the
  table as a tile table (:func:`tile_table`). '''
  return dtype in (torch.float16, torch.bfloat16) and \
      bool(_lib.lib().oc_conv_tiled_supported(K, c_in, c_out, _lib.dtype_code(dtype)))


class TileTable:
  r''' A tile table (uint8 tensor `tiles`) with the row order it was built in (`perm`, int32
  positions -> table rows, or None for the natural order). '''

  def __init__(self, tiles, perm=None):
    self.tiles = tiles
    self.perm = perm


ORDER_CHUNK_LOG2 = 19   # tables of more than 2^21 rows are ordered by tap mask within chunks of 2^19 consecutive rows


def tap_mask_order(table, taps, chunk_log2=None):
  r''' Rows of `table` sorted (stably) by the bit mask of their valid taps, as an int32
  permutation.  Tiles of a tile table built in this order hold rows with the same few taps,
  and the kernels skip the taps that are empty in a whole tile.  The key is the mask with its
  bits reordered - taps whose frequency over the table is farthest from one half are the most
  significant - so that the rows with a rare tap sit together (12.3 -> 11.2 taps per tile on
  the benchmark's nempty table, 17.2 -> 17.0 on the full one).  The sort runs within chunks
  of ``2**chunk_log2`` consecutive rows (0: over all rows at once; default: 2**19 for tables of
  more than 2**21 rows, else all rows at once): rows are in z-order, so
  a chunk is a neighbourhood of the octree and the rows a tile gathers stay close in memory
  however many octrees the batch holds; half a million rows per chunk lose 3 % of the skipped
  taps of the global order and run 2 % faster on the 4 M-row benchmark level. '''
  _lib.require_cuda(table)
  n = table.shape[0]
  if chunk_log2 is None:      # tables of up to 2^21 rows are sorted as a whole (3 % faster at 1 M rows)
    chunk_log2 = ORDER_CHUNK_LOG2 if n > (1 << 21) else 0
  perm = torch.empty(n, dtype=torch.int32, device=table.device)
  ws = _lib.workspace(_lib.lib().oc_tap_order_workspace_bytes(n), table.device)
  _lib.call('oc_tap_order', _lib.ptr(table), _idx_bytes(table), table.shape[1], _lib.int_array(taps), len(taps), n,
            int(chunk_log2), _lib.ptr(perm), _lib.ptr(ws), ws.numel(), _lib.stream(table.device))
  return perm


def tile_table(table, taps, n_in=0, perm=None):
  r''' Regroups columns `taps` of a neighbour table into blocks of 128 rows (16-byte
  header with the mask of non-empty taps, then one row of 128 int32 per tap): the form
  the tensor-core kernel fetches with one bulk copy per tile.  Returns a uint8 tensor.
  `n_in` > 0: the number of feature rows the table indexes; larger entries are dropped
  and make the next ``_lib.status_check`` raise (the kernels trust the tile table).
  `perm` (int32, a permutation of the rows): position j of the tile table holds row perm[j];
  give the result to :func:`conv_gather` wrapped in a :class:`TileTable` with the same `perm`. '''
  _lib.require_cuda(table)
  K, n_out = len(taps), table.shape[0]
  tiles = torch.empty(_lib.lib().oc_tile_table_bytes(n_out, K), dtype=torch.uint8, device=table.device)
  _lib.call('oc_tile_table_build', _lib.ptr(table), _idx_bytes(table), table.shape[1],
            _lib.int_array(taps), K, n_out, int(n_in), _lib.ptr(perm), _lib.ptr(tiles), tiles.numel(),
            _lib.stream(table.device))
  return tiles


def conv_gather(data, weights, w_transposed, bias, table, taps, c_in, c_out, tiles=None):
  r''' ``out[r] = sum_k data[table[r, taps[k]]] @ Wk (+ bias)`` with
  ``Wk = weights[k]`` (``w_transposed=False``, weights ``(K, c_in, c_out)``) or
  ``weights[k].T`` (``w_transposed=True``, weights ``(K, c_out, c_in)``).
  `tiles`: ``tile_table(table, taps)``, used instead of `table` where
  :func:`tiled_supported` holds. '''
  _lib.require_cuda(data, weights, table)
  data = data.contiguous()
  weights = weights.contiguous()
  if weights.dtype != torch.float32 and weights.dtype != data.dtype:
    weights = weights.to(data.dtype)
  if bias is not None:
    bias = bias.to(data.dtype).contiguous()
  K = len(taps)
  n_out = table.shape[0]
  assert data.shape[1] == c_in and weights.numel() == K * c_in * c_out
  dt = _lib.dtype_code(data.dtype)
  out = torch.empty(n_out, c_out, dtype=data.dtype, device=data.device)
  ws = _lib.workspace(_lib.lib().oc_conv_workspace_bytes(K, c_in, c_out, dt), data.device)
  if tiles is not None and n_out > 0 and tiled_supported(K, c_in, c_out, data.dtype):
    perm = None
    if isinstance(tiles, TileTable):
      tiles, perm = tiles.tiles, tiles.perm
    _lib.call('oc_conv_fwd_tiled', _lib.ptr(data), data.shape[0], _lib.ptr(weights),
              _lib.dtype_code(weights.dtype), int(w_transposed), _lib.ptr(bias), _lib.ptr(tiles),
              _lib.ptr(perm), K, n_out, c_in, c_out, dt, _lib.ptr(out), _lib.ptr(ws), ws.numel(),
              _lib.stream(data.device))
    return out
  _lib.call('oc_conv_fwd', _lib.ptr(data), data.shape[0], _lib.ptr(weights),
            _lib.dtype_code(weights.dtype), int(w_transposed), _lib.ptr(bias), _lib.ptr(table),
            _idx_bytes(table), table.shape[1], _lib.int_array(taps), K, n_out, c_in, c_out, dt,
            _lib.ptr(out), _lib.ptr(ws), ws.numel(), _lib.stream(data.device))
  return out


def conv_wgrad(data, grad_out, table, taps, c_in, c_out, want_bias_grad=False, tiles=None):
  r''' ``gw[k] = sum_r data[table[r, taps[k]]].T @ grad_out[r]`` as fp32
  ``(K, c_in, c_out)``; optionally also ``grad_out.sum(0)``.  `tiles`: as in
  :func:`conv_gather`. '''
  _lib.require_cuda(data, grad_out, table)
  data = data.contiguous()
  grad_out = grad_out.contiguous()
  assert data.dtype == grad_out.dtype
  K = len(taps)
  n_out = table.shape[0]
  assert grad_out.shape[0] == n_out and grad_out.shape[1] == c_out and data.shape[1] == c_in
  dt = _lib.dtype_code(data.dtype)
  gw = torch.empty(K, c_in, c_out, dtype=torch.float32, device=data.device)
  gb = torch.empty(c_out, dtype=torch.float32, device=data.device) if want_bias_grad else None
  ws = _lib.workspace(_lib.lib().oc_conv_wgrad_workspace_bytes(K, c_in, c_out, n_out, dt),
                      data.device)
  perm = None
  if isinstance(tiles, TileTable):
    tiles, perm = tiles.tiles, tiles.perm
  if tiles is not None and n_out > 0 and tiled_supported(K, c_in, c_out, data.dtype):
    _lib.call('oc_conv_wgrad_tiled', _lib.ptr(data), data.shape[0], _lib.ptr(grad_out), n_out,
              _lib.ptr(tiles), _lib.ptr(perm), K, c_in, c_out, dt, _lib.ptr(gw), _lib.ptr(gb), _lib.ptr(ws), ws.numel(),
              _lib.stream(data.device))
    return gw, gb
  _lib.call('oc_conv_wgrad', _lib.ptr(data), data.shape[0], _lib.ptr(grad_out), n_out,
            _lib.ptr(table), _idx_bytes(table), table.shape[1], _lib.int_array(taps), K, c_in,
            c_out, dt, _lib.ptr(gw), _lib.ptr(gb), _lib.ptr(ws), ws.numel(),
            _lib.stream(data.device))
  return gw, gb


class OctreeConvBase:
  r''' Shape bookkeeping shared by conv and deconv (octree_conv.py:30-113). '''

  def __init__(self, in_channels: int, out_channels: int, kernel_size: List[int] = [3],
               stride: int = 1, nempty: bool = False, max_buffer: int = int(2e8)):
    super().__init__()
    self.in_channels = in_channels
    self.out_channels = out_channels
    self.kernel_size = resize_with_last_val(kernel_size)
    self.kernel = list2str(self.kernel_size)
    self.stride = stride
    self.nempty = nempty
    self.max_buffer = max_buffer  # accepted for signature parity; there is no buffer
    self.kdim = self.kernel_size[0] * self.kernel_size[1] * self.kernel_size[2]
    self.in_conv = in_channels if self.is_conv_layer() else out_channels
    self.out_conv = out_channels if self.is_conv_layer() else in_channels
    self.weights_shape = (self.kdim, self.in_conv, self.out_conv)

  def is_conv_layer(self):
    raise NotImplementedError

  def setup(self, octree: Octree, depth: int):
    r''' Depths and heights of the tensors involved (octree_conv.py:51-89). '''
    self.in_depth = depth
    self.out_depth = depth
    self.neigh_depth = depth
    if self.stride == 2:
      if self.is_conv_layer():
        self.out_depth = depth - 1
      else:
        self.out_depth = depth + 1
        self.neigh_depth = depth + 1
    if self.nempty:
      self.in_h = int(octree.nnum_nempty[self.in_depth])
      self.out_h = int(octree.nnum_nempty[self.out_depth])
    else:
      self.in_h = int(octree.nnum[self.in_depth])
      self.out_h = int(octree.nnum[self.out_depth])
      if self.stride == 2:
        if self.is_conv_layer():
          self.out_h = int(octree.nnum_nempty[self.out_depth])
        else:
          self.in_h = int(octree.nnum_nempty[self.in_depth])
    self.in_shape = (self.in_h, self.in_channels)
    self.out_shape = (self.out_h, self.out_channels)

  def check(self, data: torch.Tensor):
    assert tuple(data.shape) == self.in_shape, (
        'The shape of input data is wrong: expected {}, got {}.'.format(self.in_shape, data.shape))


class _OctreeConv(OctreeConvBase):
  def is_conv_layer(self): return True


class _OctreeDeconv(OctreeConvBase):
  def is_conv_layer(self): return False


def wgrad_by_mask(c_in, c_out, nempty=False):
  r''' Whether the weight-gradient kernel should read the tile table ordered by tap mask
  (shared with the forward pass) or one in natural row order.  The mask order skips taps but
  scatters the grad_out rows, and with many channels a CTA holds few taps, so that the CTAs
  of the frequent taps bound the launch.  Measured on the depth-8 benchmark level: the mask
  order wins up to 128 channels (C=64 1.57 -> 1.42 ms, C=128 3.60 -> 3.56 ms) and on tables
  over the non-empty nodes at every width (a quarter of their slots are valid; C=256
  3.69 -> 3.21 ms); at 256 channels on a full table the natural order is 6 % faster. '''
  return nempty or max(c_in, c_out) <= 128


def _tiles(octree, depth, kernel, stride, nempty, transposed, K, c_in, c_out, data, by_mask=True):
  r''' The octree's cached tile table of this convolution, or None where the
  tensor-core kernel does not apply (then the plain table is used). '''
  if not tiled_supported(K, c_in, c_out, data.dtype):
    return None
  return octree.conv_tiles(depth, kernel, stride, nempty, transposed, by_mask)


class OctreeConvFunction(Function):
  r''' Octree convolution with autograd (octree_conv.py:219-254). '''

  @staticmethod
  def forward(ctx, data, weights, bias, octree, depth, in_channels, out_channels,
              kernel_size=[3, 3, 3], stride=1, nempty=False):
    conv = _OctreeConv(in_channels, out_channels, kernel_size, stride, nempty)
    conv.setup(octree, depth)
    conv.check(data)
    table, taps = octree.conv_table(depth, conv.kernel, stride, nempty)
    assert table.shape[0] == conv.out_h
    tiles = _tiles(octree, depth, conv.kernel, stride, nempty, False, len(taps), in_channels, out_channels, data)
    out = conv_gather(data, weights, False, bias, table, taps, in_channels, out_channels, tiles)
    ctx.save_for_backward(data, weights)
    ctx.conf = (octree, depth, conv.kernel, stride, nempty, in_channels, out_channels,
                bias is not None)
    return out

  @staticmethod
  def backward(ctx, grad):
    data, weights = ctx.saved_tensors
    octree, depth, kernel, stride, nempty, cin, cout, has_bias = ctx.conf
    grad = grad.contiguous()
    grad_in = grad_w = grad_b = None
    if ctx.needs_input_grad[0]:
      table_t, taps_t = octree.conv_table_transposed(depth, kernel, stride, nempty)
      tiles = _tiles(octree, depth, kernel, stride, nempty, True, len(taps_t), cout, cin, grad)
      grad_in = conv_gather(grad, weights, True, None, table_t, taps_t, cout, cin, tiles)
    if ctx.needs_input_grad[1] or (has_bias and ctx.needs_input_grad[2]):
      table, taps = octree.conv_table(depth, kernel, stride, nempty)
      tiles = _tiles(octree, depth, kernel, stride, nempty, False, len(taps), cin, cout, data,
                     by_mask=wgrad_by_mask(cin, cout, nempty))
      gw, gb = conv_wgrad(data, grad, table, taps, cin, cout, has_bias and ctx.needs_input_grad[2], tiles)
      grad_w = gw.to(weights.dtype) if ctx.needs_input_grad[1] else None
      grad_b = gb
    return (grad_in, grad_w, grad_b) + (None,) * 7


class OctreeDeconvFunction(Function):
  r''' Octree deconvolution with autograd (octree_conv.py:257-292). '''

  @staticmethod
  def forward(ctx, data, weights, bias, octree, depth, in_channels, out_channels,
              kernel_size=[3, 3, 3], stride=1, nempty=False):
    deconv = _OctreeDeconv(in_channels, out_channels, kernel_size, stride, nempty)
    deconv.setup(octree, depth)
    deconv.check(data)
    nd = deconv.neigh_depth
    table_t, taps_t = octree.conv_table_transposed(nd, deconv.kernel, stride, nempty)
    assert table_t.shape[0] == deconv.out_h
    tiles = _tiles(octree, nd, deconv.kernel, stride, nempty, True, len(taps_t), in_channels, out_channels, data)
    out = conv_gather(data, weights, True, bias, table_t, taps_t, in_channels, out_channels, tiles)
    ctx.save_for_backward(data, weights)
    ctx.conf = (octree, nd, deconv.kernel, stride, nempty, in_channels, out_channels,
                bias is not None)
    return out

  @staticmethod
  def backward(ctx, grad):
    data, weights = ctx.saved_tensors
    octree, nd, kernel, stride, nempty, cin, cout, has_bias = ctx.conf
    grad = grad.contiguous()
    grad_in = grad_w = grad_b = None
    table, taps = octree.conv_table(nd, kernel, stride, nempty)
    if ctx.needs_input_grad[0]:
      tiles = _tiles(octree, nd, kernel, stride, nempty, False, len(taps), cout, cin, grad)
      grad_in = conv_gather(grad, weights, False, None, table, taps, cout, cin, tiles)
    if ctx.needs_input_grad[1]:
      # weights are (K, out_channels, in_channels): gathered operand = grad
      tiles = _tiles(octree, nd, kernel, stride, nempty, False, len(taps), cout, cin, grad,
                     by_mask=wgrad_by_mask(cin, cout, nempty))
      gw, _ = conv_wgrad(grad, data, table, taps, cout, cin, False, tiles)
      grad_w = gw.to(weights.dtype)
    if has_bias and ctx.needs_input_grad[2]:
      from .octree_norm import col_stats
      grad_b = col_stats(grad)[0]
    return (grad_in, grad_w, grad_b) + (None,) * 7


def octree_conv(data, weights, octree, depth, in_channels, out_channels,
                kernel_size=[3, 3, 3], stride=1, nempty=False, max_buffer=int(2e8)):
  r''' Functional form with the reference's argument order (octree_conv.py:296). '''
  return OctreeConvFunction.apply(data, weights, None, octree, depth, in_channels, out_channels,
                                  kernel_size, stride, nempty)


def octree_deconv(data, weights, octree, depth, in_channels, out_channels,
                  kernel_size=[3, 3, 3], stride=1, nempty=False, max_buffer=int(2e8)):
  r''' Functional form with the reference's argument order (octree_conv.py:297). '''
  return OctreeDeconvFunction.apply(data, weights, None, octree, depth, in_channels,
                                    out_channels, kernel_size, stride, nempty)


def _autocast(data):
  if torch.is_autocast_enabled('cuda') and data.is_floating_point():
    return data.to(torch.get_autocast_dtype('cuda'))
  return data


class OctreeConv(OctreeConvBase, torch.nn.Module):
  r''' Performs octree convolution.

  Same constructor as the reference (octree_conv.py:300-345): ``in_channels``,
  ``out_channels``, ``kernel_size`` from ``[3]``, ``[2]``, ``[3,1,1]``, ``[1,3,1]``,
  ``[1,1,3]``, ``[3,3,1]``, ``[1,3,3]``, ``[3,1,3]``, ``stride`` 1 or 2, ``nempty``,
  ``use_bias``.  ``method`` and ``max_buffer`` are accepted and ignored: there is
  one implementation and it has no buffer.  Under ``torch.autocast('cuda')`` the
  input is cast to the autocast dtype so the convolution runs in bf16 / fp16.
  '''

  def __init__(self, in_channels: int, out_channels: int, kernel_size: List[int] = [3],
               stride: int = 1, nempty: bool = False, method: str = 'triton',
               use_bias: bool = False, max_buffer: int = int(2e8)):
    super().__init__(in_channels, out_channels, kernel_size, stride, nempty, max_buffer)
    self.use_bias = use_bias
    self.method = method
    self.weights = torch.nn.Parameter(torch.Tensor(*self.weights_shape))
    self.bias = torch.nn.Parameter(torch.Tensor(out_channels)) if use_bias else None
    self.reset_parameters()

  def reset_parameters(self):
    xavier_uniform_(self.weights)
    if self.use_bias:
      torch.nn.init.zeros_(self.bias)

  def is_conv_layer(self): return True

  def forward(self, data: torch.Tensor, octree: Octree, depth: int):
    data = _autocast(data)
    out = OctreeConvFunction.apply(data, self.weights, self.bias, octree, depth,
                                   self.in_channels, self.out_channels, self.kernel_size,
                                   self.stride, self.nempty)
    if self.stride == 2 and not self.nempty:
      out = octree_pad(out, octree, depth - 1)
    return out

  def extra_repr(self) -> str:
    return ('in_channels={}, out_channels={}, kernel_size={}, stride={}, '
            'nempty={}, bias={}').format(self.in_channels, self.out_channels, self.kernel_size,
                                         self.stride, self.nempty, self.use_bias)


class OctreeDeconv(OctreeConv):
  r''' Performs octree deconvolution (octree_conv.py:433-466); weights have
  shape ``(K, out_channels, in_channels)``. '''

  def is_conv_layer(self): return False

  def forward(self, data: torch.Tensor, octree: Octree, depth: int):
    data = _autocast(data)
    if self.stride == 2 and not self.nempty:
      data = octree_depad(data, octree, depth)
    return OctreeDeconvFunction.apply(data, self.weights, self.bias, octree, depth,
                                      self.in_channels, self.out_channels, self.kernel_size,
                                      self.stride, self.nempty)

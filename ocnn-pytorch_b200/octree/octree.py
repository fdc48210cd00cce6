"""Octree index structure with the attributes and methods of the reference's
`ocnn.octree.Octree` (ocnn/octree/octree.py:18-773): per-depth `keys` (int64),
`children` (int32), `neighs` (int64, 27 columns), leaf `points` / `normals` /
`features`, CPU `nnum` / `nnum_nempty`, and the `lut_*` tables.  All device work
is done by liboctconv kernels; tensors must live on a CUDA device."""
import ctypes
from typing import List, Union

import torch

from .. import _lib
from .points import Points
from .shuffled_key import xyz2key, key2xyz

# kernel name -> columns of the 27-column neighbour table (octree.py:98-106)
KERNEL_TAPS = {
    '333': list(range(27)),
    '222': [13, 14, 16, 17, 22, 23, 25, 26],
    '311': [4, 13, 22],
    '131': [10, 13, 16],
    '113': [12, 13, 14],
    '331': [1, 4, 7, 10, 13, 16, 19, 22, 25],
    '313': [3, 4, 5, 12, 13, 14, 21, 22, 23],
    '133': [9, 10, 11, 12, 13, 14, 15, 16, 17],
}


def _range_grid(lo: int, hi: int):
  rng = range(lo, hi + 1)
  return [(a, b, c) for a in rng for b in rng for c in rng]


def _parent_child_luts():
  r''' (8,27) tables of octree.py:86-95: for child i and tap k of a node, which
  tap of the parent and which child of that neighbour holds the cell. '''
  lut_parent, lut_child = [], []
  for c in _range_grid(2, 3):
    rp, rc = [], []
    for d in _range_grid(-1, 1):
      g = [c[a] + d[a] for a in range(3)]
      rp.append((g[0] // 2) * 9 + (g[1] // 2) * 3 + (g[2] // 2))
      rc.append((g[0] % 2) * 4 + (g[1] % 2) * 2 + (g[2] % 2))
    lut_parent.append(rp)
    lut_child.append(rc)
  return lut_parent, lut_child


_LUTS = {}


def _device_luts(device):
  r''' The constant look-up tables of an octree (octree.py:86-106) on `device`, created once per
  device: they are read-only attributes, and uploading them for every new Octree costs more
  host time than a small octree build takes on the GPU. '''
  key = str(device)
  if key not in _LUTS:
    lp, lc = _parent_child_luts()
    _LUTS[key] = (torch.tensor(lp, device=device), torch.tensor(lc, device=device),
                  {k: torch.tensor(v, device=device) for k, v in KERNEL_TAPS.items() if k != '333'})
  lp, lc, lk = _LUTS[key]
  return lp, lc, dict(lk)


class Octree:
  r''' Builds and holds a (batched) octree on a CUDA device.

  Args:
    depth (int): The octree depth.
    full_depth (int): Layers with depth <= :attr:`full_depth` are dense.
    batch_size (int): Number of octrees merged in this object.
    device: A CUDA device.  (The object can be created with ``'cpu'`` but every
        method that computes raises on CPU tensors: there is no CPU path.)
  '''

  def __init__(self, depth: int, full_depth: int = 2, batch_size: int = 1,
               device: Union[torch.device, str] = 'cpu', **kwargs):
    self.depth = depth
    self.full_depth = full_depth
    self.batch_size = batch_size
    self.device = torch.device(device) if isinstance(device, str) else device
    self.reset()

  # ------------------------------------------------------------------ state
  def reset(self):
    num = self.depth + 1
    self.keys = [None] * num
    self.children = [None] * num
    self.neighs = [None] * num
    self.features = [None] * num
    self.normals = [None] * num
    self.points = [None] * num
    self.nempty_masks = [None] * num
    self.nempty_indices = [None] * num
    self.nempty_neighs = [None] * num
    self.nnum = torch.zeros(num, dtype=torch.long)
    self.nnum_nempty = torch.zeros(num, dtype=torch.long)
    batch_size = self.batch_size
    self.batch_nnum = torch.zeros(num, batch_size, dtype=torch.long)
    self.batch_nnum_nempty = torch.zeros(num, batch_size, dtype=torch.long)
    self.lut_parent, self.lut_child, self.lut_kernel = _device_luts(self.device)
    self._table_cache = {}

  def _invalidate(self, depth=None):
    r''' Drops cached neighbour-table variants (all, or those of one depth). '''
    if depth is None:
      self._table_cache = {}
    else:
      self._table_cache = {k: v for k, v in self._table_cache.items() if k[1] != depth}

  def _stream(self):
    return _lib.stream(self.device)

  # ------------------------------------------------------------ accessors
  def key(self, depth: int, nempty: bool = False):
    key = self.keys[depth]
    if nempty:
      key = key[self.nempty_index(depth)]
    return key

  def xyzb(self, depth: int, nempty: bool = False):
    return key2xyz(self.key(depth, nempty), depth)

  def batch_id(self, depth: int, nempty: bool = False):
    batch_id = self.keys[depth] >> 48
    if nempty:
      batch_id = batch_id[self.nempty_index(depth)]
    return batch_id

  def nempty_mask(self, depth: int, reset: bool = False):
    if self.nempty_masks[depth] is None or reset:
      self.nempty_masks[depth] = self.children[depth] >= 0
    return self.nempty_masks[depth]

  def nempty_index(self, depth: int, reset: bool = False):
    r''' Indices (int64) of the non-empty nodes of :attr:`depth` (octree.py:160-172). '''
    if self.nempty_indices[depth] is None or reset:
      children = self.children[depth]
      _lib.require_cuda(children)
      n = int(self.nnum_nempty[depth])
      index = torch.empty(n, dtype=torch.int64, device=children.device)
      nnum = children.numel()
      ws = _lib.workspace(_lib.lib().oc_nempty_index_workspace_bytes(nnum), children.device)
      _lib.call('oc_nempty_index', _lib.ptr(children), nnum, _lib.ptr(index), _lib.ptr(ws),
                ws.numel(), self._stream())
      self.nempty_indices[depth] = index
    return self.nempty_indices[depth]

  def _variant(self, depth: int, taps, stride: int, nempty: bool, out_dtype=torch.int64):
    r''' get_neigh core: row select (stride 2 / non-empty rows) + optional remap
    through children + column select, in one kernel. '''
    neigh = self.neighs[depth]
    assert neigh is not None, 'construct_neigh(%d) must be called first' % depth
    rows, row_stride = None, 1
    if stride == 2:
      n_rows, row_stride = neigh.shape[0] // 8, 8
    elif nempty:
      rows = self.nempty_index(depth)
      n_rows = rows.numel()
    else:
      n_rows = neigh.shape[0]
    children = self.children[depth] if nempty else None
    out = torch.empty(n_rows, len(taps), dtype=out_dtype, device=neigh.device)
    _lib.call('oc_neigh_variant', _lib.ptr(neigh), _lib.ptr(children), _lib.ptr(rows), row_stride,
              n_rows, _lib.int_array(taps), len(taps), _lib.ptr(out),
              8 if out_dtype == torch.int64 else 4, self._stream())
    return out

  def nempty_neigh(self, depth: int, reset: bool = False):
    r''' Neighbour table restricted to, and numbered by, the non-empty nodes
    (octree.py:174-199). '''
    if self.nempty_neighs[depth] is None or reset:
      self.nempty_neighs[depth] = self._variant(depth, KERNEL_TAPS['333'], 1, True)
    return self.nempty_neighs[depth]

  def remap_nempty_neigh(self, neigh: torch.Tensor, depth: int):
    r''' In-place remap of valid entries through ``children[depth]`` (octree.py:188-199). '''
    valid = neigh >= 0
    child = self.children[depth]
    neigh[valid] = child[neigh[valid]].long()
    return neigh

  # ------------------------------------------------------------- building
  def build_octree(self, point_cloud: Points, bbmin=-1.0, bbmax=1.0):
    r''' Builds the octree from a point cloud (octree.py:201-287): keys,
    children and node counts of every depth, averaged leaf signals, and the
    returned ``idx`` (point -> rank of its non-empty leaf). '''
    self.device = point_cloud.device
    assert point_cloud.batch_size == self.batch_size, 'Inconsistent batch_size'
    pts = point_cloud.points
    _lib.require_cuda(pts)
    device = pts.device
    pts = pts.float().contiguous()
    npts = pts.shape[0]
    depth, full_depth, B = self.depth, self.full_depth, self.batch_size

    box = bbmax - bbmin
    if isinstance(box, torch.Tensor):
      box = box.max().item()
    assert box > 0, 'The bounding box size must be greater than 0.'
    mul = (2 ** depth) / box
    if isinstance(bbmin, torch.Tensor):
      bb = [float(v) for v in bbmin.flatten().tolist()]
      bb = bb * 3 if len(bb) == 1 else bb
    else:
      bb = [float(bbmin)] * 3
    h_bb = _lib.f32_array(bb)

    bid, bid_code = None, _lib.OC_COORD_F32
    if B > 1:
      bid = point_cloud.batch_id.view(-1)
      if bid.dtype == torch.int64:
        bid_code = _lib.OC_I64
      elif bid.dtype == torch.int32:
        bid_code = _lib.OC_I32
      elif bid.dtype != torch.float32:
        bid, bid_code = bid.long(), _lib.OC_I64
      bid = bid.contiguous()

    L = _lib.lib()
    ws = _lib.workspace(L.oc_build_workspace_bytes(npts, depth, full_depth, B), device)
    h_nne = (ctypes.c_int64 * (depth + 1))()
    s = _lib.stream(device)
    _lib.call('oc_build_octree_count', _lib.ptr(pts), _lib.ptr(bid), bid_code, npts, depth,
              full_depth, B, h_bb, mul, _lib.ptr(ws), ws.numel(), h_nne, s)
    nne = [int(v) for v in h_nne]
    nnum = [(B << (3 * d)) if d <= full_depth else 8 * nne[d - 1] for d in range(depth + 1)]

    self.reset()
    self.nnum = torch.tensor(nnum, dtype=torch.long)
    self.nnum_nempty = torch.tensor(nne, dtype=torch.long)
    for d in range(depth + 1):
      self.keys[d] = torch.empty(nnum[d], dtype=torch.int64, device=device)
      self.children[d] = torch.empty(nnum[d], dtype=torch.int32, device=device)

    normals = point_cloud.normals
    features = point_cloud.features
    nleaf = nne[depth]
    out_pts = torch.empty(nleaf, 3, dtype=torch.float32, device=device)
    out_nrm = out_feat = None
    nfeat = 0
    if normals is not None:
      normals = normals.float().contiguous()
      out_nrm = torch.empty(nleaf, 3, dtype=torch.float32, device=device)
    if features is not None:
      features = features.float().contiguous()
      nfeat = features.shape[1]
      out_feat = torch.empty(nleaf, nfeat, dtype=torch.float32, device=device)
    idx = torch.empty(npts, dtype=torch.int64, device=device)
    _lib.call('oc_build_octree_emit', _lib.ptr(pts), _lib.ptr(normals), _lib.ptr(features), nfeat,
              npts, depth, full_depth, B, h_bb, mul, _lib.ptr(ws), h_nne,
              _lib.ptr_array(self.keys), _lib.ptr_array(self.children), _lib.ptr(out_pts),
              _lib.ptr(out_nrm), _lib.ptr(out_feat), _lib.ptr(idx), s)
    self.points[depth] = out_pts
    self.normals[depth] = out_nrm
    self.features[depth] = out_feat
    return idx

  def octree_grow_full(self, depth: int, update_neigh: bool = True):
    r''' Makes layer :attr:`depth` dense (octree.py:289-321). '''
    assert depth <= self.full_depth, 'error'
    _lib.require_cuda(torch.empty(0, device=self.device))
    num = (1 << (3 * depth)) * self.batch_size
    self.nnum[depth] = num
    self.nnum_nempty[depth] = num
    self.keys[depth] = torch.empty(num, dtype=torch.int64, device=self.device)
    self.children[depth] = torch.empty(num, dtype=torch.int32, device=self.device)
    _lib.call('oc_full_layer', depth, self.batch_size, _lib.ptr(self.keys[depth]),
              _lib.ptr(self.children[depth]), self._stream())
    self._invalidate(depth)
    if update_neigh:
      self.construct_neigh(depth)

  def octree_split(self, split: torch.Tensor, depth: int):
    r''' Sets which nodes of :attr:`depth` are non-empty (octree.py:323-351). '''
    split = split.to(torch.int64)
    csum = torch.cumsum(split, dim=0)
    children = (csum - split).to(torch.int32)
    children[split == 0] = -1
    nnum_nempty = int(csum[-1].item()) if split.numel() > 0 else 0
    if nnum_nempty == 0:
      nnum_nempty = 1
      children[0] = 0
    self.children[depth] = children
    self.nnum_nempty[depth] = nnum_nempty
    self.nempty_masks[depth] = None
    self.nempty_indices[depth] = None
    self.nempty_neighs[depth] = None
    self._invalidate(depth)
    self._invalidate(depth + 1)

  def octree_grow(self, depth: int, update_neigh: bool = True):
    r''' Adds layer :attr:`depth` under the non-empty nodes of depth-1
    (octree.py:353-402). '''
    if depth > self.depth:
      assert depth == self.depth + 1
      self.depth = depth
      for lst in (self.keys, self.children, self.neighs, self.features, self.normals,
                  self.points, self.nempty_masks, self.nempty_indices, self.nempty_neighs):
        lst.append(None)
      zero = torch.zeros(1, dtype=torch.long)
      self.nnum = torch.cat([self.nnum, zero])
      self.nnum_nempty = torch.cat([self.nnum_nempty, zero])
      zero = torch.zeros([1, self.batch_size], dtype=torch.long)
      self.batch_nnum = torch.cat([self.batch_nnum, zero], dim=0)
      self.batch_nnum_nempty = torch.cat([self.batch_nnum_nempty, zero], dim=0)
    nnum = int(self.nnum_nempty[depth - 1]) * 8
    self.nnum[depth] = nnum
    self.nnum_nempty[depth] = nnum
    keys_p, children_p = self.keys[depth - 1], self.children[depth - 1]
    self.keys[depth] = torch.empty(nnum, dtype=torch.int64, device=keys_p.device)
    self.children[depth] = torch.empty(nnum, dtype=torch.int32, device=keys_p.device)
    _lib.call('oc_grow_layer', _lib.ptr(keys_p), _lib.ptr(children_p), keys_p.numel(),
              _lib.ptr(self.keys[depth]), _lib.ptr(self.children[depth]), self._stream())
    self.nempty_masks[depth] = None
    self.nempty_indices[depth] = None
    self.nempty_neighs[depth] = None
    self._invalidate(depth)
    if update_neigh:
      self.construct_neigh(depth)

  # ----------------------------------------------------------- neighbours
  def construct_neigh(self, depth: int):
    r''' Builds the (nnum[depth], 27) int64 neighbour table (octree.py:404-439). '''
    device = self.device
    if depth <= self.full_depth:
      n = (1 << (3 * depth)) * self.batch_size
      neigh = torch.empty(n, 27, dtype=torch.int64, device=device)
      _lib.call('oc_neigh_full', depth, self.batch_size, _lib.ptr(neigh), self._stream())
    else:
      neigh_p, child_p = self.neighs[depth - 1], self.children[depth - 1]
      assert neigh_p is not None, 'construct_neigh(%d) must be called first' % (depth - 1)
      n = int(self.nnum_nempty[depth - 1]) * 8
      neigh = torch.empty(n, 27, dtype=torch.int64, device=device)
      _lib.call('oc_neigh_from_parent', _lib.ptr(neigh_p), _lib.ptr(child_p), child_p.numel(),
                _lib.ptr(neigh), None, self._stream())
    self.neighs[depth] = neigh
    self.nempty_neighs[depth] = None
    self._invalidate(depth)

  def construct_all_neigh(self):
    for depth in range(1, self.depth + 1):
      self.construct_neigh(depth)

  def get_neigh(self, depth: int, kernel: str = '333', stride: int = 1, nempty: bool = False):
    r''' Neighbour table for a kernel shape / stride / nempty mode
    (octree.py:490-523), int64 ``(rows, K)``.  Variants are cached per
    ``(depth, kernel, stride, nempty)`` until the layer changes. '''
    if stride not in (1, 2):
      raise ValueError('Unsupported stride {}'.format(stride))
    if kernel not in KERNEL_TAPS:
      raise ValueError('Unsupported kernel {}'.format(kernel))
    if kernel == '333' and stride == 1:
      return self.nempty_neigh(depth) if nempty else self.neighs[depth]
    key = ('neigh', depth, kernel, stride, nempty)
    if key not in self._table_cache:
      self._table_cache[key] = self._variant(depth, KERNEL_TAPS[kernel], stride, nempty)
    return self._table_cache[key]

  def conv_table(self, depth: int, kernel: str, stride: int, nempty: bool):
    r''' Table description used by the convolution kernels for the *gather*
    direction: ``(table, taps)`` with ``table[r, taps[k]]`` the input row of tap
    k of output row r.  Stride-1 kernels address the 27-column table directly
    through `taps`, so sub-kernels need no table of their own. '''
    if stride not in (1, 2):
      raise ValueError('Unsupported stride {}'.format(stride))
    if kernel not in KERNEL_TAPS:
      raise ValueError('Unsupported kernel {}'.format(kernel))
    if stride == 1:
      table = self.nempty_neigh(depth) if nempty else self.neighs[depth]
      assert table is not None, 'construct_neigh(%d) must be called first' % depth
      return table, KERNEL_TAPS[kernel]
    table = self.get_neigh(depth, kernel, stride, nempty)
    return table, list(range(table.shape[1]))

  def conv_table_transposed(self, depth: int, kernel: str, stride: int, nempty: bool):
    r''' Table for the *scatter* direction (input gradient of a conv, forward of
    a deconv) expressed as a gather, so no atomics are needed.
    Stride 1: the same table read at the mirrored taps ``26 - t`` (the relation
    ``neigh[n, t] == m  <=>  neigh[m, 26 - t] == n`` holds for 3x3x3 tables).
    Stride 2: the inverse table ``inv[target, k] = row``, built once and cached. '''
    table, taps = self.conv_table(depth, kernel, stride, nempty)
    if stride == 1:
      return table, [26 - t for t in taps]
    key = ('inverse', depth, kernel, stride, nempty)
    if key not in self._table_cache:
      n_targets = int(self.nnum_nempty[depth] if nempty else self.nnum[depth])
      K = len(taps)
      inv = torch.empty(n_targets, K, dtype=torch.int32, device=table.device)
      _lib.call('oc_neigh_inverse', _lib.ptr(table), 8, table.shape[0], table.shape[1],
                _lib.int_array(taps), K, n_targets, _lib.ptr(inv), self._stream())
      self._table_cache[key] = inv
    return self._table_cache[key], list(range(len(taps)))

  def conv_tiles(self, depth: int, kernel: str, stride: int, nempty: bool, transposed: bool = False,
                 by_mask: bool = True):
    r''' The table of :meth:`conv_table` (or :meth:`conv_table_transposed`) as a tile
    table for the tensor-core convolution kernels, built once and cached like the
    neighbour tables themselves.  Its rows are ordered by the bit mask of their valid taps
    (:func:`tap_mask_order`): a tile then holds rows with the same few taps and the empty taps
    are skipped - for the inverse table of a stride-2 convolution this groups the rows by child
    index.  The result carries the row order (:class:`TileTable`).  ``by_mask=False`` keeps the
    natural row order, which the weight-gradient kernel prefers above 64 channels
    (``nn.wgrad_by_mask``). '''
    key = ('tiles', depth, kernel, stride, nempty, transposed, by_mask)
    if key not in self._table_cache:
      from ..nn.octree_conv import tile_table, tap_mask_order, TileTable
      table, taps = (self.conv_table_transposed if transposed else self.conv_table)(depth, kernel, stride, nempty)
      if transposed and stride == 2:     # the inverse table indexes the rows of the forward table
        n_in = self.conv_table(depth, kernel, stride, nempty)[0].shape[0]
      else:
        n_in = int(self.nnum_nempty[depth] if nempty else self.nnum[depth])
      perm = tap_mask_order(table, taps) if by_mask else None
      self._table_cache[key] = TileTable(tile_table(table, taps, n_in, perm), perm)
    return self._table_cache[key]

  def batch_offsets(self, depth: int, nempty: bool = False):
    r''' Host list of batch_size+1 row offsets of each octree at :attr:`depth`
    (rows of one octree are contiguous because keys sort batch-major). '''
    key = ('offsets', depth, nempty)
    if key not in self._table_cache:
      keys = self.keys[depth]
      children = self.children[depth] if nempty else None
      B = self.batch_size
      nnum = keys.numel()
      nbytes = 2 * ((B + 1) * 8 + 256) + _lib.lib().oc_nempty_index_workspace_bytes(nnum) + 512
      ws = _lib.workspace(nbytes, keys.device)
      h = (ctypes.c_int64 * (B + 1))()
      _lib.call('oc_batch_offsets', _lib.ptr(keys), _lib.ptr(children), nnum, B, h, _lib.ptr(ws),
                ws.numel(), self._stream())
      self._table_cache[key] = [int(v) for v in h]
    return self._table_cache[key]

  # --------------------------------------------------------------- search
  def search_xyzb(self, query: torch.Tensor, depth: int, nempty: bool = False):
    key = xyz2key(query[:, 0], query[:, 1], query[:, 2], query[:, 3], depth)
    return self.search_key(key, depth, nempty)

  def search_key(self, query: torch.Tensor, depth: int, nempty: bool = False):
    r''' Index of each query key among the node keys, -1 if absent
    (octree.py:464-488). '''
    key = self.key(depth, nempty).contiguous()
    query = query.long().contiguous()
    _lib.require_cuda(key, query)
    idx = torch.empty_like(query)
    _lib.call('oc_search_key', _lib.ptr(key), key.numel(), _lib.ptr(query), query.numel(),
              _lib.ptr(idx), self._stream())
    return idx

  # ------------------------------------------------------------- features
  def get_input_feature(self, feature: str, nempty: bool = False):
    r''' Initial input features from the leaf signals (octree.py:525-568). '''
    from ..nn.octree_pad import octree_pad
    features = list()
    depth = self.depth
    feature = feature.upper()
    if 'N' in feature:
      features.append(self.normals[depth])
    if 'L' in feature or 'D' in feature:
      local_points = self.points[depth].frac() - 0.5
    if 'D' in feature:
      dis = torch.sum(local_points * self.normals[depth], dim=1, keepdim=True)
      features.append(dis)
    if 'L' in feature:
      features.append(local_points)
    if 'P' in feature:
      scale = 2 ** (1 - depth)
      features.append(self.points[depth] * scale - 1.0)
    if 'F' in feature:
      features.append(self.features[depth])
    out = torch.cat(features, dim=1)
    if not nempty:
      out = octree_pad(out, self, depth)
    return out

  # --------------------------------------------------------------- moving
  def to(self, device: Union[torch.device, str], non_blocking: bool = False):
    if isinstance(device, str):
      device = torch.device(device)
    if self.device == device:
      return self

    def mv(prop):
      return [p.to(device, non_blocking=non_blocking) if isinstance(p, torch.Tensor) else None
              for p in prop]

    octree = Octree.init_like(self, device)
    octree.keys = mv(self.keys)
    octree.children = mv(self.children)
    octree.neighs = mv(self.neighs)
    octree.features = mv(self.features)
    octree.normals = mv(self.normals)
    octree.points = mv(self.points)
    octree.nnum = self.nnum.clone()
    octree.nnum_nempty = self.nnum_nempty.clone()
    octree.batch_nnum = self.batch_nnum.clone()
    octree.batch_nnum_nempty = self.batch_nnum_nempty.clone()
    return octree

  def cuda(self, non_blocking: bool = False):
    return self.to(torch.device('cuda', torch.cuda.current_device()), non_blocking)

  def cpu(self):
    return self.to('cpu')

  def merge_octrees(self, octrees: List['Octree']):
    r''' Merges single octrees into one batch (octree.py:653-717): keys get the
    batch index in bits 48+, children are offset by the running non-empty count. '''
    batch_size = len(octrees)
    self.batch_size = batch_size
    for i in range(1, batch_size):
      condition = (octrees[i].depth == self.depth and
                   octrees[i].full_depth == self.full_depth and
                   octrees[i].device == self.device)
      assert condition, 'The check of merge_octrees failed'
    batch_nnum = torch.stack([octrees[i].nnum for i in range(batch_size)], dim=1)
    batch_nnum_nempty = torch.stack([octrees[i].nnum_nempty for i in range(batch_size)], dim=1)
    self.nnum = torch.sum(batch_nnum, dim=1)
    self.nnum_nempty = torch.sum(batch_nnum_nempty, dim=1)
    self.batch_nnum = batch_nnum
    self.batch_nnum_nempty = batch_nnum_nempty
    zeros = torch.zeros(batch_nnum_nempty.shape[0], 1, dtype=torch.long)
    nnum_cum = torch.cat([zeros, torch.cumsum(batch_nnum_nempty, dim=1)], dim=1)
    for d in range(self.depth + 1):
      keys, children = [None] * batch_size, [None] * batch_size
      for i in range(batch_size):
        key = octrees[i].keys[d] & ((1 << 48) - 1)
        keys[i] = key | (i << 48)
        child = octrees[i].children[d].clone()
        mask = child >= 0
        child[mask] = child[mask] + int(nnum_cum[d, i])
        children[i] = child
      self.keys[d] = torch.cat(keys, dim=0)
      self.children[d] = torch.cat(children, dim=0)
      if d == self.depth:
        for name in ('features', 'normals', 'points'):
          if getattr(octrees[0], name)[d] is not None:
            getattr(self, name)[d] = torch.cat([getattr(o, name)[d] for o in octrees], dim=0)
    self._invalidate()
    return self

  @classmethod
  def init_like(cls, octree: 'Octree', device: Union[torch.device, str, None] = None):
    device = device if device is not None else octree.device
    return cls(depth=octree.depth, full_depth=octree.full_depth,
               batch_size=octree.batch_size, device=device)

  @classmethod
  def init_octree(cls, depth: int, full_depth: int = 2, batch_size: int = 1,
                  device: Union[torch.device, str] = 'cpu'):
    octree = cls(depth, full_depth, batch_size, device)
    for d in range(full_depth + 1):
      octree.octree_grow_full(depth=d)
    return octree


def merge_octrees(octrees: List['Octree']):
  r''' Wrapper of :meth:`Octree.merge_octrees`. '''
  return Octree.init_like(octrees[0]).merge_octrees(octrees)


def init_octree(depth: int, full_depth: int = 2, batch_size: int = 1,
                device: Union[torch.device, str] = 'cpu'):
  r''' Wrapper of :meth:`Octree.init_octree`. '''
  return Octree.init_octree(depth, full_depth, batch_size, device)

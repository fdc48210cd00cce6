"""CPU oracle (numpy) for the octree hot path — TEST INFRASTRUCTURE ONLY.

A plain restatement of the reference algorithms of octree-nn/ocnn-pytorch, each
function citing the reference file:line it follows.  Only `tests/`, the smoke
check and the benchmark's CPU-baseline leg may import this module; the product
(`ocnn-pytorch_b200/`) never does.

Parity pinning: `tests/test_oracle.py` checks every function here against golden
vectors produced by the reference itself (`tests/golden/make_golden.py` imports
the reference and stores its outputs, including the reference's own test
fixtures test_00{1..5}.npz / batch_45.npz and its 3-point hand case).
"""
import numpy as np

KERNEL_TAPS = {   # ocnn/octree/octree.py:98-106
    '333': list(range(27)),
    '222': [13, 14, 16, 17, 22, 23, 25, 26],
    '311': [4, 13, 22],
    '131': [10, 13, 16],
    '113': [12, 13, 14],
    '331': [1, 4, 7, 10, 13, 16, 19, 22, 25],
    '313': [3, 4, 5, 12, 13, 14, 21, 22, 23],
    '133': [9, 10, 11, 12, 13, 14, 15, 16, 17],
}


# ---------------------------------------------------------------- shuffled key
def _interleave(x, y, z, depth):
  '''KeyLUT.xyz2key, ocnn/octree/shuffled_key.py:37-44.'''
  key = np.zeros_like(x)
  for i in range(depth):
    mask = np.int64(1) << i
    key = (key | ((x & mask) << (2 * i + 2)) | ((y & mask) << (2 * i + 1)) |
           ((z & mask) << (2 * i + 0)))
  return key


def xyz2key(x, y, z, b=None, depth=16):
  '''ocnn/octree/shuffled_key.py:60-90.  `.long()` == truncation toward zero.'''
  x, y, z = (np.trunc(np.asarray(v)).astype(np.int64) if np.asarray(v).dtype.kind == 'f'
             else np.asarray(v).astype(np.int64) for v in (x, y, z))
  mask = 255 if depth > 8 else (1 << depth) - 1
  key = _interleave(x & mask, y & mask, z & mask, 8)
  if depth > 8:
    mask = (1 << (depth - 8)) - 1
    key16 = _interleave((x >> 8) & mask, (y >> 8) & mask, (z >> 8) & mask, 8)
    key = (key16 << 24) | key
  if b is not None:
    bb = np.asarray(b)
    bb = np.trunc(bb).astype(np.int64) if bb.dtype.kind == 'f' else bb.astype(np.int64)
    key = (bb << 48) | key
  return key


def key2xyz(key, depth=16):
  '''ocnn/octree/shuffled_key.py:93-115 (9 key bits per loop iteration).'''
  key = np.asarray(key, dtype=np.int64)
  b = key >> 48
  key = key & ((np.int64(1) << 48) - 1)
  x = np.zeros_like(key)
  y = np.zeros_like(key)
  z = np.zeros_like(key)
  n = (depth + 2) // 3
  for i in range(n):
    k = (key >> (i * 9)) & 511
    for j in range(3):
      x = x | (((k >> (3 * j + 2)) & 1) << (i * 3 + j))
      y = y | (((k >> (3 * j + 1)) & 1) << (i * 3 + j))
      z = z | (((k >> (3 * j + 0)) & 1) << (i * 3 + j))
  return x, y, z, b


# ---------------------------------------------------------------- octree build
def scatter_add(src, index, dim_size):
  '''ocnn/utils.py:117-147 along dim 0 (sequential accumulation in index order).'''
  out = np.zeros((dim_size,) + src.shape[1:], dtype=src.dtype)
  np.add.at(out, index, src)
  return out


def build_octree(points, normals=None, features=None, batch_id=None, batch_size=1, depth=6,
                 full_depth=2, bbmin=-1.0, bbmax=1.0):
  '''Octree.build_octree, ocnn/octree/octree.py:201-287 (+ Points.normalize,
  ocnn/octree/points.py:223-244).  Returns a dict of per-depth lists.'''
  points = np.asarray(points, dtype=np.float32)
  box = np.max(np.asarray(bbmax, dtype=np.float64) - np.asarray(bbmin, dtype=np.float64))
  mul = np.float32((2 ** depth) / box)
  pts = ((points - np.asarray(bbmin, dtype=np.float32)).astype(np.float32) * mul).astype(np.float32)
  b = None if batch_size == 1 else np.asarray(batch_id).reshape(-1)
  key = xyz2key(pts[:, 0], pts[:, 1], pts[:, 2], b, depth)
  node_key, idx, counts = np.unique(key, return_inverse=True, return_counts=True)

  num = depth + 1
  keys, children = [None] * num, [None] * num
  nnum = np.zeros(num, dtype=np.int64)
  nnum_nempty = np.zeros(num, dtype=np.int64)
  for d in range(full_depth + 1):           # octree_grow_full, octree.py:289-321
    n = 1 << (3 * d)
    nnum[d] = nnum_nempty[d] = n * batch_size
    k = np.arange(n, dtype=np.int64)[None, :] | (np.arange(batch_size, dtype=np.int64)[:, None] << 48)
    keys[d] = k.reshape(-1)
    children[d] = np.arange(n * batch_size, dtype=np.int32)

  for d in range(depth, full_depth, -1):    # octree.py:235-259
    pkey = node_key >> 3
    pkey, pidx = np.unique(pkey, return_inverse=True)
    k = (pkey[:, None] << 3) + np.arange(8, dtype=np.int64)
    keys[d] = k.reshape(-1)
    nnum[d] = keys[d].size
    nnum_nempty[d] = node_key.size
    addr = (pidx.astype(np.int64) << 3) | (node_key % 8)
    ch = -np.ones(nnum[d], dtype=np.int32)
    ch[addr] = np.arange(nnum_nempty[d], dtype=np.int32)
    children[d] = ch
    node_key = pkey if batch_size == 1 else (((pkey >> 45) << 48) | (pkey & ((np.int64(1) << 45) - 1)))

  d = full_depth                            # octree.py:263-270
  ch = -np.ones_like(children[d])
  nempty_idx = node_key if batch_size == 1 else (
      ((node_key >> 48) << (3 * d)) | (node_key & ((np.int64(1) << 48) - 1)))
  ch[nempty_idx] = np.arange(node_key.size, dtype=np.int32)
  children[d] = ch
  nnum_nempty[d] = node_key.size

  nleaf = counts.size                       # octree.py:273-281
  cnt = counts.astype(np.float32)[:, None]
  out = dict(keys=keys, children=children, nnum=nnum, nnum_nempty=nnum_nempty, idx=idx.astype(np.int64))
  out['points'] = scatter_add(pts, idx, nleaf) / cnt
  if normals is not None:
    s = scatter_add(np.asarray(normals, dtype=np.float32), idx, nleaf)
    nrm = np.sqrt((s.astype(np.float32) ** 2).sum(1, keepdims=True))
    out['normals'] = s / np.maximum(nrm, 1e-12)
  if features is not None:
    out['features'] = scatter_add(np.asarray(features, dtype=np.float32), idx, nleaf) / cnt
  return out


# ---------------------------------------------------------------- neighbours
def _range_grid(lo, hi):
  '''ocnn/utils.py:46-74.'''
  r = np.arange(lo, hi + 1, dtype=np.int64)
  g = np.stack(np.meshgrid(r, r, r, indexing='ij'), axis=-1)
  return g.reshape(-1, 3)


def neigh_luts():
  '''lut_parent / lut_child, ocnn/octree/octree.py:86-95.'''
  neigh_grid = _range_grid(2, 3)[:, None, :] + _range_grid(-1, 1)[None, :, :]   # (8, 27, 3)
  parent = neigh_grid // 2
  child = neigh_grid % 2
  return (parent * np.array([9, 3, 1])).sum(2), (child * np.array([4, 2, 1])).sum(2)


def construct_neigh_full(depth, batch_size):
  '''construct_neigh, dense branch, ocnn/octree/octree.py:411-428.'''
  nnum = 1 << (3 * depth)
  key = np.arange(nnum, dtype=np.int64)
  x, y, z, _ = key2xyz(key, depth)
  xyz = np.stack([x, y, z], axis=-1)[:, None, :] + _range_grid(-1, 1)[None]
  xyz = xyz.reshape(-1, 3)
  neigh = xyz2key(xyz[:, 0], xyz[:, 1], xyz[:, 2], depth=depth)
  neigh = neigh[None, :] + np.arange(batch_size, dtype=np.int64)[:, None] * nnum
  bound = 1 << depth
  invalid = np.logical_or((xyz < 0).any(1), (xyz >= bound).any(1))
  neigh[:, invalid] = -1
  return neigh.reshape(-1, 27)


def construct_neigh_from_parent(neigh_p, children_p):
  '''construct_neigh, parent-derived branch, ocnn/octree/octree.py:430-439.'''
  lut_parent, lut_child = neigh_luts()
  nempty = children_p >= 0
  n_p = neigh_p[nempty]                     # (N, 27)
  n_p = n_p[:, lut_parent]                  # (N, 8, 27)
  c_p = children_p[n_p].astype(np.int64)    # negative indices wrap, masked below
  invalid = np.logical_or(c_p < 0, n_p < 0)
  neigh = c_p * 8 + lut_child
  neigh[invalid] = -1
  return neigh.reshape(-1, 27)


def construct_all_neigh(children, nnum, depth, full_depth, batch_size):
  '''construct_all_neigh, ocnn/octree/octree.py:441-446.'''
  neighs = [None] * (depth + 1)
  for d in range(1, depth + 1):
    if d <= full_depth:
      neighs[d] = construct_neigh_full(d, batch_size)
    else:
      neighs[d] = construct_neigh_from_parent(neighs[d - 1], children[d - 1])
  return neighs


def nempty_index(children_d):
  '''ocnn/octree/octree.py:160-172.'''
  return np.nonzero(children_d >= 0)[0].astype(np.int64)


def get_neigh(neigh_d, children_d, kernel='333', stride=1, nempty=False):
  '''Octree.get_neigh + remap_nempty_neigh, ocnn/octree/octree.py:188-199, 490-523.'''
  def remap(n):
    n = n.copy()
    valid = n >= 0
    n[valid] = children_d[n[valid]].astype(np.int64)
    return n
  if stride == 1 and not nempty:
    neigh = neigh_d
  elif stride == 2 and not nempty:
    neigh = neigh_d[::8].copy()
  elif stride == 1 and nempty:
    neigh = remap(neigh_d[nempty_index(children_d)])
  elif stride == 2 and nempty:
    neigh = remap(neigh_d[::8])
  else:
    raise ValueError('Unsupported stride {}'.format(stride))
  if kernel == '333':
    return neigh
  return neigh[:, KERNEL_TAPS[kernel]]


# ---------------------------------------------------------------- pad / conv
def octree_pad(data, children_d, val=0.0):
  '''ocnn/nn/octree_pad.py:13-29.'''
  out = np.full((children_d.size, data.shape[1]), val, dtype=data.dtype)
  out[nempty_index(children_d)] = data
  return out


def octree_depad(data, children_d):
  '''ocnn/nn/octree_pad.py:32-39.'''
  return data[nempty_index(children_d)]


def octree2col(data, neigh):
  '''ocnn/nn/octree2col.py:15-39: (N, K, C) gather, zeros where neigh < 0.'''
  out = np.zeros((neigh.shape[0], neigh.shape[1], data.shape[1]), dtype=data.dtype)
  valid = neigh >= 0
  out[valid] = data[neigh[valid]]
  return out


def col2octree(col, neigh, dim_size):
  '''ocnn/nn/octree2col.py:42-53: scatter-add of (N, K, C) columns.'''
  valid = neigh >= 0
  return scatter_add(col[valid], neigh[valid], dim_size)


def conv_forward(data, weights, neigh):
  '''forward_gemm, ocnn/nn/octree_conv.py:115-143.  weights (K, Cin, Cout).'''
  col = octree2col(data, neigh)
  return col.reshape(col.shape[0], -1) @ weights.reshape(-1, weights.shape[2])


def conv_backward(grad, weights, neigh, in_h):
  '''backward_gemm, ocnn/nn/octree_conv.py:145-168: grad @ W^T then col2octree.'''
  K, cin, _ = weights.shape
  buf = grad @ weights.reshape(-1, weights.shape[2]).T
  return col2octree(buf.reshape(-1, K, cin), neigh, in_h)


def conv_weight_grad(data, grad, neigh):
  '''weight_gemm, ocnn/nn/octree_conv.py:170-202: col^T @ grad -> (K, Cin, Cout).'''
  col = octree2col(data, neigh)
  K, cin = col.shape[1], col.shape[2]
  return (col.reshape(col.shape[0], -1).T @ grad).reshape(K, cin, grad.shape[1])


def deconv_forward(data, weights, neigh, out_h):
  '''OctreeDeconvFunction.forward, ocnn/nn/octree_conv.py:257-275: weights
  (K, Cout, Cin); the conv's backward_gemm applied to the data.'''
  return conv_backward(data, weights, neigh, out_h)


def deconv_backward(grad, weights, neigh):
  '''OctreeDeconvFunction.backward (input), octree_conv.py:281-285.'''
  return conv_forward(grad, weights, neigh)


def deconv_weight_grad(data, grad, neigh):
  '''OctreeDeconvFunction.backward (weights), octree_conv.py:287-291.'''
  return conv_weight_grad(grad, data, neigh)


def dwconv_forward(data, weights, neigh):
  '''OctreeDWConvBase.forward_gemm, ocnn/nn/octree_dwconv.py:30-58; weights (K,1,C).'''
  col = octree2col(data, neigh)
  return np.einsum('ikc,kc->ic', col, weights.reshape(weights.shape[0], -1))


def dwconv_backward(grad, weights, neigh, in_h):
  '''OctreeDWConvBase.backward_gemm, ocnn/nn/octree_dwconv.py:60-86.'''
  buf = np.einsum('ic,kc->ikc', grad, weights.reshape(weights.shape[0], -1))
  return col2octree(buf, neigh, in_h)


def dwconv_weight_grad(data, grad, neigh):
  '''OctreeDWConvBase.weight_gemm, ocnn/nn/octree_dwconv.py:88-118.'''
  col = octree2col(data, neigh)
  return np.einsum('ikc,ic->kc', col, grad)[:, None, :]


# ---------------------------------------------------------------- pool / upsample
def max_pool(data, children_d, children_dm1, nempty=False):
  '''octree_max_pool, ocnn/nn/octree_pool.py:17-38.  Returns (out, indices).'''
  if nempty:
    data = octree_pad(data, children_d, -np.inf)
  v = data.reshape(-1, 8, data.shape[1])
  idx = v.argmax(1)
  out = v.max(1)
  if not nempty:
    out = octree_pad(out, children_dm1)
  return out, idx.astype(np.int64)


def nearest_upsample(data, children_d, children_dp1, nempty=False):
  '''octree_nearest_upsample, ocnn/nn/octree_interp.py:140-162.'''
  out = data
  if not nempty:
    out = octree_depad(out, children_d)
  out = np.repeat(out[:, None, :], 8, axis=1).reshape(-1, data.shape[1])
  if nempty:
    out = octree_depad(out, children_dp1)
  return out


# ---------------------------------------------------------------- norms
def batch_norm_train(x, weight, bias, eps=1e-5):
  '''torch.nn.BatchNorm1d (ocnn/nn/octree_norm.py:16) in training mode.
  Returns (out, batch mean, biased var).'''
  x64 = x.astype(np.float64)
  mean = x64.mean(0)
  var = x64.var(0)
  out = (x64 - mean) / np.sqrt(var + eps) * weight + bias
  return out.astype(np.float32), mean.astype(np.float32), var.astype(np.float32)


def group_norm(x, batch_id, batch_size, group, weights, bias, eps=1e-5):
  '''OctreeGroupNorm.forward, ocnn/nn/octree_norm.py:45-80.'''
  C = x.shape[1]
  cpg = C // group

  def adjust(t):
    if cpg > 1:
      t = t.reshape(-1, group, cpg).sum(-1, keepdims=True)
      t = np.repeat(t, cpg, axis=2).reshape(-1, C)
    return t
  ones = np.ones((x.shape[0], 1), dtype=x.dtype)
  count = scatter_add(ones, batch_id, batch_size) * cpg
  inv_count = 1.0 / (count + eps)
  mean = adjust(scatter_add(x, batch_id, batch_size) * inv_count)
  out = x - mean[batch_id]
  var = adjust(scatter_add(out ** 2, batch_id, batch_size) * inv_count)
  inv_std = 1.0 / np.sqrt(var + eps)
  out = out * inv_std[batch_id]
  return out * weights.reshape(1, -1) + bias.reshape(1, -1)


# ---------------------------------------------------------------- key search, point interpolation
def search_key(keys, query):
  '''Octree.search_key, ocnn/octree/octree.py:464-488: position of each query key in the
  sorted node keys, -1 if absent.'''
  keys = np.asarray(keys, dtype=np.int64)
  query = np.asarray(query, dtype=np.int64)
  idx = np.searchsorted(keys, query)
  ok = idx < keys.shape[0]
  ok[ok] = keys[idx[ok]] == query[ok]
  return np.where(ok, idx, -1).astype(np.int64)


def search_xyzb(keys, query, depth):
  '''Octree.search_xyzb, ocnn/octree/octree.py:448-462 (coordinates are truncated by xyz2key).'''
  return search_key(keys, xyz2key(query[:, 0], query[:, 1], query[:, 2], query[:, 3], depth))


def nearest_pts(data, keys, depth, pts, bound_check=False):
  '''octree_nearest_pts, ocnn/nn/octree_interp.py:16-48.  `keys`: the node keys that the rows of
  `data` belong to (all nodes, or the non-empty ones).  Returns (out, idx with -1 = no row).'''
  idx = search_xyzb(keys, pts, depth)
  valid = idx > -1
  if bound_check:
    valid &= np.logical_and(pts[:, :3] >= 0, pts[:, :3] < 2 ** depth).all(1)
  out = np.zeros((pts.shape[0], data.shape[1]), dtype=data.dtype)
  out[valid] = data[idx[valid]]
  return out, np.where(valid, idx, -1)


def nearest_pts_backward(grad, idx, n_rows):
  '''Gradient of nearest_pts with respect to data: rows of grad added at idx (>= 0).'''
  gd = np.zeros((n_rows, grad.shape[1]), dtype=np.float64)
  v = idx >= 0
  np.add.at(gd, idx[v], grad[v].astype(np.float64))
  return gd.astype(grad.dtype)


_GRID = np.array([[0, 0, 0], [0, 0, 1], [0, 1, 0], [0, 1, 1],
                  [1, 0, 0], [1, 0, 1], [1, 1, 0], [1, 1, 1]], dtype=np.float32)


def linear_corners(keys, depth, pts, bound_check=False):
  '''Steps 1-2 of octree_linear_pts, ocnn/nn/octree_interp.py:63-88: the 8 surrounding cell
  centres of every point as (idx (N,8) with -1 = absent, weight (N,8) float32).'''
  xyzf = pts[:, :3].astype(np.float32) - np.float32(0.5)
  xyzi = np.floor(xyzf)
  frac = xyzf - xyzi
  xyzn = (xyzi[:, None, :] + _GRID[None]).reshape(-1, 3)
  batch = np.repeat(pts[:, 3], 8)
  idx = search_xyzb(keys, np.concatenate([xyzn, batch[:, None]], axis=1), depth)
  valid = idx > -1
  if bound_check:
    valid &= np.logical_and(xyzn >= 0, xyzn < 2 ** depth).all(1)
  w = np.abs(np.prod((np.float32(1.0) - _GRID)[None] - frac[:, None, :], axis=2)).astype(np.float32)
  return np.where(valid, idx, -1).reshape(-1, 8), w


def linear_pts(data, keys, depth, pts, bound_check=False):
  '''octree_linear_pts, ocnn/nn/octree_interp.py:51-98: weighted mean of the existing corners,
  out = (sum_j w_j data[idx_j]) / (sum_j w_j + 1e-12).'''
  idx, w = linear_corners(keys, depth, pts, bound_check)
  v = idx >= 0
  wv = np.where(v, w, 0).astype(np.float64)
  g = data.astype(np.float64)[np.where(v, idx, 0)]                 # (N, 8, C)
  out = (g * wv[:, :, None]).sum(1)
  norm = wv.sum(1, keepdims=True)
  return (out / (norm + 1e-12)).astype(data.dtype)


def linear_pts_backward(grad, keys, depth, pts, n_rows, bound_check=False):
  '''Gradient of linear_pts with respect to data.'''
  idx, w = linear_corners(keys, depth, pts, bound_check)
  v = idx >= 0
  wv = np.where(v, w, 0).astype(np.float64)
  coef = wv / (wv.sum(1, keepdims=True) + 1e-12)                   # (N, 8)
  gd = np.zeros((n_rows, grad.shape[1]), dtype=np.float64)
  contrib = coef[:, :, None] * grad.astype(np.float64)[:, None, :]
  np.add.at(gd, idx[v], contrib[v])
  return gd.astype(grad.dtype)


# ---------------------------------------------------------------- average / global pooling, align, voxels
def avg_pool(data, neigh):
  '''octree_avg_pool, ocnn/nn/octree_pool.py:68-103: mean over the existing entries of each row of
  the neighbour table, weight 1 / (count + 1e-8).  Returns (out, val) with val the row weights.'''
  mask = neigh >= 0
  val = (1.0 / (mask.sum(1) + 1e-8)).astype(np.float32)
  g = data.astype(np.float64)[np.where(mask, neigh, 0)] * mask[:, :, None]
  return (g.sum(1) * val[:, None].astype(np.float64)).astype(data.dtype), val


def avg_pool_backward(grad, neigh, n_in):
  '''Gradient of avg_pool with respect to data.'''
  mask = neigh >= 0
  val = 1.0 / (mask.sum(1) + 1e-8)
  gd = np.zeros((n_in, grad.shape[1]), dtype=np.float64)
  r, k = np.nonzero(mask)
  np.add.at(gd, neigh[r, k], grad.astype(np.float64)[r] * val[r, None])
  return gd.astype(grad.dtype)


def global_pool(data, batch_id, batch_size):
  '''octree_global_pool, ocnn/nn/octree_pool.py:106-124: per-octree mean (count clamped to >= 1).
  Returns (out, count).'''
  count = np.bincount(batch_id, minlength=batch_size).astype(np.float64)
  count[count < 1] = 1
  s = np.zeros((batch_size, data.shape[1]), dtype=np.float64)
  np.add.at(s, batch_id, data.astype(np.float64))
  return (s / count[:, None]).astype(data.dtype), count


def global_pool_backward(grad, batch_id, count):
  return (grad.astype(np.float64)[batch_id] / count[batch_id, None]).astype(grad.dtype)


def align(value, key, query):
  '''search_value / octree_align, ocnn/nn/octree_align.py:13-48: value of the node with the same
  key, zeros where the query key does not exist.  Returns (out fp32, idx).'''
  idx = search_key(key, query)
  out = np.zeros((query.shape[0], value.shape[1]), dtype=np.float32)
  out[idx >= 0] = value[idx[idx >= 0]]
  return out, idx


def octree2voxel(data, x, y, z, b, depth, batch_size):
  '''octree2voxel, ocnn/nn/octree2vox.py:13-31.'''
  num = 1 << depth
  vox = np.zeros((batch_size, num, num, num, data.shape[1]), dtype=data.dtype)
  vox[b, x, y, z] = data
  return vox

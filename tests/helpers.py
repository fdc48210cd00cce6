"""Shared helpers for the parity tests."""
import numpy as np


def split_by(arr, sizes):
  out, o = [], 0
  for s in sizes:
    out.append(arr[o:o + int(s)])
    o += int(s)
  assert o == arr.shape[0]
  return out


def rel_errors(a, b):
  r''' (relative L2 error, max-norm error) of a against the expectation b. '''
  a = np.asarray(a, dtype=np.float64)
  b = np.asarray(b, dtype=np.float64)
  l2 = np.linalg.norm(a - b) / max(np.linalg.norm(b), 1e-30)
  mx = np.abs(a - b).max() / max(np.abs(b).max(), 1e-30) if a.size else 0.0
  return l2, mx


def assert_close(a, b, tol, what=''):
  assert a.shape == b.shape, '%s: shape %s vs %s' % (what, a.shape, b.shape)
  l2, mx = rel_errors(a, b)
  assert l2 <= tol and mx <= tol, '%s: rel L2 %.3e, max-norm %.3e > %.1e' % (what, l2, mx, tol)


def conv_case(syn, ci):
  r''' Unpacks conv case `ci` of tests/golden/synthetic.npz. '''
  tag = 'c%02d' % ci
  meta = syn[tag + '_meta']
  c = dict(op='conv' if meta[0] == 0 else 'deconv', stride=int(meta[1]), nempty=bool(meta[2]),
           cin=int(meta[3]), cout=int(meta[4]), depth=int(meta[5]), use_bias=bool(meta[6]),
           kernel_size=[int(v) for v in meta[7:10]])
  c['kernel'] = ''.join(str(v) for v in c['kernel_size'])
  for k in ('w', 'x', 'y', 'gy', 'gx', 'gw'):
    c[k] = syn[tag + '_' + k]
  if c['use_bias']:
    c['b'], c['gb'] = syn[tag + '_b'], syn[tag + '_gb']
  return c


def octree_from_golden(syn):
  r''' Per-depth keys / children / neigh lists of the synthetic golden octree. '''
  nnum = syn['nnum']
  keys = split_by(syn['key'], nnum)
  children = split_by(syn['child'], nnum)
  neighs = [None] + split_by(syn['neigh'].astype(np.int64), nnum[1:])
  return keys, children, neighs


def tap_sort_key(valid, chunk_log2=0):
  """Sort key of oc_tap_order for a (rows, K) boolean matrix of valid taps: the mask with its bits
  reordered (taps whose frequency is farthest from one half are most significant, ties to the
  lower tap), under the number of the row's chunk of 2**chunk_log2 rows."""
  valid = np.asarray(valid).astype(np.int64)
  n, K = valid.shape
  score = np.abs(2 * valid.sum(axis=0) - n)
  ranked = sorted(range(K), key=lambda t: (-int(score[t]), t))       # most significant first
  bitpos = np.empty(K, np.int64)
  for rank, t in enumerate(ranked):
    bitpos[t] = K - 1 - rank
  key = (valid << bitpos[None, :]).sum(axis=1)
  if chunk_log2:
    key = key | ((np.arange(n, dtype=np.int64) >> chunk_log2) << K)
  return key

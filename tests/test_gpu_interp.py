"""GPU parity of key search and point interpolation (Octree.search_key / search_xyzb,
octree_nearest_pts, octree_linear_pts, OctreeInterp) against the reference's stored answers
for the merged octree 4+5 (test/data/search_key.npz, test/data/interp.npz) and against its
gradients on seeded points, through the C ABI."""
import numpy as np
import pytest
import torch

import ocnn_pytorch_b200 as b200
from oracle import octree_oracle as orc
from gpu_utils import dev, to_np, build

pytestmark = pytest.mark.gpu


def T(a, dtype=None, grad=False):
  t = torch.from_numpy(np.ascontiguousarray(a)).to(dev())
  if dtype is not None:
    t = t.to(dtype)
  return t.requires_grad_() if grad else t


@pytest.fixture(scope='module')
def octree45(golden):
  d, b45 = golden['octrees'], golden['batch45']
  pts = np.concatenate([d['4_points'], d['5_points']])
  nrm = np.concatenate([d['4_normals'], d['5_normals']])
  bid = np.concatenate([np.zeros(len(d['4_points']), np.float32), np.ones(len(d['5_points']), np.float32)])
  octree, _ = build(pts, nrm, batch_id=bid, batch_size=2, depth=int(b45['depth']), full_depth=int(b45['full_depth']))
  return octree


def test_search_key_golden(golden, octree45):
  it = golden['interp']
  depth = 5
  xyzb = T(it['sk_xyzb'].astype(np.int64))
  key = b200.octree.xyz2key(xyzb[:, 0], xyzb[:, 1], xyzb[:, 2], xyzb[:, 3], depth)
  for nempty, want in ((False, it['sk_idx']), (True, it['sk_idx_ne'])):
    got = octree45.search_key(key, depth, nempty)
    assert got.dtype == torch.int64
    assert np.array_equal(to_np(got), want)
    assert np.array_equal(to_np(octree45.search_xyzb(xyzb, depth, nempty)), want)
    # float coordinates are truncated like the reference's .long()
    assert np.array_equal(to_np(octree45.search_xyzb(xyzb.float() + 0.25, depth, nempty)), want)
  # every node finds itself, a key between two nodes and keys past both ends are absent
  keys = octree45.keys[depth]
  assert torch.equal(octree45.search_key(keys, depth), torch.arange(keys.numel(), device=dev()))
  ne = octree45.key(depth, True)
  assert torch.equal(octree45.search_key(ne, depth, True), torch.arange(ne.numel(), device=dev()))
  probe = torch.tensor([-5, int(keys[-1]) + 1, 1 << 60], device=dev())
  assert (octree45.search_key(probe, depth) == -1).all()
  assert octree45.search_key(torch.empty(0, dtype=torch.int64, device=dev()), depth).numel() == 0


def test_interp_golden(golden, octree45):
  it = golden['interp']
  depth = 5
  data, pts = T(it['it_data']), T(it['it_pts'])
  data_ne = b200.nn.octree_depad(data, octree45, depth)
  for name, fn in (('linear', b200.nn.octree_linear_pts), ('near', b200.nn.octree_nearest_pts)):
    for ne, dd in ((False, data), (True, data_ne)):
      got = fn(dd, octree45, depth, pts, nempty=ne)
      assert np.allclose(to_np(got), it['it_' + name + ('_ne' if ne else '')], atol=1e-6), (name, ne)


@pytest.mark.parametrize('nempty', [False, True])
@pytest.mark.parametrize('bound_check', [False, True])
def test_interp_gradients_and_bound_check(golden, octree45, nempty, bound_check):
  it = golden['interp']
  depth = 5
  tag = '_ne' if nempty else ''
  pts = T(it['g_pts'])
  gy = T(it['g_gy' + tag])
  for name, fn in (('linear', b200.nn.octree_linear_pts), ('near', b200.nn.octree_nearest_pts)):
    dd = T(it['g_data' + tag], grad=True)
    y = fn(dd, octree45, depth, pts.clone(), nempty=nempty, bound_check=bound_check)
    y.backward(gy)
    key = 'g_%s%s_bc%d' % (name, tag, int(bound_check))
    assert np.allclose(to_np(y), it[key], atol=1e-5), key
    assert np.allclose(to_np(dd.grad), it[key + '_grad'], atol=1e-5), key
  # half precision: same corners, fp32 accumulation, rounded output
  dd = T(it['g_data' + tag], torch.float16)
  y16 = b200.nn.octree_linear_pts(dd, octree45, depth, pts.clone(), nempty=nempty, bound_check=bound_check)
  assert y16.dtype == torch.float16
  assert np.allclose(to_np(y16), it['g_linear%s_bc%d' % (tag, int(bound_check))], atol=2e-2)


def test_interp_module_and_corners(golden, octree45):
  it = golden['interp']
  depth = 5
  m = b200.nn.OctreeInterp('linear', nempty=True, bound_check=True, rescale_pts=True)
  pts = T(it['m_pts'].copy())
  out = m(T(it['g_data_ne']), octree45, depth, pts)
  assert np.allclose(to_np(out), it['m_out'], atol=1e-5)
  # the corner kernel against the oracle: indices exact, weights to rounding
  keys = octree45.key(depth, True)
  p = T(it['g_pts'])
  L = b200._lib
  for bc in (0, 1):
    idx8 = torch.empty(p.shape[0], 8, dtype=torch.int64, device=dev())
    w8 = torch.empty(p.shape[0], 8, dtype=torch.float32, device=dev())
    L.call('oc_interp_corners', L.ptr(keys), keys.numel(), L.ptr(p), p.shape[0], depth, bc, L.ptr(idx8), L.ptr(w8),
           L.stream(dev()))
    eidx, ew = orc.linear_corners(to_np(keys), depth, it['g_pts'], bool(bc))
    assert np.array_equal(to_np(idx8), eidx)
    assert np.allclose(to_np(w8), ew, atol=1e-6)
  with pytest.raises(AssertionError):
    b200.nn.octree_nearest_pts(T(it['g_data']), octree45, depth, p, nempty=True)      # wrong row count
  with pytest.raises(b200._lib.OctConvError):
    L.call('oc_interp_corners', L.ptr(keys), keys.numel(), L.ptr(p), p.shape[0], 17, 0, L.ptr(idx8), L.ptr(w8),
           L.stream(dev()))

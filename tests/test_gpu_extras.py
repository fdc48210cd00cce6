"""GPU parity of octree_avg_pool, octree_global_pool, octree_align, octree2voxel and
OctreeDropPath against the reference's outputs and gradients on the merged octree 4+5
(tests/golden/extras.npz), through the C ABI."""
import numpy as np
import pytest
import torch

import ocnn_pytorch_b200 as b200
from gpu_utils import dev, to_np, build

pytestmark = pytest.mark.gpu


def T(a, dtype=None, grad=False):
  t = torch.from_numpy(np.ascontiguousarray(a)).to(dev())
  if dtype is not None:
    t = t.to(dtype)
  return t.requires_grad_() if grad else t


def _octree(golden, order):
  d, b45 = golden['octrees'], golden['batch45']
  a, b = order
  pts = np.concatenate([d['%d_points' % a], d['%d_points' % b]])
  nrm = np.concatenate([d['%d_normals' % a], d['%d_normals' % b]])
  bid = np.concatenate([np.zeros(len(d['%d_points' % a]), np.float32), np.ones(len(d['%d_points' % b]), np.float32)])
  octree, _ = build(pts, nrm, batch_id=bid, batch_size=2, depth=int(b45['depth']), full_depth=int(b45['full_depth']))
  return octree


@pytest.fixture(scope='module')
def octree45(golden):
  return _octree(golden, (4, 5))


@pytest.fixture(scope='module')
def octree54(golden):
  return _octree(golden, (5, 4))


@pytest.mark.parametrize('nempty', [False, True])
def test_avg_and_global_pool(golden, octree45, nempty):
  ex = golden['extras']
  tag = '_ne' if nempty else ''
  depth = 5
  for kernel, stride in (('222', 2), ('333', 2), ('333', 1)):
    key = 'avg_%s_%d%s' % (kernel, stride, tag)
    x = T(ex['x' + tag], grad=True)
    y = b200.nn.octree_avg_pool(x, octree45, depth, kernel, stride, nempty)
    y.backward(T(ex[key + '_gy']))
    assert np.allclose(to_np(y), ex[key], atol=1e-6), key
    assert np.allclose(to_np(x.grad), ex[key + '_gx'], atol=1e-6), key
  m = b200.nn.OctreeAvgPool([2], 2, nempty)
  assert np.allclose(to_np(m(T(ex['x' + tag]), octree45, depth)), ex['avg_222_2' + tag], atol=1e-6)
  x = T(ex['x' + tag], grad=True)
  y = b200.nn.OctreeGlobalPool(nempty)(x, octree45, depth)
  y.backward(T(ex['glob%s_gy' % tag]))
  assert np.allclose(to_np(y), ex['glob' + tag], atol=1e-6)
  assert np.allclose(to_np(x.grad), ex['glob%s_gx' % tag], atol=1e-7)
  y16 = b200.nn.octree_global_pool(T(ex['x' + tag], torch.float16), octree45, depth, nempty)
  assert y16.dtype == torch.float16 and np.allclose(to_np(y16), ex['glob' + tag], atol=2e-3)


@pytest.mark.parametrize('nempty', [False, True])
def test_align_and_voxel(golden, octree45, octree54, nempty):
  ex = golden['extras']
  tag = '_ne' if nempty else ''
  depth = 5
  x = T(ex['x' + tag], grad=True)
  y = b200.nn.octree_align(x, octree45, octree54, depth, nempty)
  y.backward(T(ex['align%s_gy' % tag]))
  assert y.dtype == torch.float32
  assert np.array_equal(to_np(y), ex['align' + tag])
  assert np.allclose(to_np(x.grad), ex['align%s_gx' % tag], atol=1e-6)
  # an octree aligned with itself returns its own features
  assert torch.equal(b200.nn.octree_align(x.detach(), octree45, octree45, depth, nempty), x.detach())
  v_in = T(ex['vox_x' + tag], grad=True)
  v = b200.nn.Octree2Voxel(nempty)(v_in, octree45, 4)
  v.backward(T(ex['vox%s_gy' % tag]))
  assert np.array_equal(to_np(v), ex['vox' + tag])
  assert np.array_equal(to_np(v_in.grad), ex['vox%s_gx' % tag])


def test_drop_path(octree45):
  depth = 5
  n = int(octree45.nnum[depth])
  x = torch.randn(n, 7, device=dev(), requires_grad=True)
  m = b200.nn.OctreeDropPath(0.5, nempty=False, scale_by_keep=True)
  m.eval()
  assert m(x, octree45, depth) is x
  m.train()
  offs = octree45.batch_offsets(depth, False)
  seen = set()
  for seed in range(8):
    torch.manual_seed(seed)
    y = m(x, octree45, depth)
    mask = m.last_mask.view(-1)
    seen.update(mask.tolist())
    want = torch.cat([x[offs[b]:offs[b + 1]] * mask[b] for b in range(2)])
    assert torch.equal(y, want.to(y.dtype))
    g = torch.randn_like(y)
    x.grad = None
    y.backward(g)
    want_g = torch.cat([g[offs[b]:offs[b + 1]] * mask[b] for b in range(2)])
    assert torch.equal(x.grad, want_g)
  assert seen == {0.0, 2.0}                      # dropped, or kept and divided by the keep probability
  m2 = b200.nn.OctreeDropPath(0.3, scale_by_keep=False).train()
  torch.manual_seed(0)
  y = m2(x.detach().half(), octree45, depth)
  assert y.dtype == torch.float16 and set(m2.last_mask.view(-1).tolist()) <= {0.0, 1.0}
  assert b200.nn.OctreeDropPath(0.0).train()(x, octree45, depth) is x

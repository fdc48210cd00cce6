"""Generates the golden vectors under tests/golden/ by running the REFERENCE
implementation (octree-nn/ocnn-pytorch, pure PyTorch on CPU).

Run from the repository root on a machine that has the reference checkout:

    REFERENCE_ROOT=/path/to/ocnn-pytorch python tests/golden/make_golden.py

Outputs (all produced by the reference's own code, never by this repository's
kernels or oracle):
  hand3.npz      the 3-point octree of the reference's test/test_octree.py:19-85
  octrees.npz    the reference's fixtures test/data/octree/test_00{1..5}.npz
                 (points, normals and their stored key/child/nnum) re-packed
  batch45.npz    test/data/batch_45.npz re-packed (merged octree 4+5 incl. neigh)
  interp.npz     test/data/search_key.npz and test/data/interp.npz re-packed (queries and
                 the stored answers for the merged octree 4+5), plus the reference's
                 gradients, bound_check and out-of-range behaviour on seeded points
  extras.npz     average / global pooling, octree_align, octree2voxel on the merged octree 4+5
                 (forward and gradients, seeded features)
  synthetic.npz  a small seeded batch: octree, neighbour tables and variants,
                 conv / deconv / dwconv forward + gradients, pooling, upsampling,
                 normalisation, key encode/decode edge cases
"""
import os
import sys

import numpy as np
import torch

REF = os.environ.get('REFERENCE_ROOT', '/root/reference')
ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, REF)
sys.path.insert(0, ROOT)
os.environ['OCNN_DISABLE_TRITON'] = '1'

import ocnn  # noqa: E402  (the reference)
import ocnn_pytorch_b200 as b200  # noqa: E402  (only for the seeded cloud generator)

OUT = os.path.dirname(os.path.abspath(__file__))
torch.manual_seed(0)


def cat_or_empty(lst):
  return torch.cat([t.reshape(-1) for t in lst]).numpy()


def hand3():
  points = torch.Tensor([[-1, -1, -1], [0, 0, -1], [0.0625, 0.0625, -1]])
  normals = torch.Tensor([[1, 0, 0], [-1, 0, 0], [0, 1, 0]])
  features = torch.Tensor([[1, -1], [2, -2], [3, -3]])
  pc = ocnn.octree.Points(points, normals, features)
  octree = ocnn.octree.Octree(depth=5, full_depth=1)
  idx = octree.build_octree(pc)
  # the literal expectations of the reference test (test/test_octree.py:31-84)
  assert octree.nnum.tolist() == [1, 8, 16, 16, 16, 16]
  assert octree.nnum_nempty.tolist() == [1, 2, 2, 2, 2, 3]
  assert octree.keys[5].tolist() == [0, 1, 2, 3, 4, 5, 6, 7, 24576, 24577, 24578, 24579, 24580,
                                     24581, 24582, 24583]
  assert octree.children[5].tolist() == [0, -1, -1, -1, -1, -1, -1, -1, 1, -1, -1, -1, -1, -1, 2, -1]
  octree.construct_all_neigh()
  np.savez_compressed(
      os.path.join(OUT, 'hand3.npz'), points=points.numpy(), normals=normals.numpy(),
      features=features.numpy(), depth=5, full_depth=1, nnum=octree.nnum.numpy(),
      nnum_nempty=octree.nnum_nempty.numpy(), key=cat_or_empty(octree.keys),
      child=cat_or_empty(octree.children), idx=idx.numpy(),
      out_points=octree.points[5].numpy(), out_normals=octree.normals[5].numpy(),
      out_features=octree.features[5].numpy(),
      neigh=torch.cat(octree.neighs[1:], 0).numpy())


def ref_fixtures():
  out = {}
  for i in range(1, 6):
    d = np.load(os.path.join(REF, 'test/data/octree/test_%03d.npz' % i))
    pc = ocnn.octree.Points(torch.from_numpy(d['points']), torch.from_numpy(d['normals']))
    octree = ocnn.octree.Octree(d['depth'].item(), d['full_depth'].item())
    idx = octree.build_octree(pc)
    # the stored arrays are what the reference's own test compares against
    assert np.array_equal(torch.cat(octree.keys).numpy(), d['key'])
    assert np.array_equal(torch.cat(octree.children).numpy(), d['child'])
    for k in ('points', 'normals', 'depth', 'full_depth', 'nnum', 'nnum_nempty', 'key', 'child'):
      out['%d_%s' % (i, k)] = d[k]
    out['%d_feature' % i] = d['feature'][:, :3]
    out['%d_idx' % i] = idx.numpy().astype(np.int32)
    out['%d_avg_points' % i] = octree.points[octree.depth].numpy()
  np.savez_compressed(os.path.join(OUT, 'octrees.npz'), **out)

  d = np.load(os.path.join(REF, 'test/data/batch_45.npz'))
  np.savez_compressed(os.path.join(OUT, 'batch45.npz'), depth=d['depth'], full_depth=d['full_depth'],
                      key=d['key'], child=d['child'], nnum=d['nnum'], nnum_nempty=d['nnum_nempty'],
                      feature=d['feature'][:, :3], neigh=d['neigh'])


def interp():
  """Key search and point interpolation (test_octree.py:138-155, test_octree_interp.py:20-42)."""
  out = {}
  octs = []
  for i in (4, 5):
    d = np.load(os.path.join(REF, 'test/data/octree/test_%03d.npz' % i))
    pc = ocnn.octree.Points(torch.from_numpy(d['points']), torch.from_numpy(d['normals']))
    o = ocnn.octree.Octree(d['depth'].item(), d['full_depth'].item())
    o.build_octree(pc)
    octs.append(o)
  octree = ocnn.octree.merge_octrees(octs)
  octree.construct_all_neigh()
  depth = 5
  sk = np.load(os.path.join(REF, 'test/data/search_key.npz'))
  xyzb = torch.from_numpy(sk['xyzb']).long()
  key = ocnn.octree.xyz2key(xyzb[:, 0], xyzb[:, 1], xyzb[:, 2], xyzb[:, 3], depth)
  # the stored answers are what the reference's own test compares against
  assert np.array_equal(octree.search_key(key, depth, False).numpy(), sk['idx'])
  assert np.array_equal(octree.search_key(key, depth, True).numpy(), sk['idx_ne'])
  out['sk_xyzb'], out['sk_idx'], out['sk_idx_ne'] = sk['xyzb'], sk['idx'], sk['idx_ne']

  it = np.load(os.path.join(REF, 'test/data/interp.npz'))
  data = torch.from_numpy(it['data'])
  pts = torch.from_numpy(it['pts'])
  data_ne = ocnn.nn.octree_depad(data, octree, depth)
  for name, fn in (('linear', ocnn.nn.octree_linear_pts), ('near', ocnn.nn.octree_nearest_pts)):
    for ne, dd in ((False, data), (True, data_ne)):
      got = fn(dd, octree, depth, pts, nempty=ne)
      assert np.allclose(got.numpy(), it[name + ('_ne' if ne else '')], atol=1e-6)
  for k in ('pts', 'data', 'linear', 'linear_ne', 'near', 'near_ne'):
    out['it_' + k] = it[k]

  # gradients, bound_check, points outside the box and the module with rescaling (seeded)
  g = torch.Generator().manual_seed(5)
  C = 6
  pts2 = torch.rand(3000, 4, generator=g)
  pts2[:, :3] = pts2[:, :3] * 36.0 - 2.0              # a band of 2 cells outside [0, 32) on every side
  pts2[:, 3] = (pts2[:, 3] > 0.5).float()
  out['g_pts'] = pts2.numpy()
  for ne in (False, True):
    n = int(octree.nnum_nempty[depth] if ne else octree.nnum[depth])
    dd = torch.randn(n, C, generator=g, requires_grad=True)
    gy = torch.randn(3000, C, generator=g)
    tag = '_ne' if ne else ''
    out['g_data' + tag] = dd.detach().numpy()
    out['g_gy' + tag] = gy.numpy()
    for name, fn in (('linear', ocnn.nn.octree_linear_pts), ('near', ocnn.nn.octree_nearest_pts)):
      for bc in (False, True):
        dd.grad = None
        y = fn(dd, octree, depth, pts2.clone(), nempty=ne, bound_check=bc)
        y.backward(gy)
        out['g_%s%s_bc%d' % (name, tag, int(bc))] = y.detach().numpy()
        out['g_%s%s_bc%d_grad' % (name, tag, int(bc))] = dd.grad.numpy().copy()
  m = ocnn.nn.OctreeInterp('linear', nempty=True, bound_check=True, rescale_pts=True)
  praw = torch.rand(500, 4, generator=g) * 2 - 1
  praw[:, 3] = (praw[:, 3] > 0).float()
  out['m_pts'] = praw.numpy().copy()
  dd = torch.from_numpy(out['g_data_ne'])
  out['m_out'] = m(dd, octree, depth, praw.clone()).numpy()
  np.savez_compressed(os.path.join(OUT, 'interp.npz'), **out)


def _batch_octree(ids):
  octs = []
  for i in ids:
    d = np.load(os.path.join(REF, 'test/data/octree/test_%03d.npz' % i))
    pc = ocnn.octree.Points(torch.from_numpy(d['points']), torch.from_numpy(d['normals']))
    o = ocnn.octree.Octree(d['depth'].item(), d['full_depth'].item())
    o.build_octree(pc)
    octs.append(o)
  octree = ocnn.octree.merge_octrees(octs)
  octree.construct_all_neigh()
  return octree


def extras():
  """octree_avg_pool, octree_global_pool (octree_pool.py:68-124), octree_align (octree_align.py),
  octree2voxel (octree2vox.py) of the reference on the merged octree 4+5."""
  out = {}
  octree = _batch_octree((4, 5))
  other = _batch_octree((5, 4))          # same shapes in the other order: keys differ in the batch bits
  g = torch.Generator().manual_seed(11)
  C, depth = 5, 5
  for ne in (False, True):
    tag = '_ne' if ne else ''
    n = int(octree.nnum_nempty[depth] if ne else octree.nnum[depth])
    x = torch.randn(n, C, generator=g, requires_grad=True)
    out['x' + tag] = x.detach().numpy()
    for kernel, stride in (('222', 2), ('333', 2), ('333', 1)):
      x.grad = None
      y = ocnn.nn.octree_avg_pool(x, octree, depth, kernel, stride, ne)
      gy = torch.randn(y.shape, generator=g)
      y.backward(gy)
      key = 'avg_%s_%d%s' % (kernel, stride, tag)
      out[key], out[key + '_gy'], out[key + '_gx'] = y.detach().numpy(), gy.numpy(), x.grad.numpy().copy()
    x.grad = None
    y = ocnn.nn.octree_global_pool(x, octree, depth, ne)
    gy = torch.randn(y.shape, generator=g)
    y.backward(gy)
    out['glob' + tag], out['glob%s_gy' % tag], out['glob%s_gx' % tag] = y.detach().numpy(), gy.numpy(), x.grad.numpy().copy()
    x.grad = None
    y = ocnn.nn.octree_align(x, octree, other, depth, ne)
    gy = torch.randn(y.shape, generator=g)
    y.backward(gy)
    out['align' + tag], out['align%s_gy' % tag], out['align%s_gx' % tag] = y.detach().numpy(), gy.numpy(), x.grad.numpy().copy()
  for ne in (False, True):
    tag = '_ne' if ne else ''
    d4 = 4
    n = int(octree.nnum_nempty[d4] if ne else octree.nnum[d4])
    x = torch.randn(n, 3, generator=g, requires_grad=True)
    v = ocnn.nn.octree2voxel(x, octree, d4, ne)
    gy = torch.randn(v.shape, generator=g)
    v.backward(gy)
    out['vox_x' + tag], out['vox' + tag], out['vox%s_gy' % tag], out['vox%s_gx' % tag] = \
        x.detach().numpy(), v.detach().numpy(), gy.numpy(), x.grad.numpy().copy()
  np.savez_compressed(os.path.join(OUT, 'extras.npz'), **out)


def synthetic():
  out = {}
  depth, full_depth, B = 5, 2, 2
  clouds = [b200.synthetic.spheres_cloud(1000 * 1 + i, 3000) for i in range(B)]
  feats = [np.random.default_rng(77 + i).standard_normal((3000, 3)).astype(np.float32) for i in range(B)]
  pcs = [ocnn.octree.Points(torch.from_numpy(p), torch.from_numpy(n), torch.from_numpy(f))
         for (p, n), f in zip(clouds, feats)]
  pc = ocnn.octree.merge_points(pcs)
  octree = ocnn.octree.Octree(depth, full_depth, batch_size=B)
  idx = octree.build_octree(pc)
  octree.construct_all_neigh()
  out['points'] = pc.points.numpy()
  out['normals'] = pc.normals.numpy()
  out['features'] = pc.features.numpy()
  out['batch_id'] = pc.batch_id.numpy()
  out['depth'], out['full_depth'], out['batch_size'] = depth, full_depth, B
  out['nnum'] = octree.nnum.numpy()
  out['nnum_nempty'] = octree.nnum_nempty.numpy()
  out['key'] = cat_or_empty(octree.keys)
  out['child'] = cat_or_empty(octree.children)
  out['idx'] = idx.numpy().astype(np.int32)
  out['out_points'] = octree.points[depth].numpy()
  out['out_normals'] = octree.normals[depth].numpy()
  out['out_features'] = octree.features[depth].numpy()
  out['neigh'] = torch.cat(octree.neighs[1:], 0).numpy().astype(np.int32)
  for d in (3, depth):
    for kernel in ('333', '222', '311', '131', '113', '331', '313', '133'):
      for stride in (1, 2):
        for nempty in (False, True):
          ng = octree.get_neigh(d, kernel, stride, nempty)
          out['gn_%d_%s_%d_%d' % (d, kernel, stride, int(nempty))] = ng.numpy().astype(np.int32)

  # ---- convolution cases: (name, module ctor, depth, Cin, Cout)
  g = torch.Generator().manual_seed(5)
  cases = []
  for kernel in ([3], [2], [3, 1, 1], [1, 3, 3], [3, 1, 3]):
    for stride in (1, 2):
      for nempty in (False, True):
        cases.append(('conv', kernel, stride, nempty, 5, 7))
        cases.append(('deconv', kernel, stride, nempty, 5, 7))
  cases.append(('conv', [3], 1, False, 16, 32))
  cases.append(('conv', [3], 1, True, 32, 16))
  cases.append(('deconv', [2], 2, True, 32, 16))
  cases.append(('conv', [2], 2, False, 16, 32))
  for ci, (op, kernel, stride, nempty, cin, cout) in enumerate(cases):
    d = 3 if op == 'deconv' and stride == 2 else 4
    cls = ocnn.nn.OctreeConv if op == 'conv' else ocnn.nn.OctreeDeconv
    m = cls(cin, cout, kernel, stride, nempty, method='block_gemm', use_bias=(ci % 3 == 0))
    with torch.no_grad():
      m.weights.copy_(torch.randn(m.weights.shape, generator=g) * 0.2)
      if m.use_bias:
        m.bias.copy_(torch.randn(cout, generator=g))
    n_in = int(octree.nnum_nempty[d] if nempty else octree.nnum[d])
    x = torch.randn(n_in, cin, generator=g, requires_grad=True)
    y = m(x, octree, d)
    gy = torch.randn(y.shape, generator=g)
    y.backward(gy)
    tag = 'c%02d' % ci
    out[tag + '_meta'] = np.array([0 if op == 'conv' else 1, stride, int(nempty), cin, cout, d,
                                   int(m.use_bias)] + m.kernel_size, dtype=np.int64)
    out[tag + '_w'] = m.weights.detach().numpy()
    if m.use_bias:
      out[tag + '_b'] = m.bias.detach().numpy()
      out[tag + '_gb'] = m.bias.grad.numpy()
    out[tag + '_x'] = x.detach().numpy()
    out[tag + '_y'] = y.detach().numpy()
    out[tag + '_gy'] = gy.numpy()
    out[tag + '_gx'] = x.grad.numpy()
    out[tag + '_gw'] = m.weights.grad.numpy()
  out['n_conv_cases'] = len(cases)

  # ---- depth-wise conv
  dcases = [([3], 1, False), ([3], 1, True), ([2], 2, False), ([3, 3, 1], 2, True)]
  for ci, (kernel, stride, nempty) in enumerate(dcases):
    C = 12
    m = ocnn.nn.OctreeDWConv(C, kernel, stride, nempty)
    with torch.no_grad():
      m.weights.copy_(torch.randn(m.weights.shape, generator=g) * 0.3)
    n_in = int(octree.nnum_nempty[4] if nempty else octree.nnum[4])
    x = torch.randn(n_in, C, generator=g, requires_grad=True)
    y = m(x, octree, 4)
    gy = torch.randn(y.shape, generator=g)
    y.backward(gy)
    tag = 'd%02d' % ci
    out[tag + '_meta'] = np.array([stride, int(nempty), C] + m.kernel_size, dtype=np.int64)
    out[tag + '_w'] = m.weights.detach().numpy()
    out[tag + '_x'], out[tag + '_y'] = x.detach().numpy(), y.detach().numpy()
    out[tag + '_gy'], out[tag + '_gx'] = gy.numpy(), x.grad.numpy()
    out[tag + '_gw'] = m.weights.grad.numpy()
  out['n_dw_cases'] = len(dcases)

  # ---- pooling / upsampling / pad
  for nempty in (False, True):
    t = 'p%d' % int(nempty)
    n_in = int(octree.nnum_nempty[5] if nempty else octree.nnum[5])
    x = torch.randn(n_in, 7, generator=g, requires_grad=True)
    y, ind = ocnn.nn.octree_max_pool(x, octree, 5, nempty, return_indices=True)
    gy = torch.randn(y.shape, generator=g)
    y.backward(gy)
    out[t + '_x'], out[t + '_y'], out[t + '_ind'] = x.detach().numpy(), y.detach().numpy(), ind.numpy().astype(np.int8)
    out[t + '_gy'], out[t + '_gx'] = gy.numpy(), x.grad.numpy()
    t = 'u%d' % int(nempty)
    n_in = int(octree.nnum_nempty[4] if nempty else octree.nnum[4])
    x = torch.randn(n_in, 5, generator=g, requires_grad=True)
    y = ocnn.nn.octree_interp.octree_nearest_upsample(x, octree, 4, nempty)
    gy = torch.randn(y.shape, generator=g)
    y.backward(gy)
    out[t + '_x'], out[t + '_y'] = x.detach().numpy(), y.detach().numpy()
    out[t + '_gy'], out[t + '_gx'] = gy.numpy(), x.grad.numpy()
  x = torch.randn(int(octree.nnum_nempty[5]), 3, generator=g)
  out['pad_x'] = x.numpy()
  out['pad_y'] = ocnn.nn.octree_pad(x, octree, 5, 1.5).numpy()
  out['depad_y'] = ocnn.nn.octree_depad(torch.from_numpy(out['pad_y']), octree, 5).numpy()

  # ---- norms
  for ni, (C, group, nempty) in enumerate([(8, 2, False), (12, 12, True), (16, 4, True)]):
    t = 'g%d' % ni
    m = ocnn.nn.OctreeGroupNorm(C, group, nempty, min_group_channels=1)
    with torch.no_grad():
      m.weights.copy_(torch.rand(1, C, generator=g) + 0.5)
      m.bias.copy_(torch.randn(1, C, generator=g))
    n_in = int(octree.nnum_nempty[5] if nempty else octree.nnum[5])
    x = (torch.randn(n_in, C, generator=g) * 2 + 0.3).requires_grad_()
    y = m(x, octree, 5)
    gy = torch.randn(y.shape, generator=g)
    y.backward(gy)
    out[t + '_meta'] = np.array([C, m.group, int(nempty)], dtype=np.int64)
    out[t + '_w'], out[t + '_b'] = m.weights.detach().numpy(), m.bias.detach().numpy()
    out[t + '_x'], out[t + '_y'] = x.detach().numpy(), y.detach().numpy()
    out[t + '_gy'], out[t + '_gx'] = gy.numpy(), x.grad.numpy()
    out[t + '_gw'], out[t + '_gb'] = m.weights.grad.numpy(), m.bias.grad.numpy()
  bn = ocnn.nn.OctreeBatchNorm(9)
  with torch.no_grad():
    bn.weight.copy_(torch.rand(9, generator=g) + 0.5)
    bn.bias.copy_(torch.randn(9, generator=g))
  x = (torch.randn(int(octree.nnum[5]), 9, generator=g) * 1.7 - 0.4).requires_grad_()
  y = bn(x)
  gy = torch.randn(y.shape, generator=g)
  y.backward(gy)
  out['bn_w'], out['bn_b'] = bn.weight.detach().numpy(), bn.bias.detach().numpy()
  out['bn_x'], out['bn_y'], out['bn_gy'], out['bn_gx'] = (x.detach().numpy(), y.detach().numpy(),
                                                          gy.numpy(), x.grad.numpy())
  out['bn_gw'], out['bn_gb'] = bn.weight.grad.numpy(), bn.bias.grad.numpy()
  out['bn_rm'], out['bn_rv'] = bn.running_mean.numpy(), bn.running_var.numpy()
  bn.eval()
  out['bn_y_eval'] = bn(x.detach()).detach().numpy()

  # ---- shuffled keys: round trip and float edge cases (test_shuffled_key.py:17-29)
  gi = torch.Generator().manual_seed(9)
  xyz = torch.randint(0, 2 ** 16, (3, 2000), generator=gi)
  bb = torch.randint(0, 2 ** 15, (2000,), generator=gi)
  out['k16_xyzb'] = torch.cat([xyz, bb[None]], 0).numpy()
  out['k16_key'] = ocnn.octree.xyz2key(xyz[0], xyz[1], xyz[2], bb, depth=16).numpy()
  fl = torch.tensor([1.9, -0.5, -1.0, 0.0, 7.99, 8.0, 255.5, 256.0, 1023.7, 1024.0, -3.2, 65535.9])
  for d in (3, 8, 9, 10, 16):
    out['kf_key_%d' % d] = ocnn.octree.xyz2key(fl, fl.flip(0), fl.roll(3), None, depth=d).numpy()
    kk = torch.from_numpy(out['k16_key'])
    x, y, z, b = ocnn.octree.key2xyz(kk, d)
    out['k2x_%d' % d] = torch.stack([x, y, z, b]).numpy()
  out['kf_in'] = fl.numpy()

  np.savez_compressed(os.path.join(OUT, 'synthetic.npz'), **out)


if __name__ == '__main__':
  hand3()
  ref_fixtures()
  interp()
  extras()
  synthetic()
  for f in sorted(os.listdir(OUT)):
    if f.endswith('.npz'):
      print(f, os.path.getsize(os.path.join(OUT, f)) // 1024, 'KiB')

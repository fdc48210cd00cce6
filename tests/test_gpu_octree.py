"""GPU parity of keys, octree construction and neighbour tables: bit-exact
against the reference's golden vectors and against the numpy oracle.  All calls
go through the C-ABI library (via the package's ctypes binding)."""
import numpy as np
import pytest
import torch

import ocnn_pytorch_b200 as b200
from oracle import octree_oracle as orc
from helpers import split_by
from gpu_utils import dev, to_np, build, synthetic_octree

pytestmark = pytest.mark.gpu


def test_keys(golden):
  syn = golden['synthetic']
  d = dev()
  x, y, z, b = (torch.from_numpy(v).to(d) for v in syn['k16_xyzb'])
  key = b200.octree.xyz2key(x, y, z, b, 16)
  assert np.array_equal(to_np(key), syn['k16_key'])
  for dt in (torch.int32, torch.float32, torch.float64):
    assert torch.equal(b200.octree.xyz2key(x.to(dt), y.to(dt), z.to(dt), b.to(dt), 16), key)
  dec = torch.stack(b200.octree.key2xyz(key, 16))
  assert np.array_equal(to_np(dec), syn['k16_xyzb'])
  fl = torch.from_numpy(syn['kf_in']).to(d)
  for depth in (3, 8, 9, 10, 16):
    k = b200.octree.xyz2key(fl, fl.flip(0), fl.roll(3), None, depth)
    assert np.array_equal(to_np(k), syn['kf_key_%d' % depth]), depth
    dec = torch.stack(b200.octree.key2xyz(torch.from_numpy(syn['k16_key']).to(d), depth))
    assert np.array_equal(to_np(dec), syn['k2x_%d' % depth]), depth
  # scalar batch index and empty input
  assert torch.equal(b200.octree.xyz2key(x, y, z, 3, 16), (3 << 48) | b200.octree.xyz2key(x, y, z, None, 16))
  e = torch.empty(0, dtype=torch.int64, device=d)
  assert b200.octree.xyz2key(e, e, e, None, 5).numel() == 0


def _check(octree, data, prefix=''):
  g = lambda k: data[prefix + k]
  assert np.array_equal(octree.nnum.numpy(), g('nnum'))
  assert np.array_equal(octree.nnum_nempty.numpy(), g('nnum_nempty'))
  assert np.array_equal(to_np(torch.cat(octree.keys)), g('key'))
  assert np.array_equal(to_np(torch.cat(octree.children)), g('child'))


def test_build_hand_case(golden):
  h = golden['hand3']
  octree, idx = build(h['points'], h['normals'], h['features'], depth=5, full_depth=1)
  _check(octree, h)
  assert np.array_equal(to_np(idx), h['idx'])
  assert np.array_equal(to_np(octree.normals[5]), h['out_normals'])
  assert np.array_equal(to_np(octree.features[5]), h['out_features'])
  assert np.allclose(to_np(octree.points[5]), h['out_points'])
  assert np.array_equal(to_np(torch.cat(octree.neighs[1:])), h['neigh'])
  idxs = [[0], [0, 6], [0, 8], [0, 8], [0, 8], [0, 8, 14]]   # test/test_octree.py:71-76
  for d in range(6):
    assert octree.nempty_index(d).tolist() == idxs[d]
    assert torch.equal(octree.nempty_mask(d), octree.children[d] >= 0)


@pytest.mark.parametrize('i', [1, 2, 3, 4, 5])
def test_build_reference_fixtures(golden, i):
  d = golden['octrees']
  p = '%d_' % i
  octree, idx = build(d[p + 'points'], d[p + 'normals'], depth=int(d[p + 'depth']),
                      full_depth=int(d[p + 'full_depth']), neigh=False)
  _check(octree, d, p)
  assert np.array_equal(to_np(idx), d[p + 'idx'])
  assert np.allclose(to_np(octree.normals[octree.depth]), d[p + 'feature'], atol=1e-6)
  assert np.allclose(to_np(octree.points[octree.depth]), d[p + 'avg_points'], atol=1e-5)


def test_batched_build_merge_and_neigh_batch45(golden):
  d, b45 = golden['octrees'], golden['batch45']
  depth, fd = int(b45['depth']), int(b45['full_depth'])
  pts = np.concatenate([d['4_points'], d['5_points']])
  nrm = np.concatenate([d['4_normals'], d['5_normals']])
  bid = np.concatenate([np.zeros(len(d['4_points']), np.float32), np.ones(len(d['5_points']), np.float32)])
  octree, _ = build(pts, nrm, batch_id=bid, batch_size=2, depth=depth, full_depth=fd)
  _check(octree, b45)
  assert np.allclose(to_np(octree.normals[depth]), b45['feature'], atol=1e-6)
  assert np.array_equal(to_np(torch.cat(octree.neighs[1:])), b45['neigh'])
  # int64 batch ids give the same octree
  o2, _ = build(pts, nrm, batch_id=bid.astype(np.int64), batch_size=2, depth=depth, full_depth=fd, neigh=False)
  _check(o2, b45)
  # merge of two single builds == batched build (test/test_octree.py:115-136)
  o4, _ = build(d['4_points'], d['4_normals'], depth=depth, full_depth=fd, neigh=False)
  o5, _ = build(d['5_points'], d['5_normals'], depth=depth, full_depth=fd, neigh=False)
  merged = b200.octree.merge_octrees([o4, o5])
  merged.construct_all_neigh()
  _check(merged, b45)
  assert np.array_equal(to_np(torch.cat(merged.neighs[1:])), b45['neigh'])
  # both neighbour branches agree on a dense layer (test/test_octree.py:181-191)
  neigh_fd = octree.neighs[fd].clone()
  L = b200._lib
  out = torch.empty_like(neigh_fd)
  L.call('oc_neigh_from_parent', L.ptr(octree.neighs[fd - 1]), L.ptr(octree.children[fd - 1]),
         octree.children[fd - 1].numel(), L.ptr(out), None, L.stream(dev()))
  assert torch.equal(out, neigh_fd)
  # batch ids and offsets
  for dd in range(depth + 1):
    x, y, z, b = octree.xyzb(dd)
    assert torch.equal(b, octree.batch_id(dd))
    offs = octree.batch_offsets(dd, False)
    assert offs == [0, int((b == 0).sum()), b.numel()]
    bne = octree.batch_id(dd, nempty=True)
    assert octree.batch_offsets(dd, True) == [0, int((bne == 0).sum()), bne.numel()]


def test_synthetic_build_neigh_and_variants(golden):
  syn = golden['synthetic']
  octree, idx = synthetic_octree(syn)
  _check(octree, syn)
  depth = octree.depth
  assert np.array_equal(to_np(idx), syn['idx'])
  assert np.allclose(to_np(octree.points[depth]), syn['out_points'], atol=1e-5)
  assert np.allclose(to_np(octree.normals[depth]), syn['out_normals'], atol=1e-6)
  assert np.allclose(to_np(octree.features[depth]), syn['out_features'], atol=1e-6)
  assert np.array_equal(to_np(torch.cat(octree.neighs[1:])), syn['neigh'])
  for d in (3, depth):
    for kernel in orc.KERNEL_TAPS:
      for stride in (1, 2):
        for nempty in (False, True):
          got = octree.get_neigh(d, kernel, stride, nempty)
          assert got.dtype == torch.int64
          assert np.array_equal(to_np(got), syn['gn_%d_%s_%d_%d' % (d, kernel, stride, int(nempty))])
          # the gather-form table of the scatter direction reproduces col2octree
          table, taps = octree.conv_table(d, kernel, stride, nempty)
          tt, tapst = octree.conv_table_transposed(d, kernel, stride, nempty)
          fwd = to_np(table)[:, taps]
          inv = to_np(tt)[:, tapst]
          r, k = np.nonzero(fwd >= 0)
          assert np.array_equal(inv[fwd[r, k], k], r)
          assert (inv >= 0).sum() == (fwd >= 0).sum()
  with pytest.raises(ValueError):
    octree.get_neigh(depth, '444', 1, False)
  with pytest.raises(ValueError):
    octree.get_neigh(depth, '333', 3, False)


def test_build_matches_oracle_on_larger_clouds():
  # seeded clouds at several depths / batch sizes, including a jittered one
  for cfg, (B, n, depth, fd, jitter) in enumerate([(1, 20000, 6, 2, 0.0), (3, 15000, 7, 3, 0.005),
                                                    (4, 5000, 8, 1, 0.0), (2, 30000, 10, 3, 0.005)]):
    clouds = [b200.synthetic.mixed_cloud(100 * cfg + i, n, jitter=jitter) for i in range(B)]
    pts = np.concatenate([c[0] for c in clouds])
    nrm = np.concatenate([c[1] for c in clouds])
    bid = np.concatenate([np.full(n, i, np.float32) for i in range(B)])
    o = orc.build_octree(pts, nrm, None, bid, B, depth, fd)
    octree, idx = build(pts, nrm, None, bid if B > 1 else None, B, depth, fd)
    assert np.array_equal(octree.nnum.numpy(), o['nnum'])
    assert np.array_equal(octree.nnum_nempty.numpy(), o['nnum_nempty'])
    for d in range(depth + 1):
      assert np.array_equal(to_np(octree.keys[d]), o['keys'][d]), (cfg, d)
      assert np.array_equal(to_np(octree.children[d]), o['children'][d]), (cfg, d)
    assert np.array_equal(to_np(idx), o['idx'])
    assert np.allclose(to_np(octree.points[depth]), o['points'], atol=1e-4)
    assert np.allclose(to_np(octree.normals[depth]), o['normals'], atol=1e-5)
    neighs = orc.construct_all_neigh(o['children'], o['nnum'], depth, fd, B)
    for d in range(1, depth + 1):
      assert np.array_equal(to_np(octree.neighs[d]), neighs[d]), (cfg, d)


def test_grow_split_reproduce_octree(golden):
  # octree_grow_full / octree_split / octree_grow rebuild the same structure
  # (test/test_octree.py:157-179)
  syn = golden['synthetic']
  ref, _ = synthetic_octree(syn)
  depth, fd, B = ref.depth, ref.full_depth, ref.batch_size
  o = b200.octree.init_octree(depth, fd, B, dev())
  for d in range(fd, depth + 1):
    split = (ref.children[d] >= 0).long()
    o.octree_split(split, d)
    if d < depth:
      o.octree_grow(d + 1)
  for d in range(depth + 1):
    assert torch.equal(o.keys[d], ref.keys[d]), d
    assert torch.equal(o.children[d], ref.children[d]), d
    if d >= 1:
      assert torch.equal(o.neighs[d], ref.neighs[d]), d


def test_build_sizes_property_full_scale():
  # depth-8 batch of 4 x 100k points: structural invariants that do not need the oracle
  B, n, depth, fd = 4, 100000, 8, 3
  clouds = [b200.synthetic.mixed_cloud(2000 + i, n) for i in range(B)]
  pts = np.concatenate([c[0] for c in clouds])
  nrm = np.concatenate([c[1] for c in clouds])
  bid = np.concatenate([np.full(n, i, np.float32) for i in range(B)])
  octree, idx = build(pts, nrm, None, bid, B, depth, fd)
  for d in range(1, depth + 1):
    keys, ch, ng = octree.keys[d], octree.children[d], octree.neighs[d]
    assert torch.all(keys[1:] > keys[:-1])                       # sorted, unique
    nne = int(octree.nnum_nempty[d])
    got = ch[ch >= 0]
    assert torch.equal(got.long(), torch.arange(nne, device=ch.device))   # ranks in order
    assert torch.equal(ng[:, 13], torch.arange(ng.shape[0], device=ng.device))
    r = torch.arange(ng.shape[0], device=ng.device)
    for k in (0, 5, 22):                                          # mirror symmetry
      m = ng[:, k]
      v = m >= 0
      assert torch.equal(ng[m[v], 26 - k], r[v])
  assert int(idx.max()) + 1 == int(octree.nnum_nempty[depth])

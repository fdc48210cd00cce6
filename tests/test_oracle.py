"""Pins the numpy oracle against vectors produced by the reference itself
(tests/golden/*.npz, see tests/golden/make_golden.py).  CPU only."""
import numpy as np
import pytest

from oracle import octree_oracle as orc
from helpers import split_by, assert_close, conv_case, octree_from_golden

F32 = 2e-5  # oracle and reference are both fp32 on CPU; only summation order differs


def test_keys_roundtrip_and_edges(golden):
  syn = golden['synthetic']
  x, y, z, b = syn['k16_xyzb']
  key = orc.xyz2key(x, y, z, b, 16)
  assert np.array_equal(key, syn['k16_key'])
  fl = syn['kf_in']
  for d in (3, 8, 9, 10, 16):
    k = orc.xyz2key(fl, fl[::-1], np.roll(fl, 3), None, d)
    assert np.array_equal(k, syn['kf_key_%d' % d]), d
    dec = np.stack(orc.key2xyz(syn['k16_key'], d))
    assert np.array_equal(dec, syn['k2x_%d' % d]), d
  xx, yy, zz, bb = orc.key2xyz(key, 16)
  assert np.array_equal(np.stack([xx, yy, zz, bb]), syn['k16_xyzb'])


def _check_build(o, data, prefix=''):
  g = lambda k: data[prefix + k]
  assert np.array_equal(o['nnum'], g('nnum'))
  assert np.array_equal(o['nnum_nempty'], g('nnum_nempty'))
  assert np.array_equal(np.concatenate(o['keys']), g('key'))
  assert np.array_equal(np.concatenate(o['children']), g('child'))


def test_build_hand_case(golden):
  h = golden['hand3']
  o = orc.build_octree(h['points'], h['normals'], h['features'], depth=5, full_depth=1)
  _check_build(o, h)
  assert np.array_equal(o['idx'], h['idx'])
  assert np.array_equal(o['normals'], h['out_normals'])
  assert np.array_equal(o['features'], h['out_features'])
  assert np.allclose(o['points'], h['out_points'])
  neighs = orc.construct_all_neigh(o['children'], o['nnum'], 5, 1, 1)
  assert np.array_equal(np.concatenate(neighs[1:]), h['neigh'])


@pytest.mark.parametrize('i', [1, 2, 3, 4, 5])
def test_build_reference_fixtures(golden, i):
  d = golden['octrees']
  p = '%d_' % i
  o = orc.build_octree(d[p + 'points'], d[p + 'normals'], depth=int(d[p + 'depth']),
                       full_depth=int(d[p + 'full_depth']))
  _check_build(o, d, p)
  assert np.array_equal(o['idx'], d[p + 'idx'])
  assert np.allclose(o['normals'], d[p + 'feature'], atol=1e-6)
  assert np.allclose(o['points'], d[p + 'avg_points'], atol=1e-5)


def test_batched_build_and_neigh_batch45(golden):
  d, b45 = golden['octrees'], golden['batch45']
  pts = np.concatenate([d['4_points'], d['5_points']])
  nrm = np.concatenate([d['4_normals'], d['5_normals']])
  bid = np.concatenate([np.zeros(len(d['4_points']), np.float32), np.ones(len(d['5_points']), np.float32)])
  depth, fd = int(b45['depth']), int(b45['full_depth'])
  o = orc.build_octree(pts, nrm, batch_id=bid, batch_size=2, depth=depth, full_depth=fd)
  _check_build(o, b45)
  assert np.allclose(o['normals'], b45['feature'], atol=1e-6)
  neighs = orc.construct_all_neigh(o['children'], o['nnum'], depth, fd, 2)
  assert np.array_equal(np.concatenate(neighs[1:]), b45['neigh'])
  # both construct_neigh branches agree at full_depth (test_octree.py:181-191)
  if fd >= 2:
    via_parent = orc.construct_neigh_from_parent(neighs[fd - 1], o['children'][fd - 1])
    assert np.array_equal(via_parent, neighs[fd])


def test_synthetic_build_and_variants(golden):
  syn = golden['synthetic']
  depth, fd, B = int(syn['depth']), int(syn['full_depth']), int(syn['batch_size'])
  o = orc.build_octree(syn['points'], syn['normals'], syn['features'], syn['batch_id'], B, depth, fd)
  _check_build(o, syn)
  assert np.array_equal(o['idx'], syn['idx'])
  assert np.allclose(o['points'], syn['out_points'], atol=1e-5)
  assert np.allclose(o['normals'], syn['out_normals'], atol=1e-6)
  assert np.allclose(o['features'], syn['out_features'], atol=1e-6)
  neighs = orc.construct_all_neigh(o['children'], o['nnum'], depth, fd, B)
  assert np.array_equal(np.concatenate(neighs[1:]), syn['neigh'])
  for d in (3, depth):
    for kernel in orc.KERNEL_TAPS:
      for stride in (1, 2):
        for nempty in (False, True):
          got = orc.get_neigh(neighs[d], o['children'][d], kernel, stride, nempty)
          assert np.array_equal(got, syn['gn_%d_%s_%d_%d' % (d, kernel, stride, int(nempty))])


def _conv_oracle(c, children, neighs):
  r''' Runs the oracle the way the reference modules compose the pieces
  (OctreeConv.forward / OctreeDeconv.forward, ocnn/nn/octree_conv.py:401-466). '''
  d, k, s, ne = c['depth'], c['kernel'], c['stride'], c['nempty']
  x, w, gy = c['x'], c['w'], c['gy']
  if c['op'] == 'conv':
    neigh = orc.get_neigh(neighs[d], children[d], k, s, ne)
    y = orc.conv_forward(x, w, neigh)
    if c['use_bias']:
      y = y + c['b']
    g = gy
    if s == 2 and not ne:
      y = orc.octree_pad(y, children[d - 1])
      g = orc.octree_depad(gy, children[d - 1])
    gx = orc.conv_backward(g, w, neigh, x.shape[0])
    gw = orc.conv_weight_grad(x, g, neigh)
    gb = g.sum(0)
  else:
    nd = d + 1 if s == 2 else d
    neigh = orc.get_neigh(neighs[nd], children[nd], k, s, ne)
    xin = orc.octree_depad(x, children[d]) if (s == 2 and not ne) else x
    out_h = int((children[nd] >= 0).sum()) if ne else children[nd].size
    y = orc.deconv_forward(xin, w, neigh, out_h)
    if c['use_bias']:
      y = y + c['b']
    gxin = orc.deconv_backward(gy, w, neigh)
    gw = orc.deconv_weight_grad(xin, gy, neigh)
    gx = orc.octree_pad(gxin, children[d]) if (s == 2 and not ne) else gxin
    gb = gy.sum(0)
  return y, gx, gw, gb


def test_conv_deconv_all_cases(golden):
  syn = golden['synthetic']
  _, children, neighs = octree_from_golden(syn)
  for ci in range(int(syn['n_conv_cases'])):
    c = conv_case(syn, ci)
    y, gx, gw, gb = _conv_oracle(c, children, neighs)
    what = 'case %d %s k%s s%d ne%d' % (ci, c['op'], c['kernel'], c['stride'], c['nempty'])
    assert_close(y, c['y'], F32, what + ' y')
    assert_close(gx, c['gx'], F32, what + ' gx')
    assert_close(gw, c['gw'], F32, what + ' gw')
    if c['use_bias']:
      assert_close(gb, c['gb'], F32, what + ' gb')


def test_dwconv(golden):
  syn = golden['synthetic']
  _, children, neighs = octree_from_golden(syn)
  for ci in range(int(syn['n_dw_cases'])):
    t = 'd%02d' % ci
    stride, nempty, C = int(syn[t + '_meta'][0]), bool(syn[t + '_meta'][1]), int(syn[t + '_meta'][2])
    kernel = ''.join(str(int(v)) for v in syn[t + '_meta'][3:6])
    neigh = orc.get_neigh(neighs[4], children[4], kernel, stride, nempty)
    x, w, gy = syn[t + '_x'], syn[t + '_w'], syn[t + '_gy']
    y = orc.dwconv_forward(x, w, neigh)
    g = gy
    if stride == 2 and not nempty:
      y = orc.octree_pad(y, children[3])
      g = orc.octree_depad(gy, children[3])
    assert_close(y, syn[t + '_y'], F32, t + ' y')
    assert_close(orc.dwconv_backward(g, w, neigh, x.shape[0]), syn[t + '_gx'], F32, t + ' gx')
    assert_close(orc.dwconv_weight_grad(x, g, neigh), syn[t + '_gw'], F32, t + ' gw')


def test_pool_upsample_pad(golden):
  syn = golden['synthetic']
  _, children, _ = octree_from_golden(syn)
  for ne in (0, 1):
    y, ind = orc.max_pool(syn['p%d_x' % ne], children[5], children[4], bool(ne))
    assert np.array_equal(y, syn['p%d_y' % ne])
    assert np.array_equal(ind, syn['p%d_ind' % ne].astype(np.int64))
    u = orc.nearest_upsample(syn['u%d_x' % ne], children[4], children[5], bool(ne))
    assert np.array_equal(u, syn['u%d_y' % ne])
  pad = orc.octree_pad(syn['pad_x'], children[5], 1.5)
  assert np.array_equal(pad, syn['pad_y'])
  assert np.array_equal(orc.octree_depad(pad, children[5]), syn['depad_y'])


def test_norms(golden):
  syn = golden['synthetic']
  keys, children, _ = octree_from_golden(syn)
  B = int(syn['batch_size'])
  for ni in range(3):
    t = 'g%d' % ni
    C, group, nempty = (int(v) for v in syn[t + '_meta'])
    bid = keys[5] >> 48
    if nempty:
      bid = bid[children[5] >= 0]
    y = orc.group_norm(syn[t + '_x'], bid, B, group, syn[t + '_w'], syn[t + '_b'])
    assert np.allclose(y, syn[t + '_y'], atol=5e-6), t
  y, mean, var = orc.batch_norm_train(syn['bn_x'], syn['bn_w'], syn['bn_b'])
  assert np.allclose(y, syn['bn_y'], atol=5e-6)
  n = syn['bn_x'].shape[0]
  assert np.allclose(0.1 * mean, syn['bn_rm'], atol=1e-6)
  assert np.allclose(0.9 + 0.1 * var * n / (n - 1), syn['bn_rv'], atol=1e-6)


def test_search_and_interp_against_reference(golden):
  # key search and point interpolation of the merged octree 4+5: the reference's stored answers
  # (test/data/search_key.npz, test/data/interp.npz) and its gradients on seeded points
  d, b45, it = golden['octrees'], golden['batch45'], golden['interp']
  depth = 5
  nnum = b45['nnum']
  off = int(nnum[:depth].sum())
  keys = b45['key'][off:off + int(nnum[depth])]
  child = b45['child'][off:off + int(nnum[depth])]
  keys_ne = keys[child >= 0]
  xyzb = it['sk_xyzb'].astype(np.int64)
  q = orc.xyz2key(xyzb[:, 0], xyzb[:, 1], xyzb[:, 2], xyzb[:, 3], depth)
  assert np.array_equal(orc.search_key(keys, q), it['sk_idx'])
  assert np.array_equal(orc.search_key(keys_ne, q), it['sk_idx_ne'])
  data, pts = it['it_data'], it['it_pts']
  data_ne = data[child >= 0]
  assert np.allclose(orc.linear_pts(data, keys, depth, pts), it['it_linear'], atol=1e-6)
  assert np.allclose(orc.linear_pts(data_ne, keys_ne, depth, pts), it['it_linear_ne'], atol=1e-6)
  assert np.allclose(orc.nearest_pts(data, keys, depth, pts)[0], it['it_near'], atol=1e-6)
  assert np.allclose(orc.nearest_pts(data_ne, keys_ne, depth, pts)[0], it['it_near_ne'], atol=1e-6)
  gp = it['g_pts']
  for tag, kk in (('', keys), ('_ne', keys_ne)):
    dd, gy = it['g_data' + tag], it['g_gy' + tag]
    for bc in (0, 1):
      y, idx = orc.nearest_pts(dd, kk, depth, gp, bool(bc))
      assert np.allclose(y, it['g_near%s_bc%d' % (tag, bc)], atol=1e-6)
      assert np.allclose(orc.nearest_pts_backward(gy, idx, dd.shape[0]), it['g_near%s_bc%d_grad' % (tag, bc)], atol=1e-5)
      assert np.allclose(orc.linear_pts(dd, kk, depth, gp, bool(bc)), it['g_linear%s_bc%d' % (tag, bc)], atol=1e-5)
      assert np.allclose(orc.linear_pts_backward(gy, kk, depth, gp, dd.shape[0], bool(bc)),
                         it['g_linear%s_bc%d_grad' % (tag, bc)], atol=1e-5)


def test_pool_align_voxel_against_reference(golden):
  # octree_avg_pool / octree_global_pool / octree_align / octree2voxel on the merged octree 4+5
  b45, ex = golden['batch45'], golden['extras']
  depth, fd, B = int(b45['depth']), int(b45['full_depth']), 2
  nnum = [int(v) for v in b45['nnum']]
  offs = np.concatenate([[0], np.cumsum(nnum)])
  keys = [b45['key'][offs[d]:offs[d + 1]] for d in range(depth + 1)]
  child = [b45['child'][offs[d]:offs[d + 1]] for d in range(depth + 1)]
  noffs = np.concatenate([[0], np.cumsum(nnum[1:])])
  neigh = [None] + [b45['neigh'][noffs[d - 1]:noffs[d]] for d in range(1, depth + 1)]
  d = 5
  for ne in (False, True):
    tag = '_ne' if ne else ''
    x = ex['x' + tag]
    for kernel, stride in (('222', 2), ('333', 2), ('333', 1)):
      ng = orc.get_neigh(neigh[d], child[d], kernel, stride, ne)
      key = 'avg_%s_%d%s' % (kernel, stride, tag)
      y, _ = orc.avg_pool(x, ng)
      assert np.allclose(y, ex[key], atol=1e-6), key
      assert np.allclose(orc.avg_pool_backward(ex[key + '_gy'], ng, x.shape[0]), ex[key + '_gx'], atol=1e-6), key
    kk = keys[d][child[d] >= 0] if ne else keys[d]
    bid = (kk >> 48).astype(np.int64)
    y, cnt = orc.global_pool(x, bid, B)
    assert np.allclose(y, ex['glob' + tag], atol=1e-6)
    assert np.allclose(orc.global_pool_backward(ex['glob%s_gy' % tag], bid, cnt), ex['glob%s_gx' % tag], atol=1e-7)
    # the query octree holds the same two shapes in the other order: swap the batch bit of the keys
    q = np.sort(kk ^ (np.int64(1) << 48))
    y, idx = orc.align(x, kk, q)
    assert np.allclose(y, ex['align' + tag], atol=0)
    assert np.allclose(orc.nearest_pts_backward(ex['align%s_gy' % tag], idx, x.shape[0]), ex['align%s_gx' % tag], atol=1e-6)
    d4 = 4
    k4 = keys[d4][child[d4] >= 0] if ne else keys[d4]
    xx, yy, zz, bb = orc.key2xyz(k4, d4)
    v = orc.octree2voxel(ex['vox_x' + tag], xx, yy, zz, bb, d4, B)
    assert np.array_equal(v, ex['vox' + tag])
    assert np.array_equal(ex['vox%s_gy' % tag][bb, xx, yy, zz], ex['vox%s_gx' % tag])

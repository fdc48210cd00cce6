"""GPU parity of the octree operators against the reference's golden outputs and
the numpy oracle.  Tolerances (relative L2 and max-norm, both must hold):
fp32 1e-4; fp16 / bf16 1e-2 against an fp32 computation on the same rounded
inputs.  Integer outputs (pool indices) and pure copies must be equal."""
import os

import numpy as np
import pytest
import torch

import ocnn_pytorch_b200 as b200
from oracle import octree_oracle as orc
from helpers import assert_close, conv_case, octree_from_golden, tap_sort_key
from gpu_utils import dev, to_np, build, synthetic_octree

pytestmark = pytest.mark.gpu

TOL32 = 1e-4
TOL16 = 1e-2


def T(a, dtype=torch.float32, grad=False):
  t = torch.from_numpy(np.ascontiguousarray(a)).to(dev()).to(dtype)
  return t.requires_grad_() if grad else t


@pytest.fixture(scope='module')
def syn_octree(golden):
  octree, _ = synthetic_octree(golden['synthetic'])
  return octree


def _make(c):
  cls = b200.nn.OctreeConv if c['op'] == 'conv' else b200.nn.OctreeDeconv
  m = cls(c['cin'], c['cout'], c['kernel_size'], c['stride'], c['nempty'], use_bias=c['use_bias']).to(dev())
  with torch.no_grad():
    m.weights.copy_(T(c['w']))
    if c['use_bias']:
      m.bias.copy_(T(c['b']))
  return m


def test_conv_deconv_golden_fp32(golden, syn_octree):
  syn = golden['synthetic']
  for ci in range(int(syn['n_conv_cases'])):
    c = conv_case(syn, ci)
    m = _make(c)
    x = T(c['x'], grad=True)
    y = m(x, syn_octree, c['depth'])
    y.backward(T(c['gy']))
    what = 'case %d %s k%s s%d ne%d' % (ci, c['op'], c['kernel'], c['stride'], c['nempty'])
    assert_close(to_np(y), c['y'], TOL32, what + ' y')
    assert_close(to_np(x.grad), c['gx'], TOL32, what + ' gx')
    assert_close(to_np(m.weights.grad), c['gw'], TOL32, what + ' gw')
    if c['use_bias']:
      assert_close(to_np(m.bias.grad), c['gb'], TOL32, what + ' gb')


@pytest.mark.parametrize('dtype', [torch.float16, torch.bfloat16])
def test_conv_deconv_golden_half(golden, syn_octree, dtype):
  # inputs rounded to the half type; expectation = oracle in fp32 on the rounded values
  syn = golden['synthetic']
  keys, children, neighs = octree_from_golden(syn)
  from test_oracle import _conv_oracle
  for ci in range(int(syn['n_conv_cases'])):
    c = conv_case(syn, ci)
    rnd = lambda a: to_np(T(a, dtype))
    c2 = dict(c)
    for k in ('x', 'w', 'gy') + (('b',) if c['use_bias'] else ()):
      c2[k] = rnd(c[k])
    ey, egx, egw, egb = _conv_oracle(c2, children, neighs)
    m = _make(c).to(dtype)
    x = T(c['x'], dtype, grad=True)
    y = m(x, syn_octree, c['depth'])
    assert y.dtype == dtype
    y.backward(T(c['gy'], dtype))
    what = '%s case %d %s k%s s%d ne%d' % (dtype, ci, c['op'], c['kernel'], c['stride'], c['nempty'])
    assert_close(to_np(y), ey, TOL16, what + ' y')
    assert_close(to_np(x.grad), egx, TOL16, what + ' gx')
    assert_close(to_np(m.weights.grad), egw, TOL16, what + ' gw')
    if c['use_bias']:
      assert_close(to_np(m.bias.grad), egb, TOL16, what + ' gb')


def _oracle_conv333(octree_np, x, w, gy, nempty, d):
  neigh = orc.get_neigh(octree_np['neighs'][d], octree_np['children'][d], '333', 1, nempty)
  y = orc.conv_forward(x, w, neigh)
  return y, orc.conv_backward(gy, w, neigh, x.shape[0]), orc.conv_weight_grad(x, gy, neigh)


@pytest.fixture(scope='module')
def mid_octree():
  # 2 octrees, depth 6, 20k points each: the reference's CPU-runnable configuration
  B, n, depth, fd = 2, 20000, 6, 2
  clouds = [b200.synthetic.spheres_cloud(1000 + i, n) for i in range(B)]
  pts = np.concatenate([c[0] for c in clouds])
  nrm = np.concatenate([c[1] for c in clouds])
  bid = np.concatenate([np.full(n, i, np.float32) for i in range(B)])
  octree, _ = build(pts, nrm, None, bid, B, depth, fd)
  o = orc.build_octree(pts, nrm, None, bid, B, depth, fd)
  o['neighs'] = orc.construct_all_neigh(o['children'], o['nnum'], depth, fd, B)
  return octree, o


@pytest.mark.parametrize('cin,cout', [(32, 32), (1, 3), (4, 32), (30, 69), (64, 64), (96, 128),
                                      (133, 16), (256, 64), (16, 272)])
@pytest.mark.parametrize('nempty', [False, True])
def test_conv333_vs_oracle_fp32(mid_octree, cin, cout, nempty):
  octree, o = mid_octree
  d = 5 if cin * cout > 64 * 64 else 6
  rng = np.random.default_rng(cin * 1000 + cout)
  n = int(o['nnum_nempty'][d] if nempty else o['nnum'][d])
  x = rng.standard_normal((n, cin)).astype(np.float32)
  w = (rng.standard_normal((27, cin, cout)) / np.sqrt(27 * cin)).astype(np.float32)
  gy = rng.standard_normal((n, cout)).astype(np.float32)
  ey, egx, egw = _oracle_conv333(o, x, w, gy, nempty, d)
  m = b200.nn.OctreeConv(cin, cout, [3], 1, nempty).to(dev())
  with torch.no_grad():
    m.weights.copy_(T(w))
  xt = T(x, grad=True)
  y = m(xt, octree, d)
  y.backward(T(gy))
  assert_close(to_np(y), ey, TOL32, 'y')
  assert_close(to_np(xt.grad), egx, TOL32, 'gx')
  assert_close(to_np(m.weights.grad), egw, TOL32, 'gw')


@pytest.mark.parametrize('dtype', [torch.float16, torch.bfloat16])
@pytest.mark.parametrize('cin,cout', [(32, 32), (64, 64), (16, 48), (96, 96), (128, 128), (64, 128),
                                      (128, 64), (256, 256), (384, 256), (192, 128), (32, 272),
                                      (4, 32), (69, 133)])
@pytest.mark.parametrize('nempty', [False, True])
def test_conv333_vs_oracle_half(mid_octree, cin, cout, nempty, dtype):
  octree, o = mid_octree
  d = 5 if cin * cout > 64 * 64 else 6
  rng = np.random.default_rng(cin * 1000 + cout + 7)
  n = int(o['nnum_nempty'][d] if nempty else o['nnum'][d])
  rnd = lambda a: to_np(T(a, dtype))
  x = rnd(rng.standard_normal((n, cin)).astype(np.float32))
  w = rnd((rng.standard_normal((27, cin, cout)) / np.sqrt(27 * cin)).astype(np.float32))
  gy = rnd(rng.standard_normal((n, cout)).astype(np.float32))
  ey, egx, egw = _oracle_conv333(o, x, w, gy, nempty, d)
  m = b200.nn.OctreeConv(cin, cout, [3], 1, nempty).to(dev()).to(dtype)
  with torch.no_grad():
    m.weights.copy_(T(w, dtype))
  xt = T(x, dtype, grad=True)
  y = m(xt, octree, d)
  y.backward(T(gy, dtype))
  assert_close(to_np(y), ey, TOL16, 'y')
  assert_close(to_np(xt.grad), egx, TOL16, 'gx')
  assert_close(to_np(m.weights.grad), egw, TOL16, 'gw')


def test_tile_table_layout_and_equivalence(mid_octree):
  # The tile table is the neighbour table regrouped in blocks of 128 rows; a convolution
  # given the tile table returns bit-for-bit what it returns given the plain table.
  octree, o = mid_octree
  for d, kernel, stride, nempty, transposed in [(6, '333', 1, False, False), (6, '333', 1, True, True),
                                                (5, '313', 1, False, False), (6, '222', 2, False, False),
                                                (6, '333', 2, True, True), (3, '333', 1, False, False)]:
    table, taps = (octree.conv_table_transposed if transposed else octree.conv_table)(d, kernel, stride, nempty)
    tiles = octree.conv_tiles(d, kernel, stride, nempty, transposed)
    assert octree.conv_tiles(d, kernel, stride, nempty, transposed) is tiles      # cached
    K, n_out = len(taps), table.shape[0]
    # the octree's tile tables come with their rows sorted by the mask of valid taps
    assert isinstance(tiles, b200.nn.TileTable)
    raw_t = tiles.tiles
    order = to_np(tiles.perm).astype(np.int64)
    assert np.array_equal(np.sort(order), np.arange(n_out))
    row_key = tap_sort_key(to_np(table)[:, taps] >= 0)           # the mask, rare / ubiquitous taps in the high bits
    assert (np.diff(row_key[order]) >= 0).all()                  # never decreases along the table
    assert np.array_equal(order, np.argsort(row_key, kind='stable'))    # ties keep the table's order
    if transposed and stride == 2:
      cidx = to_np(octree.key(d, nempty) & 7)[order]              # which groups the rows by child index
      assert len(np.unique(cidx[:-1] != cidx[1:], return_counts=True)[1]) <= 2 and (cidx[:-1] != cidx[1:]).sum() < 64
    # a table built in the natural order gives the same results
    plain_tiles = b200.nn.tile_table(table, taps)
    assert plain_tiles.dtype == torch.uint8
    nt = (n_out + 127) // 128
    nt = (nt + 1) // 2 * 2                  # padded to an even number of blocks
    blk = 16 + K * 512
    assert raw_t.dtype == torch.uint8 and raw_t.numel() == nt * blk
    raw = to_np(raw_t).reshape(nt, blk)
    hdr = raw[:, :16].copy().view(np.uint32)
    rows = raw[:, 16:].copy().view(np.int32).reshape(nt, K, 128)
    want = np.full((nt * 128, K), -1, np.int64)
    want[:n_out] = to_np(table)[:, taps][order]
    want = np.where(want < 0, -1, want).reshape(nt, 128, K).transpose(0, 2, 1)
    assert np.array_equal(rows, want)
    mask = ((want >= 0).any(axis=2) * (1 << np.arange(K))[None, :]).sum(axis=1)
    assert np.array_equal(hdr[:, 0], mask.astype(np.uint32)) and not hdr[:, 1:].any()
    n_in = int(to_np(table).max()) + 1
    for dtype, cin, cout in [(torch.float16, 64, 64), (torch.bfloat16, 32, 80), (torch.float16, 144, 16)]:
      assert b200.nn.tiled_supported(K, cin, cout, dtype)
      g = torch.Generator(device=dev()).manual_seed(d * 100 + cin)
      x = torch.randn(n_in, cin, device=dev(), generator=g).to(dtype)
      w = (torch.randn(K, cin, cout, device=dev(), generator=g) / (K * cin) ** 0.5).to(dtype)
      bias = torch.randn(cout, device=dev(), generator=g).to(dtype)
      y_plain = b200.nn.conv_gather(x, w, False, bias, table, taps, cin, cout)
      y_tiled = b200.nn.conv_gather(x, w, False, bias, table, taps, cin, cout, tiles=tiles)
      y_nat = b200.nn.conv_gather(x, w, False, bias, table, taps, cin, cout, tiles=plain_tiles)
      assert torch.equal(y_plain, y_tiled) and torch.equal(y_plain, y_nat)
      # weight gradient through the ordered table (grad_out rows are read through the row
      # order): the same sum in another order
      gy = torch.randn(n_out, cout, device=dev(), generator=g).to(dtype)
      gw_plain, gb_plain = b200.nn.conv_wgrad(x, gy, table, taps, cin, cout, True)
      gw_tiled, gb_tiled = b200.nn.conv_wgrad(x, gy, table, taps, cin, cout, True, tiles=tiles)
      gw_nat, _ = b200.nn.conv_wgrad(x, gy, table, taps, cin, cout, False, tiles=plain_tiles)
      assert torch.equal(gw_plain, gw_nat)
      assert_close(to_np(gw_tiled), to_np(gw_plain), 1e-4, 'gw through the row order')
      assert_close(to_np(gb_tiled), to_np(gb_plain), 1e-5, 'gb')
  b200._lib.status_check(dev())
  # an index past the feature rows is dropped while the tile table is built, and reported
  table, taps = octree.conv_table(6, '333', 1, False)
  n_in = int(octree.nnum[6])
  good = b200.nn.tile_table(table, taps, n_in)
  b200._lib.status_check(dev())
  bad = b200.nn.tile_table(table, taps, n_in - 100)
  with pytest.raises(b200._lib.OctConvError, match='n_in'):
    b200._lib.status_check(dev())
  b200._lib.status_check(dev())                      # the flag is cleared by the failed check
  kept = to_np(bad).reshape(-1, 16 + 27 * 512)[:, 16:].copy().view(np.int32)
  full = to_np(good).reshape(-1, 16 + 27 * 512)[:, 16:].copy().view(np.int32)
  assert np.array_equal(kept, np.where(full >= n_in - 100, -1, full))
  # shapes off the tensor-core path have no tiled form: the plain table is used
  assert not b200.nn.tiled_supported(27, 30, 64, torch.float16)
  assert not b200.nn.tiled_supported(27, 64, 64, torch.float32)


@pytest.mark.parametrize('dtype,cin,cout,n_out', [(torch.float16, 64, 64, 128 * (8 * 148 + 3) + 77),
                                                   (torch.bfloat16, 32, 96, 128 * (8 * 148 + 2)),
                                                   (torch.float16, 128, 128, 128 * (8 * 148 + 1) + 5)])
def test_conv_large_random_table(dtype, cin, cout, n_out):
  # Enough rows for the kernel to take tiles of two 128-row halves (odd and even tile counts,
  # ragged last tile).  The table is random, so rows gather from anywhere; a fifth of the
  # entries and whole taps of some tiles are empty.
  g = torch.Generator(device=dev()).manual_seed(n_out + cin)
  K, n_in = 27, 40000
  table = torch.randint(0, n_in, (n_out, K), device=dev(), generator=g)
  table[torch.rand(n_out, K, device=dev(), generator=g) < 0.2] = -1
  table[1024:1024 + 256, 5] = -1                  # tap 5 empty in two tiles
  table[4096:4096 + 128, :] = -1                  # one tile without any neighbour
  table[4224:4224 + 128, 1:] = -1                 # its partner half only has tap 0
  taps = list(range(K))
  x = torch.randn(n_in, cin, device=dev(), generator=g).to(dtype)
  w = (torch.randn(K, cin, cout, device=dev(), generator=g) / (K * cin) ** 0.5).to(dtype)
  bias = torch.randn(cout, device=dev(), generator=g).to(dtype)
  gy = torch.randn(n_out, cout, device=dev(), generator=g).to(dtype)
  tiles = b200.nn.tile_table(table, taps)
  y_plain = b200.nn.conv_gather(x, w, False, bias, table, taps, cin, cout)
  y_tiled = b200.nn.conv_gather(x, w, False, bias, table, taps, cin, cout, tiles=tiles)
  b200._lib.status_check(dev())
  assert torch.equal(y_plain, y_tiled)
  # the same rows fetched by TMA (tile::gather4) instead of cp.async: identical bits
  # (taken when Cin is a multiple of 64; otherwise the variable changes nothing)
  os.environ['OC_TMA_GATHER'] = '1'
  try:
    y_tma = b200.nn.conv_gather(x, w, False, bias, table, taps, cin, cout, tiles=tiles)
    y_tma_plain = b200.nn.conv_gather(x, w, False, bias, table, taps, cin, cout)
    b200._lib.status_check(dev())
  finally:
    del os.environ['OC_TMA_GATHER']
  assert torch.equal(y_plain, y_tma) and torch.equal(y_plain, y_tma_plain)
  # against fp32 torch on a sample of rows (including the empty tile and the ragged end)
  rows = torch.cat([torch.arange(0, 300, device=dev()), torch.arange(4090, 4360, device=dev()),
                    torch.arange(n_out - 200, n_out, device=dev())])
  t = table[rows]
  xg = x.float()[t.clamp(min=0)] * (t >= 0).unsqueeze(-1)             # (R, K, cin)
  ref = torch.einsum('rkc,kcd->rd', xg, w.float()).to(dtype).float() + bias.float()
  assert_close(to_np(y_tiled[rows]), to_np(ref), TOL16, 'y')
  # weight gradient: tile table and plain table agree bit for bit, and match fp32 torch
  gw_plain, _ = b200.nn.conv_wgrad(x, gy, table, taps, cin, cout)
  gw_tiled, gb = b200.nn.conv_wgrad(x, gy, table, taps, cin, cout, True, tiles=tiles)
  b200._lib.status_check(dev())
  assert torch.equal(gw_plain, gw_tiled)
  ref_gw = torch.zeros(K, cin, cout, device=dev())
  for k in range(K):
    tk = table[:, k]
    ref_gw[k] = (x.float()[tk.clamp(min=0)] * (tk >= 0).unsqueeze(-1)).t() @ gy.float()
  assert_close(to_np(gw_tiled), to_np(ref_gw), 2e-3, 'gw')
  assert_close(to_np(gb), to_np(gy.float().sum(0)), 2e-3, 'gb')


@pytest.mark.parametrize('cin,cout', [(16, 32), (32, 16), (32, 64), (16, 16)])
def test_conv_packed_taps_all_kernel_shapes(mid_octree, cin, cout):
  # Cin = 16 / 32 share a 64-wide reduction block between 4 / 2 taps; with K = 8, 9, 27 taps the
  # last block is partly padding.  Forward, transposed weights and weight gradient against fp32 torch
  # computed from the same table, with and without the tile table.
  octree, o = mid_octree
  d = 6
  for kernel, stride, nempty in [('333', 1, False), ('222', 2, False), ('313', 1, True), ('133', 2, True),
                                 ('311', 1, False)]:
    table, taps = octree.conv_table(d, kernel, stride, nempty)
    tiles = octree.conv_tiles(d, kernel, stride, nempty)
    K, n_out = len(taps), table.shape[0]
    n_in = int(o['nnum_nempty'][d] if nempty else o['nnum'][d])
    g = torch.Generator(device=dev()).manual_seed(K * 100 + cin)
    x = torch.randn(n_in, cin, device=dev(), generator=g).half()
    w = (torch.randn(K, cin, cout, device=dev(), generator=g) / (K * cin) ** 0.5).half()
    gy = torch.randn(n_out, cout, device=dev(), generator=g).half()
    t = table[:, taps]
    xg = x.float()[t.clamp(min=0)] * (t >= 0).unsqueeze(-1)             # (n_out, K, cin)
    ref_y = torch.einsum('rkc,kcd->rd', xg, w.float())
    ref_gw = torch.einsum('rkc,rd->kcd', xg, gy.float())
    for tl in (None, tiles):
      y = b200.nn.conv_gather(x, w, False, None, table, taps, cin, cout, tiles=tl)
      yt = b200.nn.conv_gather(x, w.transpose(1, 2).contiguous(), True, None, table, taps, cin, cout, tiles=tl)
      gw, _ = b200.nn.conv_wgrad(x, gy, table, taps, cin, cout, False, tiles=tl)
      b200._lib.status_check(dev())
      assert_close(to_np(y), to_np(ref_y), TOL16, 'y %s' % kernel)
      assert torch.equal(y, yt)
      assert_close(to_np(gw), to_np(ref_gw), 2e-3, 'gw %s' % kernel)


@pytest.mark.parametrize('nempty', [False, True])
@pytest.mark.parametrize('kernel_size', [[3], [2]])
def test_strided_conv_deconv_half_matches_fp32_path(mid_octree, kernel_size, nempty):
  # Stride-2 conv and deconv on the tensor-core path (the input gradient of the conv and the forward
  # of the deconv run on the inverse table with rows grouped by child index) against the fp32 kernels,
  # which the golden tests pin to the reference.
  octree, o = mid_octree
  d = 6
  g = torch.Generator(device=dev()).manual_seed(3)
  n = int(o['nnum_nempty'][d] if nempty else o['nnum'][d])
  x32 = torch.randn(n, 32, device=dev(), generator=g)
  res = {}
  for dtype in (torch.float32, torch.float16):
    conv = b200.nn.OctreeConv(32, 64, kernel_size, 2, nempty).to(dev())
    deconv = b200.nn.OctreeDeconv(64, 32, kernel_size, 2, nempty).to(dev())
    gg = torch.Generator(device=dev()).manual_seed(4)
    with torch.no_grad():
      conv.weights.copy_(torch.randn(conv.weights.shape, device=dev(), generator=gg) * 0.05)
      deconv.weights.copy_(torch.randn(deconv.weights.shape, device=dev(), generator=gg) * 0.05)
    conv, deconv = conv.to(dtype), deconv.to(dtype)
    x = x32.detach().to(dtype).clone().requires_grad_()
    y = conv(x, octree, d)
    z = deconv(y, octree, d - 1)
    gz = torch.randn(z.shape, device=dev(), generator=gg).to(dtype)
    z.backward(gz)
    res[dtype] = [to_np(t) for t in (y, z, x.grad, conv.weights.grad, deconv.weights.grad)]
  b200._lib.status_check(dev())
  for a, b, name in zip(res[torch.float16], res[torch.float32], ('y', 'z', 'gx', 'gw_conv', 'gw_deconv')):
    assert_close(a, b, TOL16, name)


def test_conv_is_deterministic_and_linear(mid_octree):
  octree, o = mid_octree
  d, C = 6, 64
  n = int(o['nnum'][d])
  g = torch.Generator(device=dev()).manual_seed(1)
  m = b200.nn.OctreeConv(C, C).to(dev()).half()
  x1 = torch.randn(n, C, device=dev(), generator=g).half()
  x2 = torch.randn(n, C, device=dev(), generator=g).half()
  y1, y1b = m(x1, octree, d), m(x1, octree, d)
  assert torch.equal(y1, y1b)                         # no atomics anywhere: bitwise repeatable
  y2 = m(x2, octree, d)
  y12 = m((x1.float() + x2.float()).half(), octree, d)
  assert_close(to_np(y12), to_np(y1.float() + y2.float()), TOL16, 'linearity')


def test_dwconv_golden(golden, syn_octree):
  syn = golden['synthetic']
  for ci in range(int(syn['n_dw_cases'])):
    t = 'd%02d' % ci
    stride, nempty, C = int(syn[t + '_meta'][0]), bool(syn[t + '_meta'][1]), int(syn[t + '_meta'][2])
    ks = [int(v) for v in syn[t + '_meta'][3:6]]
    m = b200.nn.OctreeDWConv(C, ks, stride, nempty).to(dev())
    with torch.no_grad():
      m.weights.copy_(T(syn[t + '_w']))
    x = T(syn[t + '_x'], grad=True)
    y = m(x, syn_octree, 4)
    y.backward(T(syn[t + '_gy']))
    assert_close(to_np(y), syn[t + '_y'], TOL32, t + ' y')
    assert_close(to_np(x.grad), syn[t + '_gx'], TOL32, t + ' gx')
    assert_close(to_np(m.weights.grad), syn[t + '_gw'], TOL32, t + ' gw')


@pytest.mark.parametrize('dtype', [torch.float32, torch.bfloat16])
def test_dwconv_equals_single_channel_convs(mid_octree, dtype):
  # structure of the reference's test/test_octree_dwconv.py:18-55
  octree, o = mid_octree
  d, C = 5, 8
  n = int(o['nnum'][d])
  g = torch.Generator(device=dev()).manual_seed(3)
  x = torch.randn(n, C, device=dev(), generator=g).to(dtype)
  dw = b200.nn.OctreeDWConv(C, [3]).to(dev())
  y = dw(x, octree, d)
  for c in range(C):
    conv = b200.nn.OctreeConv(1, 1, [3]).to(dev())
    with torch.no_grad():
      conv.weights.copy_(dw.weights[:, :, c:c + 1])
    yc = conv(x[:, c:c + 1].contiguous(), octree, d)
    assert_close(to_np(y[:, c:c + 1]), to_np(yc), 1e-5 if dtype == torch.float32 else TOL16, 'channel %d' % c)


def test_pool_upsample_pad_golden(golden, syn_octree):
  syn = golden['synthetic']
  for ne in (0, 1):
    for dtype in (torch.float32, torch.float16):
      x = T(syn['p%d_x' % ne], dtype, grad=True)
      y, ind = b200.nn.octree_max_pool(x, syn_octree, 5, bool(ne), return_indices=True)
      y.backward(T(syn['p%d_gy' % ne], dtype))
      if dtype == torch.float32:
        assert np.array_equal(to_np(y), syn['p%d_y' % ne])
        assert np.array_equal(to_np(x.grad), syn['p%d_gx' % ne])
        assert np.array_equal(to_np(ind), syn['p%d_ind' % ne].astype(np.int64))
        un = b200.nn.octree_max_unpool(y.detach(), ind, syn_octree, 4, bool(ne))
        assert un.shape == x.shape
        assert torch.equal(un != 0, (x.grad != 0) | ((un != 0) & (x.grad == 0)))
      else:
        ey, eind = orc.max_pool(to_np(x), to_np(syn_octree.children[5]), to_np(syn_octree.children[4]), bool(ne))
        assert np.array_equal(to_np(y), ey)
      u = T(syn['u%d_x' % ne], dtype, grad=True)
      up = b200.nn.octree_nearest_upsample(u, syn_octree, 4, bool(ne))
      up.backward(T(syn['u%d_gy' % ne], dtype))
      if dtype == torch.float32:
        assert np.array_equal(to_np(up), syn['u%d_y' % ne])
        assert_close(to_np(u.grad), syn['u%d_gx' % ne], 1e-6, 'upsample grad')
      mod = b200.nn.OctreeUpsample('nearest', bool(ne))
      assert torch.equal(mod(u.detach(), syn_octree, 4), up.detach())
  pad = b200.nn.octree_pad(T(syn['pad_x']), syn_octree, 5, 1.5)
  assert np.array_equal(to_np(pad), syn['pad_y'])
  assert np.array_equal(to_np(b200.nn.octree_depad(pad, syn_octree, 5)), syn['depad_y'])
  # odd channel count / half type take the scalar path
  x = torch.randn(int(syn_octree.nnum_nempty[5]), 5, device=dev()).half()
  p = b200.nn.octree_pad(x, syn_octree, 5)
  assert torch.equal(b200.nn.octree_depad(p, syn_octree, 5), x)


def test_norms_golden(golden, syn_octree):
  syn = golden['synthetic']
  for ni in range(3):
    t = 'g%d' % ni
    C, group, nempty = (int(v) for v in syn[t + '_meta'])
    m = b200.nn.OctreeGroupNorm(C, group, bool(nempty), min_group_channels=1).to(dev())
    with torch.no_grad():
      m.weights.copy_(T(syn[t + '_w']))
      m.bias.copy_(T(syn[t + '_b']))
    x = T(syn[t + '_x'], grad=True)
    y = m(x, syn_octree, 5)
    y.backward(T(syn[t + '_gy']))
    assert np.allclose(to_np(y), syn[t + '_y'], atol=5e-6), t
    assert np.allclose(to_np(x.grad), syn[t + '_gx'], atol=2e-5), t
    assert np.allclose(to_np(m.weights.grad), syn[t + '_gw'], rtol=1e-4, atol=1e-3), t
    assert np.allclose(to_np(m.bias.grad), syn[t + '_gb'], rtol=1e-4, atol=1e-3), t
  bn = b200.nn.OctreeBatchNorm(9).to(dev())
  with torch.no_grad():
    bn.weight.copy_(T(syn['bn_w']))
    bn.bias.copy_(T(syn['bn_b']))
  x = T(syn['bn_x'], grad=True)
  y = bn(x)
  y.backward(T(syn['bn_gy']))
  assert np.allclose(to_np(y), syn['bn_y'], atol=5e-6)
  assert np.allclose(to_np(x.grad), syn['bn_gx'], atol=5e-6)
  assert np.allclose(to_np(bn.weight.grad), syn['bn_gw'], rtol=1e-4, atol=1e-3)
  assert np.allclose(to_np(bn.bias.grad), syn['bn_gb'], rtol=1e-4, atol=1e-3)
  assert np.allclose(to_np(bn.running_mean), syn['bn_rm'], atol=1e-6)
  assert np.allclose(to_np(bn.running_var), syn['bn_rv'], atol=1e-5)
  bn.eval()
  assert np.allclose(to_np(bn(x.detach())), syn['bn_y_eval'], atol=5e-6)


def test_conv_error_paths(syn_octree):
  m = b200.nn.OctreeConv(4, 8).to(dev())
  with pytest.raises(AssertionError):
    m(torch.zeros(3, 4, device=dev()), syn_octree, 5)               # wrong row count
  with pytest.raises(ValueError):
    b200.nn.OctreeConv(4, 8, [4]).to(dev())(torch.zeros(int(syn_octree.nnum[5]), 4, device=dev()), syn_octree, 5)
  with pytest.raises(TypeError):
    m.double()(torch.zeros(int(syn_octree.nnum[5]), 4, device=dev(), dtype=torch.float64), syn_octree, 5)


def test_tap_order_large_and_bad_row_order():
  # More rows than one wave of the helper kernels covers (grids are capped, kernels stride):
  # the order is the stable sort of the rows by their mask of valid taps (bits reordered by frequency).
  g = torch.Generator(device=dev()).manual_seed(5)
  n, K = 148 * 16 * 256 + 12345, 27
  table = torch.randint(0, 1000, (n, K), device=dev(), generator=g)
  table[torch.rand(n, K, device=dev(), generator=g) < 0.5] = -1
  table[: n // 3, 9:] = -1                        # many rows share few masks
  taps = list(range(K))
  order = to_np(b200.nn.tap_mask_order(table, taps, 0)).astype(np.int64)
  valid = to_np(table) >= 0
  assert np.array_equal(order, np.argsort(tap_sort_key(valid), kind='stable'))
  # within chunks of 2^17 rows (the default is 2^19: two chunks here)
  for lg in (17, 19):
    order_c = to_np(b200.nn.tap_mask_order(table, taps, lg)).astype(np.int64)
    assert np.array_equal(order_c, np.argsort(tap_sort_key(valid, lg), kind='stable'))
  # fewer taps than a sort pass, and a single row
  order5 = to_np(b200.nn.tap_mask_order(table[:5000], [3, 0, 7], 10)).astype(np.int64)
  assert np.array_equal(order5, np.argsort(tap_sort_key(valid[:5000][:, [3, 0, 7]], 10), kind='stable'))
  assert to_np(b200.nn.tap_mask_order(table[:1], taps)).tolist() == [0]
  # a row order that is not a permutation of the rows is reported when the tile table is built
  small = table[:1000].contiguous()
  bad = torch.arange(1000, device=dev(), dtype=torch.int32)
  bad[17] = 5000
  b200._lib.status_check(dev())
  b200.nn.tile_table(small, taps, 0, bad)
  with pytest.raises(b200._lib.OctConvError):
    b200._lib.status_check(dev())
  b200._lib.status_check(dev())

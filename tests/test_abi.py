"""CPU checks of the C-ABI library: it loads, exports every symbol declared in
include/octconv.h, validates arguments without touching a GPU, and the host
logic around it (shape rules, sharding, module signatures) behaves."""
import ctypes
import os
import re

import pytest
import torch

import ocnn_pytorch_b200 as b200
from ocnn_pytorch_b200 import _lib

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
  text = open(os.path.join(ROOT, 'include', 'octconv.h')).read()
  text = re.sub(r'/\*.*?\*/', '', text, flags=re.S)
  return sorted(set(re.findall(r'\b(oc_[a-z0-9_]+)\s*\(', text)))


def test_library_exports_every_declared_symbol():
  lib = _lib.lib()
  names = declared_symbols()
  assert len(names) >= 30
  for n in names:
    assert hasattr(lib, n), 'missing export %s' % n
    assert n in _lib.PROTOTYPES, 'no ctypes prototype for %s' % n
  assert sorted(_lib.PROTOTYPES) == names
  assert lib.oc_version() >= 100


def test_argument_errors_need_no_gpu():
  lib = _lib.lib()
  assert lib.oc_xyz2key(None, None, None, None, _lib.OC_I64, 10, 99, None, None) == -1
  assert b'depth' in lib.oc_last_error()
  assert lib.oc_xyz2key(None, None, None, None, _lib.OC_I64, 10, 5, None, None) == -1
  assert lib.oc_neigh_full(-1, 1, None, None) == -1
  taps = _lib.int_array([0, 1, 99])
  assert lib.oc_conv_fwd(None, 0, None, 0, 0, None, None, 8, 27, taps, 3, 10, 4, 4, 0, None, None, 0, None) == -1
  assert b'tap' in lib.oc_last_error()
  taps = _lib.int_array(list(range(27)))
  assert lib.oc_conv_fwd(None, 0, None, 0, 0, None, None, 8, 27, taps, 27, 10, 4, 4, 7, None, None, 0, None) == -1
  assert lib.oc_conv_fwd(None, 0, None, 0, 0, None, None, 3, 27, taps, 27, 10, 4, 4, 0, None, None, 0, None) == -1
  assert lib.oc_gn_workspace_bytes(0, 4) == 0
  assert lib.oc_conv_workspace_bytes(27, 64, 64, _lib.OC_F16) > 0
  assert lib.oc_build_workspace_bytes(1000, 6, 2, 1) > 0
  assert lib.oc_build_workspace_bytes(1000, 99, 2, 1) == 0
  with pytest.raises(_lib.OctConvError):
    _lib.call('oc_key2xyz', None, 5, 17, None, None, None, None, None)


def test_cpu_tensors_are_rejected_loudly():
  x = torch.zeros(4, dtype=torch.int64)
  with pytest.raises(RuntimeError, match='no CPU path'):
    b200.octree.xyz2key(x, x, x, None, 5)
  conv = b200.nn.OctreeConv(4, 8)
  octree = b200.Octree(3, 1)
  octree.nnum[3] = 5
  with pytest.raises((RuntimeError, AssertionError)):
    conv(torch.zeros(5, 4), octree, 3)


def test_module_signatures_and_parameter_shapes():
  c = b200.nn.OctreeConv(6, 10, [3], 1, False, 'triton', True, int(2e8))
  assert tuple(c.weights.shape) == (27, 6, 10) and tuple(c.bias.shape) == (10,)
  d = b200.nn.OctreeDeconv(6, 10, [2], 2, True)
  assert tuple(d.weights.shape) == (8, 10, 6) and d.bias is None
  w = b200.nn.OctreeDWConv(12, [3, 1, 1])
  assert tuple(w.weights.shape) == (3, 1, 12)
  a = 3 ** 0.5 * (2.0 / (27 * 64 + 27 * 64)) ** 0.5      # xavier bound, ocnn/utils.py:160-166
  c = b200.nn.OctreeConv(64, 64)
  assert abs(float(c.weights.abs().max()) - a) < 1e-3 and abs(a - 1 / 24) < 1e-9
  bn = b200.nn.OctreeBatchNorm(7)
  assert set(bn.state_dict()) == set(torch.nn.BatchNorm1d(7).state_dict())
  gn = b200.nn.OctreeNorm(32, 'group_norm', 8, 4)
  assert gn.norm.nempty == 4            # the reference passes min_group_channels positionally
  o = b200.Octree(5, 2, 3)
  assert o.lut_parent.shape == (8, 27) and o.lut_child.shape == (8, 27)
  assert o.lut_kernel['222'].tolist() == [13, 14, 16, 17, 22, 23, 25, 26]
  assert o.nnum.dtype == torch.int64 and tuple(o.batch_nnum.shape) == (6, 3)


def test_shape_rules_match_reference_table():
  o = b200.Octree(4, 1)
  o.nnum = torch.tensor([1, 8, 64, 200, 800])
  o.nnum_nempty = torch.tensor([1, 8, 25, 100, 300])
  from ocnn_pytorch_b200.nn.octree_conv import _OctreeConv, _OctreeDeconv
  cases = [(_OctreeConv, 1, False, 4, 800, 800), (_OctreeConv, 1, True, 4, 300, 300),
           (_OctreeConv, 2, False, 4, 800, 100), (_OctreeConv, 2, True, 4, 300, 100),
           (_OctreeDeconv, 2, False, 3, 100, 800), (_OctreeDeconv, 2, True, 3, 100, 300),
           (_OctreeDeconv, 1, False, 3, 200, 200)]
  for cls, stride, nempty, depth, in_h, out_h in cases:
    m = cls(4, 4, [3], stride, nempty)
    m.setup(o, depth)
    assert (m.in_h, m.out_h) == (in_h, out_h), (cls.__name__, stride, nempty)


def test_partition_octrees():
  P = b200.sharding.partition_octrees
  assert P([1] * 8, 4) == [[0, 1], [2, 3], [4, 5], [6, 7]]
  assert P([1] * 3, 1) == [[0, 1, 2]]
  parts = P([10, 1, 1, 1, 10, 1, 1, 1, 10, 3], 3)
  assert sum(parts, []) == list(range(10)) and all(len(p) > 0 for p in parts)
  assert P([5, 5], 4) == [[0], [1], [], []]
  for B, G in [(16, 8), (32, 8), (64, 8), (7, 2)]:
    parts = P(list(range(1, B + 1)), G)
    assert sum(parts, []) == list(range(B))
    assert all(len(p) > 0 for p in parts)

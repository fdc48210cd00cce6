"""convert_octree_ops: the module-tree swapper (the counterpart of convert_conv_triton,
ocnn/nn/octree_conv_t.py:139-160)."""
import os
import sys

import pytest
import torch

import ocnn_pytorch_b200 as b200

REF = os.environ.get('REFERENCE_ROOT', '/root/reference')


def test_reference_models_are_fully_swapped():
  # Needs the reference checkout (absent on the GPU box): every operator module of ocnn.models.*
  # is replaced, parameters and buffers are shared, state_dict keys do not change.
  if not os.path.isdir(os.path.join(REF, 'ocnn')):
    pytest.skip('reference checkout not present')
  sys.path.insert(0, REF)
  os.environ['OCNN_DISABLE_TRITON'] = '1'
  try:
    import ocnn
  finally:
    sys.path.remove(REF)
  models = [ocnn.models.UNet(4, 20, nempty=True), ocnn.models.ResNet(4, 10, 18, 3, nempty=False),
            ocnn.models.SegNet(4, 8, stages=3, nempty=True), ocnn.models.LeNet(4, 10, 3, nempty=False)]
  leaf_ops = ('OctreeConv', 'OctreeDeconv', 'OctreeDWConv', 'OctreeGroupNorm', 'OctreeMaxPool', 'OctreeMaxUnpool',
              'OctreeGlobalPool', 'OctreeInterp', 'Octree2Voxel', 'OctreeDropPath', 'OctreeAvgPool')
  for model in models:
    before = {k: v.data_ptr() for k, v in model.state_dict().items()}
    b200.convert_octree_ops(model)
    after = {k: v.data_ptr() for k, v in model.state_dict().items()}
    assert before == after                                  # same keys, same storage
    for name, m in model.named_modules():
      tn, mod = type(m).__name__, type(m).__module__
      assert not (mod.startswith('ocnn.') and tn in leaf_ops), (name, tn)
      assert not isinstance(m, torch.nn.BatchNorm1d), name
    kinds = {type(m).__name__ for m in model.modules() if type(m).__module__.startswith('ocnn_pytorch_b200')}
    assert 'OctreeConv' in kinds and 'OctreeBatchNorm' in kinds


def _fake(name, **attrs):
  """A stand-in for a reference module: same class name, module path and attributes."""
  cls = type(name, (torch.nn.Module,), {'__module__': 'ocnn.nn.fake'})
  m = cls()
  for k, v in attrs.items():
    setattr(m, k, v)
  return m


@pytest.mark.gpu
def test_swapped_modules_compute_with_shared_parameters(golden):
  from gpu_utils import dev, synthetic_octree
  octree, _ = synthetic_octree(golden['synthetic'])
  depth = octree.depth
  w = torch.nn.Parameter(torch.randn(27, 16, 32, device=dev()) * 0.05)
  wd = torch.nn.Parameter(torch.randn(8, 16, 32, device=dev()) * 0.05)
  box = torch.nn.Module()
  box.conv = _fake('OctreeConv', in_channels=16, out_channels=32, kernel_size=[3, 3, 3], stride=1, nempty=False,
                   use_bias=False, weights=w, bias=None)
  box.deconv = _fake('OctreeDeconv', in_channels=32, out_channels=16, kernel_size=[2, 2, 2], stride=2, nempty=False,
                     use_bias=False, weights=wd, bias=None)
  box.pool = _fake('OctreeMaxPool', nempty=False, return_indices=False)
  box.glob = _fake('OctreeGlobalPool', nempty=False)
  box.interp = _fake('OctreeInterp', method='nearest', nempty=False, bound_check=True, rescale_pts=False)
  box.drop = _fake('OctreeDropPath', drop_prob=0.25, nempty=False, scale_by_keep=True)
  box.bn = torch.nn.BatchNorm1d(32).to(dev())
  bn_w = box.bn.weight
  b200.convert_octree_ops(box)
  assert type(box.conv) is b200.nn.OctreeConv and box.conv.weights is w
  assert type(box.deconv) is b200.nn.OctreeDeconv and box.deconv.weights is wd
  assert type(box.bn) is b200.nn.OctreeBatchNorm and box.bn.weight is bn_w
  assert type(box.pool) is b200.nn.OctreeMaxPool and type(box.glob) is b200.nn.OctreeGlobalPool
  assert type(box.interp) is b200.nn.OctreeInterp and box.interp.method == 'nearest' and box.interp.bound_check
  assert type(box.drop) is b200.nn.OctreeDropPath and box.drop.drop_prob == 0.25
  x = torch.randn(int(octree.nnum[depth]), 16, device=dev())
  y = box.bn(box.conv(x, octree, depth))
  ref = b200.nn.OctreeConv(16, 32).to(dev())
  with torch.no_grad():
    ref.weights.copy_(w)
  assert torch.equal(box.conv(x, octree, depth), ref(x, octree, depth))
  p = box.pool(y, octree, depth)
  assert p.shape == (int(octree.nnum[depth - 1]), 32)
  assert box.deconv(p, octree, depth - 1).shape == (int(octree.nnum[depth]), 16)
  assert box.glob(y, octree, depth).shape == (octree.batch_size, 32)
  y.sum().backward()
  assert w.grad is not None and bn_w.grad is not None

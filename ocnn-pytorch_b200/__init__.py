"""B200-native octree sparse-convolution hot path with the operator interface of
ocnn-pytorch: `octree` (Octree, Points, shuffled keys) and `nn` (OctreeConv,
OctreeDeconv, OctreeDWConv, pooling, upsampling, normalisation).  All compute is
done by liboctconv.so (hand-written sm_100a CUDA behind a C ABI); there is no
CPU, PyTorch or Triton fallback."""
from . import _lib
from . import utils
from . import octree
from . import nn
from . import synthetic
from . import sharding
from .octree import Octree, Points
from .convert import convert_octree_ops

__version__ = '0.1.0'
__all__ = ['octree', 'nn', 'utils', 'synthetic', 'sharding', 'Octree', 'Points',
           'convert_octree_ops']

from .shuffled_key import xyz2key, key2xyz
from .points import Points, merge_points
from .octree import Octree, merge_octrees, init_octree, KERNEL_TAPS

__all__ = ['xyz2key', 'key2xyz', 'Points', 'merge_points', 'Octree', 'merge_octrees',
           'init_octree', 'KERNEL_TAPS']

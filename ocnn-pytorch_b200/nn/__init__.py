from .octree_pad import octree_pad, octree_depad
from .octree_conv import (OctreeConv, OctreeDeconv, octree_conv, octree_deconv,
                          OctreeConvFunction, OctreeDeconvFunction, conv_gather, conv_wgrad,
                          tile_table, tiled_supported, TileTable, tap_mask_order, wgrad_by_mask)
from .octree_dwconv import OctreeDWConv, octree_dwconv
from .octree_pool import (octree_max_pool, octree_max_unpool, OctreeMaxPool, OctreeMaxUnpool,
                          octree_avg_pool, octree_global_pool, OctreeAvgPool, OctreeGlobalPool)
from .octree_align import search_value, octree_align
from .octree_drop import OctreeDropPath, DropPath
from .octree2vox import octree2voxel, Octree2Voxel
from .octree_interp import (octree_nearest_upsample, OctreeUpsample, octree_nearest_pts,
                            octree_linear_pts, OctreeInterp)
from .octree_norm import (OctreeBatchNorm, OctreeGroupNorm, OctreeInstanceNorm, OctreeNorm,
                          convert_sync_batchnorm, col_stats)

__all__ = [
    'octree_pad', 'octree_depad', 'OctreeConv', 'OctreeDeconv', 'octree_conv', 'octree_deconv', 'wgrad_by_mask',
    'OctreeConvFunction', 'OctreeDeconvFunction', 'conv_gather', 'conv_wgrad', 'tile_table', 'tiled_supported', 'TileTable', 'tap_mask_order', 'OctreeDWConv',
    'octree_dwconv', 'octree_max_pool', 'octree_max_unpool', 'OctreeMaxPool', 'OctreeMaxUnpool',
    'octree_avg_pool', 'octree_global_pool', 'OctreeAvgPool', 'OctreeGlobalPool', 'search_value', 'octree_align',
    'OctreeDropPath', 'DropPath', 'octree2voxel', 'Octree2Voxel',
    'octree_nearest_upsample', 'OctreeUpsample', 'octree_nearest_pts', 'octree_linear_pts', 'OctreeInterp', 'OctreeBatchNorm', 'OctreeGroupNorm',
    'OctreeInstanceNorm', 'OctreeNorm', 'convert_sync_batchnorm', 'col_stats',
]

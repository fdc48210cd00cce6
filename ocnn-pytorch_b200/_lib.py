"""ctypes binding of liboctconv.so, the C-ABI library of sm_100a kernels.

There is no fallback of any kind: if the shared library is missing the import of
this module's :func:`lib` raises, and every operator of the package needs it.
The prototypes below mirror ``include/octconv.h`` one to one.
"""
import ctypes
import os

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, 'liboctconv.so')

OC_F32, OC_F16, OC_BF16 = 0, 1, 2
OC_I64, OC_I32, OC_COORD_F32, OC_COORD_F64, OC_I16 = 10, 11, 12, 13, 14

_vp, _i, _i64, _sz, _f = (ctypes.c_void_p, ctypes.c_int, ctypes.c_int64, ctypes.c_size_t,
                          ctypes.c_float)
_ip = ctypes.POINTER(ctypes.c_int)
_i64p = ctypes.POINTER(ctypes.c_int64)
_fp = ctypes.POINTER(ctypes.c_float)
_vpp = ctypes.POINTER(ctypes.c_void_p)

# name -> (restype, argtypes); the order of arguments is that of include/octconv.h
PROTOTYPES = {
    'oc_version': (_i, []),
    'oc_last_error': (ctypes.c_char_p, []),
    'oc_status_check': (_i, [_vp]),
    'oc_xyz2key': (_i, [_vp, _vp, _vp, _vp, _i, _i64, _i, _vp, _vp]),
    'oc_key2xyz': (_i, [_vp, _i64, _i, _vp, _vp, _vp, _vp, _vp]),
    'oc_build_workspace_bytes': (_sz, [_i64, _i, _i, _i]),
    'oc_build_octree_count': (_i, [_vp, _vp, _i, _i64, _i, _i, _i, _fp, _f, _vp, _sz, _i64p, _vp]),
    'oc_build_octree_emit': (_i, [_vp, _vp, _vp, _i, _i64, _i, _i, _i, _fp, _f, _vp, _i64p, _vpp,
                                  _vpp, _vp, _vp, _vp, _vp, _vp]),
    'oc_full_layer': (_i, [_i, _i, _vp, _vp, _vp]),
    'oc_grow_layer': (_i, [_vp, _vp, _i64, _vp, _vp, _vp]),
    'oc_neigh_full': (_i, [_i, _i, _vp, _vp]),
    'oc_neigh_from_parent': (_i, [_vp, _vp, _i64, _vp, _vp, _vp]),
    'oc_nempty_index_workspace_bytes': (_sz, [_i64]),
    'oc_nempty_index': (_i, [_vp, _i64, _vp, _vp, _sz, _vp]),
    'oc_neigh_variant': (_i, [_vp, _vp, _vp, _i64, _i64, _ip, _i, _vp, _i, _vp]),
    'oc_neigh_inverse': (_i, [_vp, _i, _i64, _i, _ip, _i, _i64, _vp, _vp]),
    'oc_avgpool_fwd': (_i, [_vp, _vp, _i, _i, _ip, _i, _i64, _i, _i, _vp, _vp, _vp]),
    'oc_avgpool_bwd': (_i, [_vp, _vp, _vp, _i, _i, _ip, _i, _i64, _i, _i, _vp, _vp]),
    'oc_global_pool_workspace_bytes': (_sz, [_i64, _i, _i]),
    'oc_global_pool_fwd': (_i, [_vp, _i64p, _i, _i, _i, _vp, _vp, _sz, _vp]),
    'oc_scale_segments': (_i, [_vp, _i64p, _i, _vp, _i, _i, _vp, _vp]),
    'oc_search_key': (_i, [_vp, _i64, _vp, _i64, _vp, _vp]),
    'oc_interp_corners': (_i, [_vp, _i64, _vp, _i64, _i, _i, _vp, _vp, _vp]),
    'oc_rows_gather': (_i, [_vp, _vp, _i64, _i, _i, _vp, _vp]),
    'oc_rows_scatter_add': (_i, [_vp, _vp, _i64, _i, _i, _vp, _vp]),
    'oc_interp_linear_fwd': (_i, [_vp, _vp, _vp, _i64, _i, _i, _vp, _vp]),
    'oc_interp_linear_bwd': (_i, [_vp, _vp, _vp, _i64, _i, _i, _vp, _vp]),
    'oc_conv_workspace_bytes': (_sz, [_i, _i, _i, _i]),
    'oc_conv_fwd': (_i, [_vp, _i64, _vp, _i, _i, _vp, _vp, _i, _i, _ip, _i, _i64, _i, _i, _i, _vp,
                         _vp, _sz, _vp]),
    'oc_conv_tiled_supported': (_i, [_i, _i, _i, _i]),
    'oc_tap_masks': (_i, [_vp, _i, _i, _ip, _i, _i64, _vp, _vp]),
    'oc_tap_order_workspace_bytes': (_sz, [_i64]),
    'oc_tap_order': (_i, [_vp, _i, _i, _ip, _i, _i64, _i, _vp, _vp, _sz, _vp]),
    'oc_tile_table_bytes': (_sz, [_i64, _i]),
    'oc_tile_table_build': (_i, [_vp, _i, _i, _ip, _i, _i64, _i64, _vp, _vp, _sz, _vp]),
    'oc_conv_fwd_tiled': (_i, [_vp, _i64, _vp, _i, _i, _vp, _vp, _vp, _i, _i64, _i, _i, _i, _vp, _vp, _sz, _vp]),
    'oc_conv_wgrad_workspace_bytes': (_sz, [_i, _i, _i, _i64, _i]),
    'oc_conv_wgrad': (_i, [_vp, _i64, _vp, _i64, _vp, _i, _i, _ip, _i, _i, _i, _i, _vp, _vp, _vp,
                           _sz, _vp]),
    'oc_conv_wgrad_tiled': (_i, [_vp, _i64, _vp, _i64, _vp, _vp, _i, _i, _i, _i, _vp, _vp, _vp, _sz, _vp]),
    'oc_dwconv_fwd': (_i, [_vp, _i64, _vp, _vp, _i, _i, _ip, _i, _i64, _i, _i, _vp, _vp]),
    'oc_dwconv_wgrad_workspace_bytes': (_sz, [_i, _i, _i64]),
    'oc_dwconv_wgrad': (_i, [_vp, _i64, _vp, _i64, _vp, _i, _i, _ip, _i, _i, _i, _vp, _vp, _sz,
                             _vp]),
    'oc_pad': (_i, [_vp, _vp, _i64, _i64, _i, _i, _f, _vp, _vp]),
    'oc_depad': (_i, [_vp, _vp, _i64, _i, _i, _vp, _vp]),
    'oc_maxpool_fwd': (_i, [_vp, _vp, _vp, _i64, _i, _i, _vp, _vp, _vp]),
    'oc_maxpool_bwd': (_i, [_vp, _vp, _vp, _vp, _i64, _i64, _i, _i, _vp, _vp]),
    'oc_upsample_fwd': (_i, [_vp, _vp, _vp, _i64, _i, _i, _vp, _vp]),
    'oc_upsample_bwd': (_i, [_vp, _vp, _vp, _i64, _i, _i, _vp, _vp]),
    'oc_colstats_workspace_bytes': (_sz, [_i64, _i]),
    'oc_colstats': (_i, [_vp, _vp, _i64, _i, _i, _vp, _vp, _vp, _sz, _vp]),
    'oc_colstats_static': (_i, [_vp, _vp, _i64, _i, _i, _vp, _vp, _vp]),
    'oc_affine_cols': (_i, [_vp, _vp, _vp, _i64, _i, _i, _vp, _vp]),
    'oc_bn_bwd_apply': (_i, [_vp, _vp, _vp, _vp, _vp, _i64, _i, _i, _vp, _vp]),
    'oc_gn_workspace_bytes': (_sz, [_i, _i]),
    'oc_gn_fwd': (_i, [_vp, _i64p, _i, _i, _i, _f, _vp, _vp, _i, _vp, _vp, _vp, _vp, _sz, _vp]),
    'oc_gn_bwd': (_i, [_vp, _vp, _i64p, _i, _i, _i, _f, _vp, _vp, _vp, _i, _vp, _vp, _vp, _vp, _sz,
                       _vp]),
    'oc_batch_offsets': (_i, [_vp, _vp, _i64, _i, _i64p, _vp, _sz, _vp]),
}

_lib = None


class OctConvError(RuntimeError):
  """Raised when a C-ABI entry point returns a non-zero status."""


def lib():
  """Loads liboctconv.so once and installs the prototypes.  Raises if it is absent."""
  global _lib
  if _lib is None:
    if not os.path.exists(LIB_PATH):
      raise ImportError(
          'liboctconv.so is missing at %s: build it with `python %s` (needs nvcc). '
          'This package has no CPU or PyTorch fallback.' % (LIB_PATH, os.path.join(_HERE, 'build.py')))
    handle = ctypes.CDLL(LIB_PATH)
    for name, (res, args) in PROTOTYPES.items():
      fn = getattr(handle, name)
      fn.restype = res
      fn.argtypes = args
    _lib = handle
  return _lib


def check(status, what=''):
  if status != 0:
    msg = lib().oc_last_error().decode(errors='replace')
    raise OctConvError('%s failed with status %d: %s' % (what or 'liboctconv call', status, msg))


def call(name, *args):
  """Calls entry point `name` and raises OctConvError on a non-zero status."""
  check(getattr(lib(), name)(*args), name)


def status_check(device=None):
  """Synchronises the current stream and raises if a tensor-core kernel abandoned a wait."""
  call('oc_status_check', stream(device))


def ptr(t):
  """Raw data pointer of a tensor (or None)."""
  if t is None:
    return None
  return ctypes.c_void_p(t.data_ptr())


def stream(device=None):
  return ctypes.c_void_p(torch.cuda.current_stream(device).cuda_stream)


def int_array(values):
  return (ctypes.c_int * len(values))(*[int(v) for v in values])


def i64_array(values):
  return (ctypes.c_int64 * len(values))(*[int(v) for v in values])


def f32_array(values):
  return (ctypes.c_float * len(values))(*[float(v) for v in values])


def ptr_array(tensors):
  return (ctypes.c_void_p * len(tensors))(*[t.data_ptr() if t is not None else None for t in tensors])


def dtype_code(dtype):
  if dtype == torch.float32:
    return OC_F32
  if dtype == torch.float16:
    return OC_F16
  if dtype == torch.bfloat16:
    return OC_BF16
  raise TypeError('unsupported feature dtype %s (float32, float16, bfloat16 only)' % dtype)


def require_cuda(*tensors):
  for t in tensors:
    if t is not None and not t.is_cuda:
      raise RuntimeError(
          'this operator runs only on CUDA tensors (got a %s tensor); there is no CPU path' %
          t.device.type)


def workspace(nbytes, device):
  return torch.empty(max(int(nbytes), 256), dtype=torch.uint8, device=device)

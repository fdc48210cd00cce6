"""Builds liboctconv.so (the C-ABI library of hand-written sm_100a kernels) in-tree with nvcc.

Usage: python build.py [--force]   (also called by __graft_entry__.build()).
nvcc cross-compiles for sm_100a without a GPU, so this runs on a CPU-only box.
"""
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, 'csrc')
LIB = os.path.join(HERE, 'liboctconv.so')
SOURCES = ['api.cu', 'keys.cu', 'build.cu', 'neigh.cu', 'conv_fma.cu', 'conv_tc.cu',
           'elementwise.cu', 'norm.cu', 'interp.cu', 'pool_extra.cu']
NVCC_FLAGS = ['-gencode', 'arch=compute_100a,code=sm_100a', '-lineinfo', '-O3', '-std=c++17',
              '--extended-lambda', '-Xcompiler', '-fPIC', '-Xcompiler', '-fvisibility=default']


def _newest_source_mtime():
  paths = [os.path.join(CSRC, f) for f in os.listdir(CSRC)]
  paths.append(os.path.join(HERE, '..', 'include', 'octconv.h'))
  return max(os.path.getmtime(p) for p in paths)


def build(force=False, verbose=False):
  """Compiles every .cu into an object and links the shared library; returns its path."""
  if not force and os.path.exists(LIB) and os.path.getmtime(LIB) >= _newest_source_mtime():
    return LIB
  nvcc = os.environ.get('NVCC', '/usr/local/cuda/bin/nvcc')
  objdir = os.path.join(HERE, 'build')
  os.makedirs(objdir, exist_ok=True)
  procs = []
  for src in SOURCES:
    obj = os.path.join(objdir, src.replace('.cu', '.o'))
    cmd = [nvcc] + NVCC_FLAGS + (['-Xptxas', '-v'] if verbose else []) + \
        ['-c', os.path.join(CSRC, src), '-o', obj]
    procs.append((src, obj, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT)))
  objs = []
  for src, obj, p in procs:
    out = p.communicate()[0].decode()
    if p.returncode != 0:
      raise RuntimeError('nvcc failed on %s:\n%s' % (src, out))
    if verbose:
      print(out)
    objs.append(obj)
  cmd = [nvcc, '-shared', '-o', LIB] + objs + ['-lcudart']
  out = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT)
  if out.returncode != 0:
    raise RuntimeError('link failed:\n%s' % out.stdout.decode())
  return LIB


if __name__ == '__main__':
  print(build(force='--force' in sys.argv, verbose='-v' in sys.argv))

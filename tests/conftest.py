import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
  sys.path.insert(0, ROOT)
GOLDEN = os.path.join(ROOT, 'tests', 'golden')


def pytest_configure(config):
  config.addinivalue_line('markers', 'gpu: test needs a CUDA device (run on a B200)')


def pytest_collection_modifyitems(config, items):
  # Keep the order of collection, but never try GPU tests on a box without one.
  try:
    import torch
    has_gpu = torch.cuda.is_available()
  except Exception:
    has_gpu = False
  if not has_gpu:
    skip = pytest.mark.skip(reason='no CUDA device')
    for item in items:
      if 'gpu' in item.keywords:
        item.add_marker(skip)


@pytest.fixture(scope='session')
def golden():
  class G:
    def __init__(self):
      self._cache = {}

    def __getitem__(self, name):
      if name not in self._cache:
        self._cache[name] = np.load(os.path.join(GOLDEN, name + '.npz'))
      return self._cache[name]
  return G()

import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
for p in (ROOT, os.path.join(ROOT, 'o-cnn_b200')):
  if p not in sys.path:
    sys.path.insert(0, p)


def pytest_configure(config):
  config.addinivalue_line('markers', 'gpu: needs a CUDA device (run on the B200 box)')


@pytest.fixture(scope='session')
def golden():
  """Inputs/outputs produced by the reference's own CPU code (tests/golden/make_golden.py)."""
  path = os.path.join(ROOT, 'tests', 'golden', 'reference_vectors.npz')
  return dict(np.load(path))


def same_bits(a, b):
  a, b = np.ascontiguousarray(a), np.ascontiguousarray(b)
  return a.shape == b.shape and a.dtype == b.dtype and \
      np.array_equal(a.view(np.uint8), b.view(np.uint8))

"""Helpers for the GPU parity tests: build a CUDA Octree from golden inputs."""
import numpy as np
import torch

import ocnn_pytorch_b200 as b200


def dev():
  return torch.device('cuda', 0)


def to_np(t):
  return t.detach().float().cpu().numpy() if t.is_floating_point() else t.detach().cpu().numpy()


def build(points, normals=None, features=None, batch_id=None, batch_size=1, depth=5, full_depth=2,
          neigh=True):
  d = dev()
  f = lambda a: None if a is None else torch.from_numpy(np.ascontiguousarray(a)).to(d)
  pc = b200.octree.Points(f(points), f(normals), f(features), batch_id=f(batch_id),
                          batch_size=batch_size)
  octree = b200.Octree(depth, full_depth, batch_size, device=d)
  idx = octree.build_octree(pc)
  if neigh:
    octree.construct_all_neigh()
  return octree, idx


def synthetic_octree(syn):
  return build(syn['points'], syn['normals'], syn['features'], syn['batch_id'],
               int(syn['batch_size']), int(syn['depth']), int(syn['full_depth']))

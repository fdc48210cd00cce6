"""Data-parallel sharding of a batch of octrees: rank r of G owns whole octrees.

Octrees of a batch never reference each other (neighbour tables stay inside one
octree, GroupNorm is per octree), so the convolution path needs no collective.
The only exchanges are BatchNorm statistics (see nn.convert_sync_batchnorm) and
gathering results."""
from typing import List, Sequence

import torch
import torch.distributed as dist


def partition_octrees(weights: Sequence[int], world_size: int) -> List[List[int]]:
  r''' Splits octree indices 0..B-1 into `world_size` contiguous groups with
  nearly equal total weight (e.g. point counts).  Contiguous groups keep the
  batch-major node order, so concatenating per-rank outputs in rank order
  reproduces the single-process row order.  Every rank gets at least one
  octree when B >= world_size. '''
  B = len(weights)
  assert world_size >= 1
  if B < world_size:
    return [[i] if i < B else [] for i in range(world_size)]
  total = float(sum(weights))
  out, start, acc = [], 0, 0.0
  for r in range(world_size):
    remaining_ranks = world_size - r
    if remaining_ranks == 1:
      out.append(list(range(start, B)))
      break
    target = (total - acc) / remaining_ranks
    end, run = start, 0.0
    max_end = B - (remaining_ranks - 1)
    while end < max_end and (end == start or run + weights[end] / 2.0 <= target):
      run += weights[end]
      end += 1
    out.append(list(range(start, end)))
    acc += run
    start = end
  return out


def rank_slice(weights: Sequence[int], rank: int, world_size: int) -> List[int]:
  return partition_octrees(weights, world_size)[rank]


def all_gather_rows(local: torch.Tensor, group=None) -> torch.Tensor:
  r''' Concatenates per-rank ``(n_r, C)`` row blocks in rank order (ragged
  all-gather: sizes are exchanged first). '''
  if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size(group) == 1:
    return local
  world = dist.get_world_size(group)
  n = torch.tensor([local.shape[0]], dtype=torch.int64, device=local.device)
  sizes = [torch.zeros_like(n) for _ in range(world)]
  dist.all_gather(sizes, n, group=group)
  sizes = [int(s.item()) for s in sizes]
  m = max(sizes)
  pad = local.new_zeros((m,) + tuple(local.shape[1:]))
  pad[:local.shape[0]] = local
  bufs = [torch.empty_like(pad) for _ in range(world)]
  dist.all_gather(bufs, pad, group=group)
  return torch.cat([b[:s] for b, s in zip(bufs, sizes)], dim=0)

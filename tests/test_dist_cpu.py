"""world_size-2 gloo test of the host-side multi-GPU plumbing: whole octrees are
dealt to ranks, per-rank row blocks gather back in batch order, and the
BatchNorm statistics exchange sums to the single-process statistics."""
import os
import sys

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, port, q):
  sys.path.insert(0, ROOT)
  import ocnn_pytorch_b200 as b200
  os.environ['MASTER_ADDR'] = '127.0.0.1'
  os.environ['MASTER_PORT'] = str(port)
  dist.init_process_group('gloo', rank=rank, world_size=world)
  try:
    weights = [30, 10, 20, 40, 5]                  # "points" per octree
    rows = [3, 1, 2, 4, 1]                         # rows each octree contributes
    mine = b200.sharding.rank_slice(weights, rank, world)
    g = torch.Generator().manual_seed(0)
    full = torch.randn(sum(rows), 6, generator=g)
    offs = [0]
    for r in rows:
      offs.append(offs[-1] + r)
    local = torch.cat([full[offs[i]:offs[i + 1]] for i in mine]) if mine else full[:0]
    gathered = b200.sharding.all_gather_rows(local)
    ok_gather = torch.equal(gathered, full)
    # the packed (sum, sum of squares, count) exchange used by OctreeBatchNorm
    packed = torch.cat([local.sum(0), (local * local).sum(0), torch.tensor([float(local.shape[0])])])
    dist.all_reduce(packed)
    ref = torch.cat([full.sum(0), (full * full).sum(0), torch.tensor([float(full.shape[0])])])
    ok_stats = torch.allclose(packed, ref, atol=1e-5)
    q.put((rank, mine, ok_gather, ok_stats))
  finally:
    dist.destroy_process_group()


def test_two_rank_sharding_gather_and_stats():
  ctx = mp.get_context('spawn')
  q = ctx.Queue()
  port = 29500 + (os.getpid() % 500)
  procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
  for p in procs:
    p.start()
  res = sorted(q.get(timeout=120) for _ in range(2))
  for p in procs:
    p.join(timeout=60)
    assert p.exitcode == 0
  assert res[0][1] + res[1][1] == [0, 1, 2, 3, 4]
  assert all(r[2] and r[3] for r in res)

"""Benchmark of the octree-convolution hot path.

    python bench.py --gpus N --steps K --warmup W [--impl reference]

A step = OctreeConv 3x3x3 stride-1 forward + backward (input and weight
gradients) over one batch of 16 depth-8 octrees (100k surface points each),
Cin = Cout = 64, fp16 — the conv micro-benchmark configuration.  Every rank owns
its own batch (weak scaling, no collective on the path).  One JSON line is
printed by rank 0.

--impl reference times the CPU restatement of the reference's gather-GEMM
(oracle/, numpy, all host threads) on a bounded sample of the same workload.
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

METRIC = 'octree_conv_fwd_bwd_tflops'
UNIT = 'TFLOP/s'
DEPTH, FULL_DEPTH, BATCH, NPTS, CH = 8, 3, 16, 100000, 64
CONFIG_ID = 2


def workload_clouds(rank=0, batch=None, npts=NPTS):
  import ocnn_pytorch_b200 as b200
  batch = BATCH if batch is None else batch
  clouds = [b200.synthetic.mixed_cloud(1000 * CONFIG_ID + 100 * rank + i, npts) for i in range(batch)]
  pts = np.concatenate([c[0] for c in clouds])
  nrm = np.concatenate([c[1] for c in clouds])
  bid = np.concatenate([np.full(npts, i, np.float32) for i in range(batch)])
  return pts, nrm, bid


# dram__bytes_read + dram__bytes_write of one forward launch, per output row, from the ncu capture of
# the 4-octree case (537.6 MB read + 112.8 MB written / 1 001 304 rows, tile table ordered by tap
# mask; traffic grows in proportion to the rows)
DRAM_BYTES_PER_ROW = 649.5


def peaks():
  path = os.path.join(ROOT, 'MEASURED_PEAKS.json')
  if os.path.exists(path):
    p = json.load(open(path))
    return dict(tflops=float(p['bf16_tflops']), tflops_sustained=float(p.get('bf16_tflops_sustained', p['bf16_tflops'])),
                hbm=float(p['hbm_gbs']), src='measured')
  return dict(tflops=1590.0, tflops_sustained=1400.0, hbm=6650.0, src='fallback')


class ClockSampler:
  """Samples SM clocks and throttle reasons with nvidia-smi while a region runs."""

  def __init__(self, index=0):
    self.index = index
    self.rows = []
    self.proc = None

  def __enter__(self):
    q = ('clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,'
         'clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,'
         'clocks_event_reasons.sw_power_cap')
    try:
      self.proc = subprocess.Popen(['nvidia-smi', '-i', str(self.index), '--query-gpu=' + q,
                                    '--format=csv,noheader,nounits', '-lms', '50'],
                                   stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
      self.thread = threading.Thread(target=self._read, daemon=True)
      self.thread.start()
    except Exception:
      self.proc = None
    return self

  def _read(self):
    for line in self.proc.stdout:
      self.rows.append([c.strip() for c in line.split(',')])

  def __exit__(self, *a):
    if self.proc is not None:
      time.sleep(0.15)
      self.proc.terminate()
      try:
        self.proc.wait(timeout=5)
      except Exception:
        self.proc.kill()

  def summary(self):
    sm, mx, reasons = [], [], set()
    names = ['hw_slowdown', 'hw_thermal_slowdown', 'sw_thermal_slowdown', 'sw_power_cap']
    for r in self.rows:
      try:
        sm.append(float(r[0]))
        mx.append(float(r[1]))
      except Exception:
        continue
      for n, v in zip(names, r[2:6]):
        if v.lower().startswith('active'):
          reasons.add(n)
    if not sm:
      return {'sm_mhz': None, 'sm_max_mhz': None, 'reasons': [], 'samples': 0}
    return {'sm_mhz': float(np.median(sm)), 'sm_max_mhz': float(max(mx)), 'reasons': sorted(reasons),
            'samples': len(sm)}


# --------------------------------------------------------------------------- CPU arm
def cpu_conv_sample(n_octrees=1, channels=CH, threads=None):
  """Builds `n_octrees` octrees of the workload with the oracle and returns a
  closure running conv forward + backward (fp32, numpy) plus its work figures."""
  from oracle import octree_oracle as orc
  pts, nrm, bid = workload_clouds(0, n_octrees)
  o = orc.build_octree(pts, nrm, None, bid, n_octrees, DEPTH, FULL_DEPTH)
  neighs = orc.construct_all_neigh(o['children'], o['nnum'], DEPTH, FULL_DEPTH, n_octrees)
  neigh = neighs[DEPTH]
  n = neigh.shape[0]
  rng = np.random.default_rng(0)
  x = rng.standard_normal((n, channels)).astype(np.float32)
  gy = rng.standard_normal((n, channels)).astype(np.float32)
  w = (rng.standard_normal((27, channels, channels)) / np.sqrt(27 * channels)).astype(np.float32)
  nnz = int((neigh >= 0).sum())

  def step():
    y = orc.conv_forward(x, w, neigh)
    gx = orc.conv_backward(gy, w, neigh, n)
    gw = orc.conv_weight_grad(x, gy, neigh)
    return float(y[0, 0] + gx[0, 0] + gw[0, 0, 0])
  return step, n, nnz


def run_reference(args):
  rank = int(os.environ.get('RANK', '0'))
  if rank != 0:
    return
  cores = os.cpu_count() or 1
  step, n, nnz = cpu_conv_sample(1)
  for _ in range(max(args.warmup, 0) and 1):
    step()
  t0 = time.perf_counter()
  for _ in range(args.steps):
    step()
  dt = (time.perf_counter() - t0) / args.steps
  flops = 3 * 2.0 * nnz * CH * CH
  val = flops / dt / 1e12
  sample = '1 of %d octrees (depth %d, %d rows, %d valid taps), fp32 numpy gather-GEMM fwd+dgrad+wgrad' % (
      BATCH, DEPTH, n, nnz)
  line = {
      'impl': 'reference', 'metric': METRIC, 'value': val, 'unit': UNIT, 'n_gpus': args.gpus,
      'steps': args.steps, 'warmup': args.warmup, 'ms_per_step': dt * 1e3, 'higher_is_better': True,
      'scaling': 'weak', 'vs_baseline': None, 'dtype': 'f32', 'data': 'synthetic',
      'config': workload_config(),
      'cpu_baseline': {'value': val, 'unit': UNIT, 'cores': cores, 'kind': 'port', 'sample': sample},
      'e2e': {'value': val, 'unit': UNIT, 'h2d_bytes_per_step': 0, 'd2h_bytes_per_step': 0},
  }
  print(json.dumps(line))


def workload_config():
  return {'workload': 'OctreeConv 3x3x3 s1 fwd+bwd, 16 octrees depth 8 (full_depth 3) x 100k surface '
                      'points, Cin=Cout=64, nempty=False',
          'l2': 'inputs (features + neighbour table, >600 MB) exceed the 126 MB L2',
          'flops': 'valid taps only: 3 passes x 2*nnz*Cin*Cout'}


# --------------------------------------------------------------------------- GPU arm
def run_ours(args):
  import torch
  import torch.distributed as dist
  import ocnn_pytorch_b200 as b200

  rank = int(os.environ.get('RANK', '0'))
  local_rank = int(os.environ.get('LOCAL_RANK', '0'))
  world = int(os.environ.get('WORLD_SIZE', '1'))
  if not torch.cuda.is_available():
    raise SystemExit('bench.py needs a CUDA device: the hot path has no CPU fallback')
  torch.cuda.set_device(local_rank)
  dev = torch.device('cuda', local_rank)
  if world > 1:
    os.environ.setdefault('MASTER_ADDR', '127.0.0.1')
    dist.init_process_group('nccl', rank=rank, world_size=world, device_id=dev)

  # ---- the batch of this rank (weak scaling: every rank has a full batch)
  pts, nrm, bid = workload_clouds(rank)
  h_pts = torch.from_numpy(pts).pin_memory()
  h_nrm = torch.from_numpy(nrm).pin_memory()
  h_bid = torch.from_numpy(bid).pin_memory()

  def build_octree():
    pc = b200.Points(h_pts.to(dev, non_blocking=True), h_nrm.to(dev, non_blocking=True),
                     batch_id=h_bid.to(dev, non_blocking=True), batch_size=BATCH)
    octree = b200.Octree(DEPTH, FULL_DEPTH, BATCH, dev)
    octree.build_octree(pc)
    octree.construct_all_neigh()
    return octree

  octree = build_octree()
  torch.cuda.synchronize()
  if args.mode == 'conv':
    return run_conv_only(args, b200, octree, dev)
  if args.mode == 'suite':
    return run_suite(args, b200, octree, dev)
  if args.mode == 'build':
    return run_build_lines(args, octree, dev, _make_emit(peaks()), torch.Generator(device=dev).manual_seed(0))
  # octree build throughput (secondary figure): host points -> octree + all neighbour tables
  t_build = []
  for i in range(3):
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    o2 = build_octree()
    torch.cuda.synchronize()
    t_build.append(time.perf_counter() - t0)
    del o2
  build_mpts = BATCH * NPTS / min(t_build) / 1e6

  n = int(octree.nnum[DEPTH])
  neigh = octree.neighs[DEPTH]
  nnz = int((neigh >= 0).sum().item())
  flops_valid = 3 * 2.0 * nnz * CH * CH
  flops_dense = 3 * 2.0 * n * 27 * CH * CH

  g = torch.Generator(device=dev).manual_seed(rank)
  conv = b200.nn.OctreeConv(CH, CH, [3], 1, False).to(dev).half()
  x = torch.randn(n, CH, device=dev, generator=g).half().requires_grad_()
  gy = torch.randn(n, CH, device=dev, generator=g).half()

  def step():
    conv.weights.grad = None
    x.grad = None
    y = conv(x, octree, DEPTH)
    y.backward(gy)
    return y

  def barrier():
    if world > 1:
      dist.barrier()
    torch.cuda.synchronize()

  for _ in range(max(args.warmup, 3)):
    step()
  barrier()
  ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
  with ClockSampler(local_rank) as clocks:
    barrier()
    ev0.record()
    for _ in range(args.steps):
      step()
    ev1.record()
    barrier()
  ms = ev0.elapsed_time(ev1) / args.steps
  if world > 1:
    t = torch.tensor([ms], device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms = float(t.item())

  # ---- dominant kernel alone: the gather implicit GEMM (forward launch)
  table, taps = octree.conv_table(DEPTH, '333', 1, False)
  tiles = octree.conv_tiles(DEPTH, '333', 1, False)
  xd = x.detach()
  reps = max(args.steps, 5)
  for _ in range(3):
    b200.nn.conv_gather(xd, conv.weights, False, None, table, taps, CH, CH, tiles)
  torch.cuda.synchronize()
  k0, k1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
  k0.record()
  for _ in range(reps):
    b200.nn.conv_gather(xd, conv.weights, False, None, table, taps, CH, CH, tiles)
  k1.record()
  torch.cuda.synchronize()
  ms_fwd = k0.elapsed_time(k1) / reps

  # ---- end to end: host buffers in, host buffers out, through the module API
  h_x = x.detach().cpu().pin_memory()
  h_gy = gy.cpu().pin_memory()
  h_y = torch.empty(n, CH, dtype=torch.float16).pin_memory()
  h_gx = torch.empty(n, CH, dtype=torch.float16).pin_memory()
  h_gw = torch.empty(27, CH, CH, dtype=torch.float32).pin_memory()

  # Three streams (upload, compute, download) and two sets of device buffers: the upload of step
  # i+1 and the download of step i-1 overlap the kernels of step i, as a data loader in front of a
  # training loop would arrange it.  Every step still moves all of its inputs and outputs.
  s_in, s_cmp, s_out = torch.cuda.Stream(dev), torch.cuda.Stream(dev), torch.cuda.Stream(dev)
  slots = []
  for _ in range(2):
    slots.append({'x': torch.empty(n, CH, dtype=torch.float16, device=dev).requires_grad_(),
                  'gy': torch.empty(n, CH, dtype=torch.float16, device=dev),
                  'in': torch.cuda.Event(), 'cmp': torch.cuda.Event(), 'out': torch.cuda.Event(), 'res': None})
    slots[-1]['cmp'].record()
    slots[-1]['out'].record()

  def e2e_step(i):
    sl = slots[i % 2]
    with torch.cuda.stream(s_in):
      s_in.wait_event(sl['cmp'])                  # the kernels that read this slot's inputs are done
      with torch.no_grad():
        sl['x'].copy_(h_x, non_blocking=True)
        sl['gy'].copy_(h_gy, non_blocking=True)
      sl['in'].record()
    with torch.cuda.stream(s_cmp):
      s_cmp.wait_event(sl['in'])
      s_cmp.wait_event(sl['out'])                 # this slot's previous results have left the device
      sl['x'].grad = None
      conv.weights.grad = None
      y = conv(sl['x'], octree, DEPTH)
      y.backward(sl['gy'])
      sl['res'] = (y.detach(), sl['x'].grad, conv.weights.grad.float())
      sl['cmp'].record()
    with torch.cuda.stream(s_out):
      s_out.wait_event(sl['cmp'])
      h_y.copy_(sl['res'][0], non_blocking=True)
      h_gx.copy_(sl['res'][1], non_blocking=True)
      h_gw.copy_(sl['res'][2], non_blocking=True)
      sl['out'].record()

  def e2e_join():
    cur = torch.cuda.current_stream(dev)
    for st in (s_in, s_cmp, s_out):
      cur.wait_stream(st)

  for st in (s_in, s_cmp, s_out):
    st.wait_stream(torch.cuda.current_stream(dev))
  for i in range(4):
    e2e_step(i)
  e2e_join()
  barrier()
  e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
  e0.record()
  for st in (s_in, s_cmp, s_out):
    st.wait_event(e0)
  for i in range(args.steps):
    e2e_step(i)
  e2e_join()
  e1.record()
  barrier()
  ms_e2e = e0.elapsed_time(e1) / args.steps
  if world > 1:
    t = torch.tensor([ms_e2e], device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_e2e = float(t.item())
  h2d = h_x.numel() * 2 + h_gy.numel() * 2
  d2h = h_y.numel() * 2 + h_gx.numel() * 2 + h_gw.numel() * 4

  pk = peaks()
  fwd_flops = 2.0 * nnz * CH * CH
  achieved = fwd_flops / (ms_fwd * 1e-3) / 1e12
  line = {
      'metric': METRIC, 'value': world * flops_valid / (ms * 1e-3) / 1e12, 'unit': UNIT,
      'n_gpus': world, 'steps': args.steps, 'warmup': max(args.warmup, 3), 'ms_per_step': ms,
      'higher_is_better': True, 'scaling': 'weak', 'vs_baseline': None, 'dtype': 'f16',
      'data': 'synthetic', 'config': workload_config(),
      'rows': n, 'valid_taps': nnz, 'dense_equiv_tflops': world * flops_dense / (ms * 1e-3) / 1e12,
      'ms_fwd_kernel': ms_fwd, 'build': {'mpts_per_s': build_mpts, 'points': BATCH * NPTS,
                                         'what': 'pinned host points -> octree + neighbour tables, depth 8'},
      'roofline': {'bound': 'tensor', 'achieved': achieved, 'peak': pk['tflops'], 'unit': 'TFLOP/s',
                   'frac': achieved / pk['tflops'], 'traffic': DRAM_BYTES_PER_ROW * n,
                   'kernel': 'conv gather implicit GEMM (forward launch), valid-tap FLOPs', 'peak_src': pk['src']},
      'e2e': {'value': world * flops_valid / (ms_e2e * 1e-3) / 1e12, 'unit': UNIT,
              'h2d_bytes_per_step': h2d, 'd2h_bytes_per_step': d2h, 'ms_per_step': ms_e2e,
              'overlap': 'upload / kernels / download on 3 streams, 2 sets of device buffers'},
      'gpu_launches': 6 * args.steps,
      'clocks': clocks.summary(),
  }
  if rank == 0 and world == 1:
    t0 = time.perf_counter()
    cstep, cn, cnnz = cpu_conv_sample(1)
    cstep()
    t1 = time.perf_counter()
    cstep()
    dt = time.perf_counter() - t1
    line['cpu_baseline'] = {
        'value': 3 * 2.0 * cnnz * CH * CH / dt / 1e12, 'unit': UNIT, 'cores': os.cpu_count() or 1,
        'kind': 'port', 'sample': '1 of %d octrees (%d rows), fp32 numpy gather-GEMM fwd+dgrad+wgrad, %.1f s' % (
            BATCH, cn, dt)}
  b200._lib.status_check(dev)
  if rank == 0:
    print(json.dumps(line))
  if world > 1:
    dist.destroy_process_group()


def run_conv_only(args, b200, octree, dev):
  """Profiler mode: warm-up + `steps` conv forward/backward passes, one JSON line with the time."""
  import torch
  n = int(octree.nnum[DEPTH])
  g = torch.Generator(device=dev).manual_seed(0)
  conv = b200.nn.OctreeConv(CH, CH, [3], 1, False).to(dev).half()
  x = torch.randn(n, CH, device=dev, generator=g).half().requires_grad_()
  gy = torch.randn(n, CH, device=dev, generator=g).half()
  for _ in range(args.warmup):
    conv(x, octree, DEPTH).backward(gy)
  torch.cuda.synchronize()
  e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
  e0.record()
  for _ in range(args.steps):
    conv(x, octree, DEPTH).backward(gy)
  e1.record()
  torch.cuda.synchronize()
  b200._lib.status_check(dev)
  # the three launches of a step, timed one by one
  table, taps = octree.conv_table(DEPTH, '333', 1, False)
  table_t, taps_t = octree.conv_table_transposed(DEPTH, '333', 1, False)
  tiles, tiles_t = octree.conv_tiles(DEPTH, '333', 1, False), octree.conv_tiles(DEPTH, '333', 1, False, True)
  tiles_w = octree.conv_tiles(DEPTH, '333', 1, False, False, by_mask=b200.nn.wgrad_by_mask(CH, CH))
  xd = x.detach()
  parts = {}
  for name, fn in (('fwd', lambda: b200.nn.conv_gather(xd, conv.weights, False, None, table, taps, CH, CH, tiles)),
                   ('dgrad', lambda: b200.nn.conv_gather(gy, conv.weights, True, None, table_t, taps_t, CH, CH, tiles_t)),
                   ('wgrad', lambda: b200.nn.conv_wgrad(xd, gy, table, taps, CH, CH, False, tiles_w))):
    fn()
    torch.cuda.synchronize()
    k0, k1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    k0.record()
    for _ in range(args.steps):
      fn()
    k1.record()
    torch.cuda.synchronize()
    parts['ms_' + name] = k0.elapsed_time(k1) / args.steps
  out = {'mode': 'conv', 'rows': n, 'batch': BATCH, 'ms_per_step': e0.elapsed_time(e1) / args.steps}
  out.update(parts)
  print(json.dumps(out))


LAST_DEVICE_ALLOCS = 0   # cudaMalloc calls of torch's allocator inside the last timed region of _time


SUITE_REPS, SUITE_WARM = None, None   # --suite-reps / --suite-warm: overrides for profiler captures


def _time(fn, reps=10, warm=3):
  import torch
  global LAST_DEVICE_ALLOCS
  reps = SUITE_REPS or reps
  warm = SUITE_WARM if SUITE_WARM is not None else warm
  for _ in range(warm):
    fn()
  torch.cuda.synchronize()
  a0 = torch.cuda.memory_stats().get('num_device_alloc', 0)
  e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
  e0.record()
  for _ in range(reps):
    fn()
  e1.record()
  torch.cuda.synchronize()
  LAST_DEVICE_ALLOCS = torch.cuda.memory_stats().get('num_device_alloc', 0) - a0
  return e0.elapsed_time(e1) / reps


def _make_emit(pk):
  def emit(name, ms, flops=None, nbytes=None, **kw):
    o = {'op': name, 'ms': round(ms, 4)}
    if flops is not None:
      o['tflops'] = round(flops / ms / 1e9, 2)
      o['frac_tensor_peak'] = round(flops / ms / 1e9 / pk['tflops'], 4)
    if nbytes is not None:
      o['gbs'] = round(nbytes / ms / 1e6, 1)
      o['frac_hbm_peak'] = round(nbytes / ms / 1e6 / pk['hbm'], 4)
    o.update(kw)
    allocs = kw.pop('allocs', LAST_DEVICE_ALLOCS)
    o.pop('allocs', None)
    if allocs:      # the timed region paid for cudaMalloc calls of torch's caching allocator
      o['device_allocs_in_timed_region'] = allocs
    print(json.dumps(o), flush=True)
  return emit


def run_suite(args, b200, octree, dev):
  """Secondary measurements: every kernel family of the path on the benchmark batch, one JSON
  line each (ms, achieved TFLOP/s or GB/s from algorithmic work, fraction of the measured peak)."""
  import torch
  pk = peaks()
  g = torch.Generator(device=dev).manual_seed(0)
  D = DEPTH

  emit = _make_emit(pk)

  for nempty in (False, True):
    n = int(octree.nnum_nempty[D] if nempty else octree.nnum[D])
    table, taps = octree.conv_table(D, '333', 1, nempty)
    table_t, taps_t = octree.conv_table_transposed(D, '333', 1, nempty)
    nnz = int((table >= 0).sum().item())
    for dtype in (torch.float16, torch.bfloat16):
      for C in (32, 64, 128, 256):
        if dtype == torch.bfloat16 and C not in (64, 256):
          continue
        x = torch.randn(n, C, device=dev, generator=g).to(dtype)
        gy = torch.randn(n, C, device=dev, generator=g).to(dtype)
        w = (torch.randn(27, C, C, device=dev, generator=g) / (27 * C) ** 0.5)
        fl = 2.0 * nnz * C * C
        tag = dict(C=C, dtype=str(dtype).split('.')[-1], nempty=nempty, rows=n, valid_taps=nnz)
        tl, tl_t = octree.conv_tiles(D, '333', 1, nempty), octree.conv_tiles(D, '333', 1, nempty, True)
        tl_w = octree.conv_tiles(D, '333', 1, nempty, False, by_mask=b200.nn.wgrad_by_mask(C, C, nempty))
        emit('conv333_fwd', _time(lambda: b200.nn.conv_gather(x, w, False, None, table, taps, C, C, tl)), flops=fl, **tag)
        emit('conv333_dgrad', _time(lambda: b200.nn.conv_gather(gy, w, True, None, table_t, taps_t, C, C, tl_t)), flops=fl, **tag)
        emit('conv333_wgrad', _time(lambda: b200.nn.conv_wgrad(x, gy, table, taps, C, C, False, tl_w)), flops=fl, **tag)
        del x, gy
  # strided / transposed path (bf16), depth-wise conv, pooling, upsampling, normalisation
  n8, n7 = int(octree.nnum[D]), int(octree.nnum[D - 1])
  for ks in ([3], [2]):
    conv = b200.nn.OctreeConv(64, 128, ks, 2, False).to(dev).bfloat16()
    deconv = b200.nn.OctreeDeconv(128, 64, ks, 2, False).to(dev).bfloat16()
    x = torch.randn(n8, 64, device=dev, generator=g).bfloat16().requires_grad_()
    gy = torch.randn(n8, 64, device=dev, generator=g).bfloat16()

    def step():
      x.grad = None
      y = deconv(conv(x, octree, D), octree, D - 1)
      y.backward(gy)
    tb, _ = octree.conv_table(D, '333' if ks == [3] else '222', 2, False)
    nz = int((tb >= 0).sum().item())
    emit('conv_s2_64to128 + deconv_s2_128to64 fwd+bwd (bf16, kernel %s)' % ks, _time(step, 5, 2),
         flops=2 * 3 * 2.0 * nz * 64 * 128, rows_fine=n8, rows_coarse=n7, valid_taps=nz)
    del x, gy
  C = 256
  s = 2
  x = torch.randn(n8, C, device=dev, generator=g).half()
  dw = b200.nn.OctreeDWConv(C, [3]).to(dev)
  table, taps = octree.conv_table(D, '333', 1, False)
  emit('dwconv333_fwd C=256 fp16', _time(lambda: dw(x, octree, D)), nbytes=2 * n8 * C * s + n8 * 27 * 8, rows=n8)
  xg = x.clone().requires_grad_()
  gdw = torch.randn(n8, C, device=dev, generator=g).half()

  def dw_step():
    xg.grad = None
    dw.weights.grad = None
    dw(xg, octree, D).backward(gdw)
  emit('dwconv333 fwd+bwd C=256 fp16', _time(dw_step), nbytes=3 * (2 * n8 * C * s + n8 * 27 * 8) + n8 * C * s, rows=n8)
  del xg, gdw
  emit('maxpool_fwd C=256 fp16', _time(lambda: b200.nn.octree_max_pool(x, octree, D)),
       nbytes=(n8 + n7) * C * s + int(octree.nnum_nempty[D - 1]) * C * 8, rows=n8)
  xc = torch.randn(n7, C, device=dev, generator=g).half()
  emit('upsample_nearest_fwd C=256 fp16', _time(lambda: b200.nn.octree_nearest_upsample(xc, octree, D - 1)),
       nbytes=(int(octree.nnum_nempty[D - 1]) + n8) * C * s, rows=n8)
  bn = b200.nn.OctreeBatchNorm(C).to(dev)
  emit('batchnorm_fwd (train) C=256 fp16', _time(lambda: bn(x)), nbytes=3 * n8 * C * s, rows=n8)
  gn = b200.nn.OctreeGroupNorm(C, 32).to(dev)
  emit('groupnorm_fwd C=256 fp16', _time(lambda: gn(x, octree, D)), nbytes=4 * n8 * C * s, rows=n8)
  idx = octree.nempty_index(D)
  xne = torch.randn(idx.numel(), C, device=dev, generator=g).half()
  emit('octree_pad C=256 fp16', _time(lambda: b200.nn.octree_pad(xne, octree, D)), nbytes=(idx.numel() + n8) * C * s)
  # key search and point interpolation: 4 M query points spread over the batch, C = 96 features at depth 8
  Ci, M = 96, 4 << 20
  xi = torch.randn(n8, Ci, device=dev, generator=g).half()
  q = torch.rand(M, 4, device=dev, generator=g)
  q[:, :3] *= float(1 << D)
  q[:, 3] = torch.floor(q[:, 3] * BATCH).clamp(max=BATCH - 1)
  # half of the queries sit on occupied cells, so that the gathers are real work
  cx, cy, cz, cb = octree.xyzb(D)
  pick = torch.randint(0, n8, (M // 2,), device=dev, generator=g)
  q[:M // 2] = torch.stack([cx[pick], cy[pick], cz[pick], cb[pick]], 1).float() + torch.tensor([0.3, 0.6, 0.4, 0.0], device=dev)
  emit('search_xyzb depth8 (4.2 M queries)', _time(lambda: octree.search_xyzb(q, D)), nbytes=M * (16 + 8 + 8) , rows=M)
  emit('octree_nearest_pts C=96 fp16', _time(lambda: b200.nn.octree_nearest_pts(xi, octree, D, q)),
       nbytes=M * (16 + 8) + M * Ci * s * 3 // 2, rows=M)
  emit('octree_linear_pts C=96 fp16', _time(lambda: b200.nn.octree_linear_pts(xi, octree, D, q)),
       nbytes=M * (16 + 8 * 12) + M * Ci * s, rows=M)
  del x, xc, xne, xi, q
  run_build_lines(args, octree, dev, emit, g)


def run_build_lines(args, octree, dev, emit, g):
  """Octree construction lines: build_octree and construct_all_neigh on clouds of 200k points."""
  import torch
  # octree construction: 64 clouds of 200k points, depth 10 (about 50 GB of neighbour tables)
  import ocnn_pytorch_b200 as B
  octree._invalidate()
  torch.cuda.empty_cache()
  nb, npts, depth = args.build_clouds, 200000, 10
  clouds = [B.synthetic.mixed_cloud(4000 + i, npts, jitter=0.005) for i in range(nb)]
  pts = torch.from_numpy(np.concatenate([c[0] for c in clouds])).to(dev)
  nrm = torch.from_numpy(np.concatenate([c[1] for c in clouds])).to(dev)
  feat = torch.randn(nb * npts, 3, device=dev, generator=g)
  bid = torch.from_numpy(np.concatenate([np.full(npts, i, np.float32) for i in range(nb)])).to(dev)
  holder = {}

  pc = B.Points(pts, nrm, feat, batch_id=bid, batch_size=nb)      # the input object, checked once

  def build_only():
    o = B.Octree(depth, 3, nb, dev)
    o.build_octree(pc)
    holder['o'] = o

  def neigh_only():
    holder['o'].neighs = [None] * (depth + 1)      # one generation of tables at a time
    holder['o'].construct_all_neigh()
  # three warm-up rounds: both generations of tables (the new one is built while the old one is
  # still referenced) then sit in torch's caching allocator, and no cudaMalloc is timed
  t_b = _time(build_only, 5, 3)
  allocs_b = LAST_DEVICE_ALLOCS
  t_n = _time(neigh_only, 5, 3)
  allocs_n = LAST_DEVICE_ALLOCS
  o = holder['o']
  P = nb * npts
  nn_ = [int(v) for v in o.nnum]
  passes = (3 * depth + 4 + 7) // 8
  build_bytes = P * (12 + 12 + 12) + P * 12 * 2 * passes + sum(nn_) * 12 + int(o.nnum_nempty[depth]) * 36
  # written: every table; read: the rows of the non-empty parents (nnum[d] / 8 of them) + all child pointers
  neigh_bytes = sum(nn_[1:]) * 27 * 8 + sum(nn_[1:]) // 8 * 27 * (8 + 4) + sum(nn_[:-1]) * 4
  emit('build_octree depth10 (%d x 200k pts, device resident)' % nb, t_b, nbytes=build_bytes, mpts_per_s=round(P / t_b / 1e3, 1), nnum=nn_, allocs=allocs_b)
  emit('construct_all_neigh depth10', t_n, nbytes=neigh_bytes, mpts_per_s=round(P / t_n / 1e3, 1), allocs=allocs_n)
  emit('build + neigh depth10', t_b + t_n, nbytes=build_bytes + neigh_bytes, mpts_per_s=round(P / (t_b + t_n) / 1e3, 1), allocs=allocs_b + allocs_n)
  B._lib.status_check(dev)


def main():
  global BATCH
  ap = argparse.ArgumentParser()
  ap.add_argument('--gpus', type=int, default=1)
  ap.add_argument('--steps', type=int, default=20)
  ap.add_argument('--warmup', type=int, default=5)
  ap.add_argument('--impl', default='ours', choices=['ours', 'reference'])
  ap.add_argument('--batch', type=int, default=BATCH,
                  help='octrees per rank (default 16 = the benchmark configuration; smaller values '
                       'are for profiler captures)')
  ap.add_argument('--build-clouds', type=int, default=64,
                  help="point clouds of 200k points in the suite's octree-construction lines")
  ap.add_argument('--suite-reps', type=int, default=None,
                  help='timed launches per suite line (default 10; 1 for a short profiler capture)')
  ap.add_argument('--suite-warm', type=int, default=None, help='warm-up launches per suite line (default 3)')
  ap.add_argument('--mode', default='full', choices=['full', 'conv', 'suite', 'build'],
                  help="'conv' runs only the timed conv steps (no build timing, e2e or CPU baseline)")
  args = ap.parse_args()
  global SUITE_REPS, SUITE_WARM
  SUITE_REPS, SUITE_WARM = args.suite_reps, args.suite_warm
  BATCH = args.batch
  if args.impl == 'reference':
    run_reference(args)
  else:
    run_ours(args)


if __name__ == '__main__':
  main()

"""Seeded synthetic point clouds standing in for the datasets and the shell
octrees of the reference's benchmarks (test/benchmark_conv.py, ScanNet-like
scenes).  numpy only; every cloud lies in [-0.99, 0.99]^3 and comes with unit
normals.  `seed = 1000 * config + octree_index` by convention."""
import numpy as np


def _unit(v):
  n = np.linalg.norm(v, axis=1, keepdims=True)
  return v / np.maximum(n, 1e-12)


def sphere_surface(rng, n, center=None, radius=None):
  center = rng.uniform(-0.6, 0.6, 3) if center is None else np.asarray(center, np.float64)
  radius = rng.uniform(0.1, 0.4) if radius is None else radius
  d = _unit(rng.standard_normal((n, 3)))
  return center + radius * d, d


def box_surface(rng, n, center=None, half=None):
  center = rng.uniform(-0.4, 0.4, 3) if center is None else np.asarray(center, np.float64)
  half = rng.uniform(0.15, 0.45, 3) if half is None else np.asarray(half, np.float64)
  area = np.array([half[1] * half[2], half[0] * half[2], half[0] * half[1]])
  axis = rng.choice(3, size=n, p=area / area.sum())
  sign = rng.choice([-1.0, 1.0], size=n)
  p = rng.uniform(-1.0, 1.0, (n, 3)) * half
  nrm = np.zeros((n, 3))
  p[np.arange(n), axis] = sign * half[axis]
  nrm[np.arange(n), axis] = sign
  return center + p, nrm


def torus_surface(rng, n, center=None, R=None, r=None):
  center = rng.uniform(-0.3, 0.3, 3) if center is None else np.asarray(center, np.float64)
  R = rng.uniform(0.3, 0.5) if R is None else R
  r = rng.uniform(0.05, 0.15) if r is None else r
  u = rng.uniform(0, 2 * np.pi, n)
  v = rng.uniform(0, 2 * np.pi, n)
  ring = np.stack([np.cos(u), np.sin(u), np.zeros(n)], 1)
  nrm = ring * np.cos(v)[:, None] + np.array([0, 0, 1.0]) * np.sin(v)[:, None]
  return center + R * ring + r * nrm, nrm


def plane_patch(rng, n):
  axis = rng.integers(0, 3)
  p = rng.uniform(-0.95, 0.95, (n, 3))
  p[:, axis] = rng.uniform(-0.9, 0.9)
  nrm = np.zeros((n, 3))
  nrm[:, axis] = 1.0
  return p, nrm


def _finish(p, nrm):
  p = np.clip(p, -0.99, 0.99).astype(np.float32)
  return p, nrm.astype(np.float32)


def spheres_cloud(seed, n_points=20000, n_spheres=3):
  r''' Points uniformly on the surfaces of `n_spheres` random spheres
  (centre U[-0.6,0.6]^3, radius U[0.1,0.4]); normals are radial. '''
  rng = np.random.default_rng(seed)
  per = [n_points // n_spheres] * n_spheres
  per[-1] += n_points - sum(per)
  parts = [sphere_surface(rng, m) for m in per]
  return _finish(np.concatenate([a for a, _ in parts]), np.concatenate([b for _, b in parts]))


def mixed_cloud(seed, n_points=100000, jitter=0.0):
  r''' Equal thirds on a random sphere, an axis-aligned box surface and a torus;
  optional N(0, jitter) noise on the coordinates. '''
  rng = np.random.default_rng(seed)
  a = n_points // 3
  parts = [sphere_surface(rng, a, radius=rng.uniform(0.3, 0.8), center=rng.uniform(-0.15, 0.15, 3)),
           box_surface(rng, a), torus_surface(rng, n_points - 2 * a)]
  p = np.concatenate([x for x, _ in parts])
  nrm = np.concatenate([y for _, y in parts])
  if jitter > 0:
    p = p + rng.normal(0.0, jitter, p.shape)
  return _finish(p, nrm)


def scene_cloud(seed, n_points=150000, n_boxes=12, n_planes=3):
  r''' Indoor-like scene: random axis-aligned boxes plus a few large planes. '''
  rng = np.random.default_rng(seed)
  k = n_boxes + n_planes
  per = [n_points // k] * k
  per[-1] += n_points - sum(per)
  parts = []
  for i in range(n_boxes):
    parts.append(box_surface(rng, per[i], center=rng.uniform(-0.7, 0.7, 3),
                             half=rng.uniform(0.05, 0.3, 3)))
  for i in range(n_planes):
    parts.append(plane_patch(rng, per[n_boxes + i]))
  return _finish(np.concatenate([a for a, _ in parts]), np.concatenate([b for _, b in parts]))


def shell_voxels(resolution):
  r''' Integer coordinates of the voxels of a thin spherical shell in a cube of
  side `resolution` (the shape used by the reference's conv benchmark,
  test/utils.py:43-70): resolution/2 - 1.25 <= |c - centre| <= resolution/2. '''
  out = []
  n = 128
  half = resolution / 2
  for i in range(0, resolution, n):
    xs = np.arange(i, min(i + n, resolution))
    for j in range(0, resolution, n):
      ys = np.arange(j, min(j + n, resolution))
      for k in range(0, resolution, n):
        zs = np.arange(k, min(k + n, resolution))
        g = np.stack(np.meshgrid(xs, ys, zs, indexing='ij'), -1).reshape(-1, 3)
        dist = np.sqrt((((g.astype(np.float32) - half + 0.5)) ** 2).sum(-1))
        out.append(g[(dist <= half) & (dist >= half - 1.25)])
  return np.concatenate(out).astype(np.int32)


def shell_points(depth):
  r''' Voxel centres of `shell_voxels(2^depth)` mapped to [-1, 1]^3, so that an
  octree of this depth built from them has exactly those leaves. '''
  res = 1 << depth
  v = shell_voxels(res)
  p = (v.astype(np.float32) + 0.5) * (2.0 / res) - 1.0
  nrm = _unit(p.astype(np.float64)).astype(np.float32)
  return p.astype(np.float32), nrm


def batch_clouds(config, batch, n_points, kind='mixed', jitter=0.0):
  r''' List of `(points, normals)` for octree indices 0..batch-1 of a benchmark
  configuration. '''
  gen = {'spheres': spheres_cloud, 'mixed': mixed_cloud, 'scene': scene_cloud}[kind]
  out = []
  for i in range(batch):
    seed = 1000 * config + i
    out.append(gen(seed, n_points, jitter=jitter) if kind == 'mixed' else gen(seed, n_points))
  return out

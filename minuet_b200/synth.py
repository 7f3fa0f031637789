"""Seeded synthetic point clouds with the shapes, sizes and value distributions
of the benchmark configurations.  No public dataset is used or reproduced: the
generators only follow the stated geometry (uniform cube, outdoor scan with a
noisy ground plane, boxes and range-dependent dropout, indoor room with boxes
and spheres).  Everything here is host-side numpy data preparation.
"""
from typing import List, Optional, Sequence, Tuple

import numpy as np


def sort_unique(coords: np.ndarray) -> np.ndarray:
    """Unique rows in lexicographic order, dimension 0 most significant."""
    coords = np.asarray(coords, dtype=np.int64)
    if coords.shape[0] == 0:
        return np.ascontiguousarray(coords.astype(np.int32))
    lo = coords.min(axis=0)
    span = coords.max(axis=0) - lo + 1
    if float(np.prod(span.astype(np.float64))) < 2.0 ** 62:
        # one 1-D unique over packed keys is an order of magnitude faster than axis=0
        key = np.zeros(coords.shape[0], dtype=np.int64)
        for k in range(coords.shape[1]):
            key = key * span[k] + (coords[:, k] - lo[k])
        key = np.unique(key)
        out = np.empty((key.shape[0], coords.shape[1]), dtype=np.int64)
        for k in range(coords.shape[1] - 1, -1, -1):
            out[:, k] = key % span[k] + lo[k]
            key //= span[k]
        return np.ascontiguousarray(out.astype(np.int32))
    coords = np.unique(coords, axis=0)
    return np.ascontiguousarray(coords.astype(np.int32))


def uniform_cloud(n: int = 50_000, extent: int = 256, seed: int = 0) -> np.ndarray:
    """``n`` distinct voxels drawn without replacement from ``[0, extent)^3``."""
    rng = np.random.default_rng(seed)
    ids = rng.choice(extent ** 3, size=n, replace=False)
    coords = np.stack([ids // (extent * extent), (ids // extent) % extent, ids % extent], axis=1)
    return sort_unique(coords)


def _box_surface(rng, centre, sides, n):
    """``n`` points on the surface of an axis-aligned box (area-weighted faces)."""
    sx, sy, sz = sides
    areas = np.array([sy * sz, sy * sz, sx * sz, sx * sz, sx * sy, sx * sy])
    face = rng.choice(6, size=n, p=areas / areas.sum())
    p = (rng.random((n, 3)) - 0.5) * np.asarray(sides)
    axis = face // 2
    sign = np.where(face % 2 == 0, -0.5, 0.5)
    p[np.arange(n), axis] = sign * np.asarray(sides)[axis]
    return p + np.asarray(centre)


def outdoor_cloud(seed: int, n_voxels: int = 120_000, voxel: float = 0.05) -> np.ndarray:
    """Outdoor-scan-like cloud: ground plane z ~ N(0, 0.1 m) over x, y in +-50 m,
    200 axis-aligned box surfaces with 1-10 m sides, points kept with probability
    1 - min(0.9, r / 60), z clipped to [-3, 1] m, voxelised at ``voxel`` metres and
    thinned (seeded) to ``n_voxels`` unique voxels."""
    rng = np.random.default_rng(seed)
    n_ground = int(n_voxels * 4.5)
    ground = np.empty((n_ground, 3))
    ground[:, :2] = rng.uniform(-50.0, 50.0, size=(n_ground, 2))
    ground[:, 2] = rng.normal(0.0, 0.1, size=n_ground)
    parts = [ground]
    for _ in range(200):
        sides = rng.uniform(1.0, 10.0, size=3)
        sides[2] = min(sides[2], 3.5)
        centre = np.array([rng.uniform(-50, 50), rng.uniform(-50, 50), sides[2] / 2 - 0.5])
        area = 2 * (sides[0] * sides[1] + sides[1] * sides[2] + sides[0] * sides[2])
        parts.append(_box_surface(rng, centre, sides, int(area * 40)))
    pts = np.concatenate(parts, axis=0)
    r = np.hypot(pts[:, 0], pts[:, 1])
    keep = rng.random(len(pts)) >= np.minimum(0.9, r / 60.0)
    pts = pts[keep]
    pts = pts[(np.abs(pts[:, 0]) < 50) & (np.abs(pts[:, 1]) < 50)]
    pts[:, 2] = np.clip(pts[:, 2], -3.0, 1.0 - 1e-6)
    vox = sort_unique(np.floor(pts / voxel))
    if len(vox) > n_voxels:
        pick = np.sort(rng.choice(len(vox), size=n_voxels, replace=False))
        vox = vox[pick]
    return np.ascontiguousarray(vox)


def indoor_cloud(seed: int, n_voxels: int = 200_000, voxel: float = 0.02) -> np.ndarray:
    """Indoor scene: surfaces of an 8 x 8 x 3 m room (floor, ceiling, four walls)
    plus 30 random boxes and spheres, voxelised at ``voxel`` metres and thinned
    (seeded) to ``n_voxels`` unique voxels."""
    rng = np.random.default_rng(seed)
    room = np.array([8.0, 8.0, 3.0])
    n_room = int(n_voxels * 2.2)
    parts = [_box_surface(rng, room / 2, room, n_room)]
    for i in range(30):
        centre = np.array([rng.uniform(0.5, 7.5), rng.uniform(0.5, 7.5), 0.0])
        if i % 2 == 0:
            sides = rng.uniform(0.3, 2.0, size=3)
            centre[2] = sides[2] / 2
            area = 2 * (sides[0] * sides[1] + sides[1] * sides[2] + sides[0] * sides[2])
            parts.append(_box_surface(rng, centre, sides, int(area * 3000)))
        else:
            radius = rng.uniform(0.15, 1.0)
            centre[2] = radius
            n = int(4 * np.pi * radius ** 2 * 3000)
            d = rng.normal(size=(n, 3))
            d /= np.linalg.norm(d, axis=1, keepdims=True)
            parts.append(centre + radius * d)
    pts = np.concatenate(parts, axis=0)
    pts = np.clip(pts, 0.0, room - 1e-6)
    vox = sort_unique(np.floor(pts / voxel))
    if len(vox) > n_voxels:
        pick = np.sort(rng.choice(len(vox), size=n_voxels, replace=False))
        vox = vox[pick]
    return np.ascontiguousarray(vox)


def make_batch(clouds: Sequence[np.ndarray]) -> Tuple[np.ndarray, Optional[np.ndarray]]:
    """Concatenate sorted clouds; returns ``(coords [N, 3] int32, batch_dims [B+1] int64)``."""
    coords = np.ascontiguousarray(np.concatenate(clouds, axis=0).astype(np.int32))
    bounds = np.zeros(len(clouds) + 1, dtype=np.int64)
    bounds[1:] = np.cumsum([len(c) for c in clouds])
    return coords, bounds


def outdoor_batch(num_clouds: int = 4, seed0: int = 1000, n_voxels: int = 120_000):
    return make_batch([outdoor_cloud(seed0 + i, n_voxels) for i in range(num_clouds)])


def indoor_batch(num_clouds: int = 8, seed0: int = 2000, n_voxels: int = 200_000):
    return make_batch([indoor_cloud(seed0 + i, n_voxels) for i in range(num_clouds)])


def kaiming_normal(shape: Tuple[int, int, int], seed: int) -> np.ndarray:
    """Kaiming-normal weights ``[K, C_in, C_out]`` with fan_in = K * C_in."""
    rng = np.random.default_rng(seed)
    k, c_in, _ = shape
    return (rng.standard_normal(shape) * np.sqrt(2.0 / (k * c_in))).astype(np.float32)


def random_small_batch(rng: np.random.Generator, num_clouds: int, n_per_cloud: int,
                       extent: int, ndim: int = 3, low: int = 0) -> Tuple[np.ndarray, np.ndarray]:
    """Small random clouds for tests: unique sorted rows in ``[low, low+extent)^ndim``."""
    clouds: List[np.ndarray] = []
    for _ in range(num_clouds):
        pts = rng.integers(low, low + extent, size=(n_per_cloud, ndim))
        clouds.append(sort_unique(pts))
    coords = np.ascontiguousarray(np.concatenate(clouds, axis=0).astype(np.int32))
    bounds = np.zeros(num_clouds + 1, dtype=np.int64)
    bounds[1:] = np.cumsum([len(c) for c in clouds])
    return coords, bounds

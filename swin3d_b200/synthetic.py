"""Seeded synthetic inputs with the shapes, sizes and value ranges of the benchmark configs.

They stand in for indoor scans (surface-sampled rooms): voxel coordinates on planar surfaces,
in-voxel offsets in [0,1), colours uniform in [0,1], normals equal to the surface normal.
Everything is generated with numpy on the host from an explicit seed.
"""
from dataclasses import dataclass
from typing import List, Optional

import numpy as np


@dataclass
class Scene:
    coords: np.ndarray   # int32 [N,4] (batch, x, y, z)
    local: np.ndarray    # float32 [N,3] in [0,1)
    rgb: np.ndarray      # float32 [N,3] in [0,1]
    normal: np.ndarray   # float32 [N,3] unit, axis aligned


def _rect(rng, axis, level, lo, hi, normal_sign):
    """All voxels of the axis-aligned rectangle {x[axis] = level, lo <= others < hi}."""
    others = [a for a in range(3) if a != axis]
    u = np.arange(lo[0], hi[0])
    v = np.arange(lo[1], hi[1])
    uu, vv = np.meshgrid(u, v, indexing="ij")
    pts = np.zeros((uu.size, 3), dtype=np.int64)
    pts[:, axis] = level
    pts[:, others[0]] = uu.ravel()
    pts[:, others[1]] = vv.ravel()
    nrm = np.zeros((uu.size, 3), dtype=np.float32)
    nrm[:, axis] = normal_sign
    return pts, nrm


def _dedup(pts, nrm):
    key = (pts[:, 0] << 42) | (pts[:, 1] << 21) | pts[:, 2]
    _, first = np.unique(key, return_index=True)
    first.sort()
    return pts[first], nrm[first]


def make_room(seed: int, target_voxels: int = 125_000, n_boxes: int = 20,
              extent_m=(8.0, 8.0, 3.0), batch_index: int = 0, dense_blobs: int = 2) -> Scene:
    """A room (floor, ceiling, four walls) with `n_boxes` axis-aligned boxes standing on the
    floor, voxelised at the voxel size that yields about `target_voxels` occupied voxels.
    Normals point into the room / out of the boxes; boxes keep a clearance of one window
    (5 voxels) from the ceiling so that no window holds both a +z and a -z normal (the last cRSE
    signal dimension must not see a difference of exactly +2, where the reference kernels read
    past their table).  A few small dense blobs add fully occupied windows (occupancy up to
    ws^3) as the benchmark description asks."""
    rng = np.random.default_rng(seed)
    ex, ey, ez = extent_m
    box_edges = rng.uniform(0.3, 1.5, size=(n_boxes, 3))
    box_edges[:, 2] = np.minimum(box_edges[:, 2], ez * 0.5)
    area = 2 * (ex * ey + ex * ez + ey * ez) + np.sum(
        2 * (box_edges[:, 0] * box_edges[:, 2] + box_edges[:, 1] * box_edges[:, 2]) +
        box_edges[:, 0] * box_edges[:, 1])
    voxel = float(np.sqrt(area / max(target_voxels, 1)))
    nx, ny, nz = (max(int(round(e / voxel)), 8) for e in (ex, ey, ez))
    parts, norms = [], []

    def add(p, n):
        parts.append(p)
        norms.append(n)

    add(*_rect(rng, 2, 0, (0, 0), (nx, ny), +1.0))           # floor, normal +z
    add(*_rect(rng, 2, nz - 1, (0, 0), (nx, ny), -1.0))      # ceiling, normal -z
    add(*_rect(rng, 0, 0, (0, 1), (ny, nz - 1), +1.0))       # walls
    add(*_rect(rng, 0, nx - 1, (0, 1), (ny, nz - 1), -1.0))
    add(*_rect(rng, 1, 0, (1, 1), (nx - 1, nz - 1), +1.0))
    add(*_rect(rng, 1, ny - 1, (1, 1), (nx - 1, nz - 1), -1.0))
    for b in range(n_boxes):
        sx, sy, sz = (max(int(round(e / voxel)), 2) for e in box_edges[b])
        sz = min(sz, nz - 12)
        if sz < 2:
            continue
        x0 = int(rng.integers(2, max(nx - sx - 2, 3)))
        y0 = int(rng.integers(2, max(ny - sy - 2, 3)))
        x1, y1, z1 = min(x0 + sx, nx - 2), min(y0 + sy, ny - 2), sz
        add(*_rect(rng, 2, z1, (x0, y0), (x1, y1), +1.0))        # top, normal +z
        add(*_rect(rng, 0, x0, (y0, 1), (y1, z1), -1.0))         # sides
        add(*_rect(rng, 0, x1 - 1, (y0, 1), (y1, z1), +1.0))
        add(*_rect(rng, 1, y0, (x0, 1), (x1, z1), -1.0))
        add(*_rect(rng, 1, y1 - 1, (x0, 1), (x1, z1), +1.0))
    for _ in range(dense_blobs):                              # fully occupied 5^3 .. 7^3 cubes
        e = 7
        x0 = int(rng.integers(2, nx - e - 2))
        y0 = int(rng.integers(2, ny - e - 2))
        z0 = 1
        g = np.stack(np.meshgrid(np.arange(x0, x0 + e), np.arange(y0, y0 + e),
                                 np.arange(z0, z0 + e), indexing="ij"), -1).reshape(-1, 3)
        nrm = np.zeros((g.shape[0], 3), dtype=np.float32)
        nrm[:, 2] = 1.0
        add(g.astype(np.int64), nrm)
    pts = np.concatenate(parts)
    nrm = np.concatenate(norms)
    pts, nrm = _dedup(pts, nrm)
    n = pts.shape[0]
    coords = np.concatenate([np.full((n, 1), batch_index, dtype=np.int64), pts], 1).astype(np.int32)
    local = rng.random((n, 3), dtype=np.float32)
    local = np.minimum(local, np.float32(1.0 - 2 ** -20))
    rgb = rng.random((n, 3), dtype=np.float32)
    return Scene(coords, local, rgb, nrm.astype(np.float32))


def make_planes_and_boxes(seed: int, n_voxels: int = 4096, grid: int = 64) -> Scene:
    """`n_voxels` distinct voxels of a grid^3 volume sampled from 3 random axis-aligned planes
    and the surfaces of 2 random axis-aligned boxes (the single-layer CPU-sized config)."""
    rng = np.random.default_rng(seed)
    parts, norms = [], []
    for _ in range(3):
        axis = int(rng.integers(0, 3))
        level = int(rng.integers(2, grid - 2))
        p, n = _rect(rng, axis, level, (0, 0), (grid, grid), 1.0)
        parts.append(p)
        norms.append(n)
    for _ in range(2):
        lo = rng.integers(2, grid // 2, size=3)
        hi = lo + rng.integers(6, grid // 2 - 2, size=3)
        for axis in range(3):
            o = [a for a in range(3) if a != axis]
            for level, sgn in ((lo[axis], -1.0), (hi[axis] - 1, 1.0)):
                if axis == 2 and sgn < 0:
                    continue  # open bottom: keeps +z / -z normals out of one window
                p, n = _rect(rng, axis, int(level), (lo[o[0]], lo[o[1]]), (hi[o[0]], hi[o[1]]), sgn)
                parts.append(p)
                norms.append(n)
    pts, nrm = _dedup(np.concatenate(parts), np.concatenate(norms))
    if pts.shape[0] < n_voxels:
        raise ValueError("not enough surface voxels; raise the grid size")
    sel = np.sort(rng.choice(pts.shape[0], size=n_voxels, replace=False))
    pts, nrm = pts[sel], nrm[sel]
    coords = np.concatenate([np.zeros((n_voxels, 1), dtype=np.int64), pts], 1).astype(np.int32)
    local = np.minimum(rng.random((n_voxels, 3), dtype=np.float32), np.float32(1.0 - 2 ** -20))
    rgb = rng.random((n_voxels, 3), dtype=np.float32)
    return Scene(coords, local, rgb, nrm.astype(np.float32))


def concat_scenes(scenes: List[Scene]) -> Scene:
    out = []
    for b, s in enumerate(scenes):
        c = s.coords.copy()
        c[:, 0] = b
        out.append(c)
    return Scene(np.concatenate(out), np.concatenate([s.local for s in scenes]),
                 np.concatenate([s.rgb for s in scenes]), np.concatenate([s.normal for s in scenes]))


def downsample_scene(scene: Scene, stride: int) -> Scene:
    """The scene as a later backbone stage sees it: voxels merged on a grid `stride` times coarser
    (coordinates become multiples of `stride`, the tensor stride of that stage, as after
    MinkowskiEngine pooling, microsoft/Swin3D Swin3D/modules/swin3d_layers.py:188-231); each coarse
    voxel keeps the signals of its first member."""
    if stride == 1:
        return scene
    c = scene.coords.astype(np.int64).copy()
    c[:, 1:] = np.floor_divide(c[:, 1:], stride) * stride
    _, first = np.unique(c, axis=0, return_index=True)
    first.sort()
    return Scene(c[first].astype(np.int32), scene.local[first], scene.rgb[first], scene.normal[first])


def signal_feats(scene: Scene, crse: str = "XYZ_RGB_NORM") -> np.ndarray:
    """float32 [N,F]: in-voxel position, then colour, then normal, as the cRSE mode asks."""
    cols = [scene.local]
    if "RGB" in crse:
        cols.append(scene.rgb)
    if "NORM" in crse:
        cols.append(scene.normal)
    return np.ascontiguousarray(np.concatenate(cols, 1), dtype=np.float32)


def quantise_signals(n_coords: np.ndarray, quant_size: int) -> np.ndarray:
    """n_cRSE = [xyz*quant, rgb*2quant, norm*2quant]  (swin3d_layers.py:514-536)."""
    out = n_coords.astype(np.float32).copy()
    out[:, 0:3] *= np.float32(quant_size)
    out[:, 3:] *= np.float32(2 * quant_size)
    return out


def table_sizes(window_size: int, quant_size: int, heads: int, head_dim: int, crse: str):
    """Elements per signal dimension: xyz tables have 2*ws*quant rows, rgb / normal tables
    2*2*(2*quant) rows (swin3d_layers.py:433-467)."""
    sizes = [2 * window_size * quant_size * heads * head_dim] * 3
    if "RGB" in crse:
        sizes += [2 * 2 * (2 * quant_size) * heads * head_dim] * 3
    if "NORM" in crse:
        sizes += [2 * 2 * (2 * quant_size) * heads * head_dim] * 3
    return sizes


def make_tables(seed: int, sizes, std: float = 0.02):
    """Three flat tables ~ N(0, std) truncated at +-2 std, like trunc_normal_(std=0.02)."""
    rng = np.random.default_rng(seed)
    n = int(sum(sizes))
    t = rng.normal(0.0, std, size=(3, n)).astype(np.float32)
    return np.clip(t, -2 * std, 2 * std)


def make_knn_scene(seed: int, n_query: int, n_src: int, cube_m: float = 10.0, n_planes: int = 6):
    """Points uniform on `n_planes` random axis-aligned planar rectangles inside a cube."""
    rng = np.random.default_rng(seed)

    def sample(n):
        which = rng.integers(0, n_planes, size=n)
        pts = np.empty((n, 3), dtype=np.float32)
        for p in range(n_planes):
            m = which == p
            cnt = int(m.sum())
            q = (rng.random((cnt, 3), dtype=np.float32) * rects[p, 1] + rects[p, 0]).astype(np.float32)
            q[:, axes[p]] = levels[p]
            pts[m] = q
        return pts

    axes = rng.integers(0, 3, size=n_planes)
    levels = rng.uniform(0.5, cube_m - 0.5, size=n_planes).astype(np.float32)
    lo = rng.uniform(0.0, cube_m * 0.4, size=(n_planes, 3)).astype(np.float32)
    ext = rng.uniform(cube_m * 0.3, cube_m * 0.6, size=(n_planes, 3)).astype(np.float32)
    rects = np.stack([lo, ext], 1)
    return sample(n_src), sample(n_query)

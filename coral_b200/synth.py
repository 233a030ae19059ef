"""Seeded synthetic inputs for the beam-search path: base vectors, training and test queries.

Stand-ins for the cross-modal datasets the reference is evaluated on (text-to-image
200-d L2; CLIP-style 512-d inner product, reference README.md:39-45): only their
shapes, metric and the base/query modality gap are modelled.  Everything here
produces *inputs*; none of it is on a timed path.  It runs on whatever torch device it
is given, so the same code makes the small CPU test cases and the full-size cases on
a GPU.  Graphs are built from these inputs by the library itself (coral_exact_knn ->
coral_build_nap -> coral_build_connect_enhance); `random_graph` only serves tests that
need no recall.
"""
from __future__ import annotations

import math
from dataclasses import dataclass

import torch

L2, IP = "l2", "ip"


def _gen(seed: int, device) -> torch.Generator:
    g = torch.Generator(device=device)
    g.manual_seed(int(seed))
    return g


def _normalize_(x: torch.Tensor) -> torch.Tensor:
    """Row-wise L2 normalisation as the reference does for inner product
    (reference src/uni.cpp:38-54): x *= 1/sqrt(sum x^2), rows of norm 0 untouched."""
    n = x.pow(2).sum(1, keepdim=True).sqrt()
    inv = torch.where(n > 0, 1.0 / n, torch.ones_like(n))
    return x.mul_(inv)


@dataclass
class Dataset:
    base: torch.Tensor          # [N, dim] fp32
    train: torch.Tensor         # [T, dim] fp32 training queries (used only to build the graph)
    test: torch.Tensor          # [Q, dim] fp32
    metric: str
    name: str


def make_l2_mixture(n: int, n_train: int, n_test: int, dim: int = 200, centers: int = 1000,
                    sigma: float = 0.3, rot_dims: int = 60, offset: float = 0.5,
                    seed: int = 20260001, device="cpu", chunk: int = 1 << 20,
                    draw_seed: int | None = None, latent_dim: int = 0, latent_jitter: float = 0.0) -> Dataset:
    """Text-to-image-like L2 case: a Gaussian mixture for the base; queries are the same
    mixture pushed through a fixed random rotation of a `rot_dims` subspace plus a fixed
    mean offset (the modality gap).  `seed` fixes the mixture and the queries; `draw_seed`
    (default: derived from seed) fixes the base points, so shards of one index can be drawn
    independently with the same structure and the same queries.

    With `latent_dim` = 0 the centres are i.i.d. N(0, I): every centre is equally far from every
    other, a point's neighbours all come from its own cluster, and a graph built from
    nearest-neighbour lists falls apart into one component per cluster.  With `latent_dim` > 0 the
    centres live in a random `latent_dim`-dimensional subspace (same overall variance), so clusters
    have near and far neighbours, and every point is also moved inside that subspace by
    `latent_jitter` x the centres' spread, so neighbouring clusters overlap the way neighbourhoods do
    in real embedding sets."""
    g = _gen(seed, device)
    gens = {False: _gen(seed + 1 if draw_seed is None else draw_seed, device), True: _gen(seed + 2, device)}
    if latent_dim > 0:
        basis, _ = torch.linalg.qr(torch.randn(dim, latent_dim, generator=g, device=device))
        lat_scale = math.sqrt(dim / latent_dim)
        ctr = (torch.randn(centers, latent_dim, generator=g, device=device) * lat_scale) @ basis.T
    else:
        basis, lat_scale = None, 0.0
        ctr = torch.randn(centers, dim, generator=g, device=device)
    qr, _ = torch.linalg.qr(torch.randn(rot_dims, rot_dims, generator=g, device=device))
    off = offset * torch.randn(dim, generator=g, device=device)

    def draw(m, as_query):
        out = torch.empty(m, dim, device=device)
        g = gens[as_query]
        for s in range(0, m, chunk):
            e = min(m, s + chunk)
            c = torch.randint(0, centers, (e - s,), generator=g, device=device)
            x = ctr[c] + sigma * torch.randn(e - s, dim, generator=g, device=device)
            if basis is not None and latent_jitter > 0:
                x += (torch.randn(e - s, latent_dim, generator=g, device=device) * (latent_jitter * lat_scale)) @ basis.T
            if as_query:
                x[:, :rot_dims] = x[:, :rot_dims] @ qr
                x += off
            out[s:e] = x
        return out

    return Dataset(draw(n, False), draw(n_train, True), draw(n_test, True), L2,
                   f"l2_mixture_{n}x{dim}")


def make_ip_cones(n: int, n_train: int, n_test: int, dim: int = 512, clusters: int = 1,
                  cos_uv: float = 0.3, sigma: float = 0.15, spread: float = 1.0, latent_dim: int = 16,
                  seed: int = 20260001, device="cpu", chunk: int = 1 << 20,
                  draw_seed: int | None = None, latent_jitter: float = 0.0) -> Dataset:
    """CLIP-like inner-product case: unit vectors.  Base points scatter around a mean
    direction u, queries around v with cos(u, v) = `cos_uv` (the modality gap).
    With `clusters` > 1 each base cluster j has its own direction normalise(u + spread*g_j)
    and a query aimed at cluster j is normalise(v + spread*g_j + noise): the two modalities
    share the cluster offsets g_j but not the mean direction.  The offsets live in a random
    `latent_dim`-dimensional subspace (0 = the full space), so that clusters have near and
    far neighbours the way real embedding sets do.  Per-point noise is isotropic with
    per-coordinate deviation sigma/sqrt(dim) (total deviation `sigma`).  `latent_jitter` > 0 also
    moves every point inside the latent subspace by that fraction of the offsets' spread, so that
    neighbouring clusters overlap; without it a nearest-neighbour list never leaves its cluster and
    a graph built from such lists has one component per cluster."""
    g = _gen(seed, device)
    u = torch.randn(dim, generator=g, device=device)
    u /= u.norm()
    w = torch.randn(dim, generator=g, device=device)
    w -= (w @ u) * u
    w /= w.norm()
    v = cos_uv * u + math.sqrt(1.0 - cos_uv * cos_uv) * w
    if clusters > 1 and latent_dim > 0:
        basis, _ = torch.linalg.qr(torch.randn(dim, latent_dim, generator=g, device=device))
        gj = (torch.randn(clusters, latent_dim, generator=g, device=device) @ basis.T) * (spread / math.sqrt(latent_dim))
    elif clusters > 1:
        gj = torch.randn(clusters, dim, generator=g, device=device) * (spread / math.sqrt(dim))
    else:
        gj = torch.zeros(1, dim, device=device)
    s = sigma / math.sqrt(dim)
    g_base = _gen(seed + 1 if draw_seed is None else draw_seed, device)
    g_query = _gen(seed + 2, device)

    def draw(m, mean, g):
        out = torch.empty(m, dim, device=device)
        for a in range(0, m, chunk):
            e = min(m, a + chunk)
            c = torch.randint(0, gj.shape[0], (e - a,), generator=g, device=device)
            x = mean + gj[c] + s * torch.randn(e - a, dim, generator=g, device=device)
            if latent_jitter > 0 and clusters > 1 and latent_dim > 0:
                x += (torch.randn(e - a, latent_dim, generator=g, device=device)
                      * (latent_jitter * spread / math.sqrt(latent_dim))) @ basis.T
            out[a:e] = _normalize_(x)
        return out

    return Dataset(draw(n, u, g_base), draw(n_train, v, g_query), draw(n_test, v, g_query), IP,
                   f"ip_cones_{n}x{dim}_c{clusters}")


# ----------------------------------------------------------------------------------------------
# exact k-NN (ground truth and training lists)
# ----------------------------------------------------------------------------------------------

def _scores(q: torch.Tensor, b: torch.Tensor, metric: str, b_sq=None) -> torch.Tensor:
    """Larger = closer.  fp32 matmul (TF32 is switched off by the callers)."""
    s = q @ b.T
    if metric == L2:
        if b_sq is None:
            b_sq = b.pow(2).sum(1)
        s = 2.0 * s - b_sq[None, :]          # -(|b|^2 - 2 q.b): |q|^2 is constant per row
    return s


@torch.no_grad()
def exact_knn(base: torch.Tensor, queries: torch.Tensor, k: int, metric: str,
              q_chunk: int = 2048, b_chunk: int = 262144) -> torch.Tensor:
    """Exact k nearest base rows per query (ties broken by the smaller id), int32 [Q, k]."""
    prev = torch.backends.cuda.matmul.allow_tf32
    torch.backends.cuda.matmul.allow_tf32 = False
    try:
        n = base.shape[0]
        out = torch.empty(queries.shape[0], k, dtype=torch.int32, device=base.device)
        for qs in range(0, queries.shape[0], q_chunk):
            q = queries[qs:qs + q_chunk]
            best_s = best_i = None
            for bs in range(0, n, b_chunk):
                b = base[bs:bs + b_chunk]
                s = _scores(q, b, metric)
                kk = min(k, s.shape[1])
                ts, ti = torch.topk(s, kk, dim=1)
                ti = ti + bs
                if best_s is None:
                    best_s, best_i = ts, ti
                else:
                    cs = torch.cat([best_s, ts], 1)
                    ci = torch.cat([best_i, ti], 1)
                    o = torch.topk(cs, min(k, cs.shape[1]), dim=1).indices
                    best_s, best_i = cs.gather(1, o), ci.gather(1, o)
            # order by (score desc, id asc)
            key = torch.argsort(best_i, dim=1, stable=True)
            bs_, bi_ = best_s.gather(1, key), best_i.gather(1, key)
            key = torch.argsort(bs_, dim=1, descending=True, stable=True)
            out[qs:qs + q.shape[0]] = bi_.gather(1, key)[:, :k].to(torch.int32)
        return out
    finally:
        torch.backends.cuda.matmul.allow_tf32 = prev


# ----------------------------------------------------------------------------------------------
# graphs for tests
# ----------------------------------------------------------------------------------------------

@dataclass
class Graph:
    adj: torch.Tensor        # int32 [N, deg_pad], -1 padded, valid ids first
    start_ids: torch.Tensor  # int32 [M]
    max_degree: int


def _pad_degree(max_degree: int) -> int:
    return 32 * ((max_degree + 31) // 32)


def random_graph(n: int, max_degree: int, n_start: int = 16, seed: int = 7, min_degree: int = 0,
                 device="cpu") -> Graph:
    """Uniform random neighbours with ragged degrees (for tests that need no recall)."""
    g = _gen(seed, device)
    deg_pad = _pad_degree(max_degree)
    adj = torch.randint(0, n, (n, deg_pad), generator=g, device=device, dtype=torch.int32)
    deg = torch.randint(min_degree, max_degree + 1, (n,), generator=g, device=device)
    col = torch.arange(deg_pad, device=device)[None, :]
    adj = torch.where(col < deg[:, None], adj, torch.full_like(adj, -1))
    start = torch.randperm(n, generator=g, device=device)[:n_start].to(torch.int32)
    return Graph(adj.contiguous(), start, max_degree)


# The benchmark configurations' data parameters (shapes from the configs; the latent structure is
# this build's choice, see make_ip_cones / make_l2_mixture).
CONFIGS = {
    "c1": dict(kind=L2, n=1_000_000, dim=200, groups=1000, latent_dim=16, latent_jitter=0.5, deg=32),
    "c2": dict(kind=IP, n=1_000_000, dim=512, groups=410, latent_dim=16, latent_jitter=0.5, deg=32),
    "c3": dict(kind=IP, n=10_000_000, dim=512, groups=4096, latent_dim=16, latent_jitter=0.5, deg=64),
    "c4": dict(kind=L2, n=12_500_000, dim=200, groups=10_000, latent_dim=16, latent_jitter=0.5, deg=32),
}


def make_config(name: str, n_train: int, n_test: int, n: int | None = None, seed: int = 20260001, device="cpu",
                draw_seed: int | None = None) -> Dataset:
    """The synthetic dataset of a benchmark configuration (optionally with fewer base points)."""
    c = CONFIGS[name]
    n = c["n"] if n is None else n
    if c["kind"] == IP:
        return make_ip_cones(n, n_train, n_test, dim=c["dim"], clusters=c["groups"], latent_dim=c["latent_dim"],
                             latent_jitter=c["latent_jitter"], seed=seed, device=device, draw_seed=draw_seed)
    return make_l2_mixture(n, n_train, n_test, dim=c["dim"], centers=c["groups"], latent_dim=c["latent_dim"],
                           latent_jitter=c["latent_jitter"], seed=seed, device=device, draw_seed=draw_seed)

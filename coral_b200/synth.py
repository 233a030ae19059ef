"""Seeded synthetic inputs for the beam-search path: vectors, queries, ground truth, graphs.

Stand-ins for the cross-modal datasets the reference is evaluated on (text-to-image
200-d L2; CLIP-style 512-d inner product, reference README.md:39-45): only their
shapes, metric and the base/query modality gap are modelled.  Everything here
produces *inputs* to the search path (a graph, entry points, queries, exact
ground truth); none of it is on the timed path.  It runs on whatever torch
device it is given so the same code builds the small CPU test cases and the
full-size cases on a GPU.

Graph construction follows the shape of the reference's build -- exact k_b-NN
lists of training queries projected onto the base set, then every node given
base-space neighbours so none is isolated (reference src/upd_gpu.cu:203-303,
src/enhance.cu:728-861) -- but is a simplified restatement whose only job is to
hand the search kernels a CORAL-shaped fixed-degree graph with good recall.
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
                    draw_seed: int | None = None) -> Dataset:
    """Text-to-image-like L2 case: a Gaussian mixture for the base; queries are the same
    mixture pushed through a fixed random rotation of a `rot_dims` subspace plus a fixed
    mean offset (the modality gap).  `seed` fixes the mixture and the queries; `draw_seed`
    (default: derived from seed) fixes the base points, so shards of one index can be drawn
    independently with the same structure and the same queries."""
    g = _gen(seed, device)
    gens = {False: _gen(seed + 1 if draw_seed is None else draw_seed, device), True: _gen(seed + 2, device)}
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
                  draw_seed: int | None = None) -> Dataset:
    """CLIP-like inner-product case: unit vectors.  Base points scatter around a mean
    direction u, queries around v with cos(u, v) = `cos_uv` (the modality gap).
    With `clusters` > 1 each base cluster j has its own direction normalise(u + spread*g_j)
    and a query aimed at cluster j is normalise(v + spread*g_j + noise): the two modalities
    share the cluster offsets g_j but not the mean direction.  The offsets live in a random
    `latent_dim`-dimensional subspace (0 = the full space), so that clusters have near and
    far neighbours the way real embedding sets do.  Per-point noise is isotropic with
    per-coordinate deviation sigma/sqrt(dim) (total deviation `sigma`)."""
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
# graph construction
# ----------------------------------------------------------------------------------------------

@dataclass
class Graph:
    adj: torch.Tensor        # int32 [N, deg_pad], -1 padded, valid ids first
    start_ids: torch.Tensor  # int32 [M]
    max_degree: int


def _pad_degree(max_degree: int) -> int:
    return 32 * ((max_degree + 31) // 32)


@torch.no_grad()
def _coarse_assign(base: torch.Tensor, n_cells: int, metric: str, seed: int, iters: int = 2,
                   chunk: int = 1 << 18):
    """A few Lloyd iterations from sampled centroids; returns (cell id per base row, centroids)."""
    n = base.shape[0]
    g = _gen(seed, base.device)
    cent = base[torch.randperm(n, generator=g, device=base.device)[:n_cells]].clone()
    assign = torch.empty(n, dtype=torch.int64, device=base.device)
    for it in range(iters + 1):
        c_sq = cent.pow(2).sum(1)
        for s in range(0, n, chunk):
            assign[s:s + chunk] = _scores(base[s:s + chunk], cent, L2, c_sq).argmax(1)
        if it == iters:
            break
        sums = torch.zeros_like(cent).index_add_(0, assign, base)
        cnt = torch.bincount(assign, minlength=n_cells).clamp_(min=1).to(base.dtype)
        cent = sums / cnt[:, None]
    return assign, cent


@torch.no_grad()
def _cell_knn(base: torch.Tensor, assign: torch.Tensor, n_cells: int, kk: int, metric: str):
    """Base-space k-NN restricted to each node's coarse cell.  int32 [N, kk], -1 padded."""
    n = base.shape[0]
    order = torch.argsort(assign, stable=True)
    counts = torch.bincount(assign, minlength=n_cells).tolist()
    out = torch.full((n, kk), -1, dtype=torch.int32, device=base.device)
    pos = 0
    for c in range(n_cells):
        m = counts[c]
        if m == 0:
            continue
        ids = order[pos:pos + m]
        pos += m
        if m == 1:
            continue
        x = base[ids]
        for s in range(0, m, 8192):
            xs = x[s:s + 8192]
            sc = _scores(xs, x, metric)
            if metric == L2:
                pass
            r = torch.arange(s, s + xs.shape[0], device=base.device)
            sc[torch.arange(xs.shape[0], device=base.device), r] = -float("inf")
            t = min(kk, m - 1)
            nb = torch.topk(sc, t, dim=1).indices
            out[ids[s:s + xs.shape[0]], :t] = ids[nb].to(torch.int32)
    return out


@torch.no_grad()
def build_graph(base: torch.Tensor, train: torch.Tensor, metric: str, max_degree: int = 32,
                k_b: int = 100, n_start: int = 16, seed: int = 20260004,
                train_knn: torch.Tensor | None = None, nap_per_node: int = 12,
                cell_size: int = 2048, list_batch: int = 2048, routers: bool = True,
                long_links: int = 4) -> Graph:
    """Fixed-degree directed graph in the reference's spirit.

    1. k_b-NN list of every training query (exact unless `train_knn` is given).
    2. Projection: inside each list, every member proposes its `nap_per_node`
       closest co-members (base-space distance) as out-neighbours and is proposed
       as in-neighbour in return.
    3. Every node also proposes its base-space neighbours inside its coarse cell,
       so nodes no training query reached still get in- and out-edges.
    4. Per node: proposals deduplicated, projection edges first then cell edges,
       each group closest first, cut to `max_degree`.
    5. Entry points: the closest base point to each of `n_start` k-means centroids
       of the training queries; with `routers`, each entry point's row is replaced by
       "router" nodes (closest base points to a finer k-means of the training queries).
    """
    dev = base.device
    n, dim = base.shape
    deg_pad = _pad_degree(max_degree)
    prev = torch.backends.cuda.matmul.allow_tf32
    torch.backends.cuda.matmul.allow_tf32 = False
    try:
        if train_knn is None:
            train_knn = exact_knn(base, train, min(k_b, n), metric)
        kb = train_knn.shape[1]
        m = min(nap_per_node, kb - 1)

        # ---- projection edges, grouped per node: nap[N, R], closest first
        src_l, dst_l, d_l = [], [], []
        eye = torch.eye(kb, dtype=torch.bool, device=dev)[None]
        for s in range(0, train_knn.shape[0], list_batch):
            ids = train_knn[s:s + list_batch].long()              # [B, kb]
            x = base[ids]                                         # [B, kb, dim]
            sc = torch.bmm(x, x.transpose(1, 2))                  # [B, kb, kb]
            if metric == L2:
                sq = x.pow(2).sum(2)
                sc = 2.0 * sc - sq[:, None, :] - sq[:, :, None]    # -|a-b|^2
            sc = sc.masked_fill(eye, -float("inf"))
            ts, ti = torch.topk(sc, m, dim=2)                     # [B, kb, m]
            u = ids[:, :, None].expand(-1, -1, m).reshape(-1).to(torch.int32)
            v = ids.gather(1, ti.reshape(ids.shape[0], -1)).reshape(-1).to(torch.int32)
            src_l += [u, v]                                       # forward and reverse proposals
            dst_l += [v, u]
            d_l += [-ts.reshape(-1), -ts.reshape(-1)]
            del x, sc, ts, ti
        key = torch.cat(src_l).long() * n + torch.cat(dst_l).long()
        dd = torch.cat(d_l)
        del src_l, dst_l, d_l
        o = torch.argsort(dd, stable=True)                        # smallest distance first ...
        key = key[o]
        del o, dd
        key = key[torch.argsort(key, stable=True)]                # ... inside every (u, v) group
        first = torch.ones_like(key, dtype=torch.bool)
        first[1:] = key[1:] != key[:-1]
        # one entry per (u, v) now; rank them per node by distance again: the distance order
        # was lost by the key sort, so recompute it for the survivors.
        key = key[first]
        del first
        uu, vv = key // n, key % n
        del key
        dd = torch.empty(uu.shape[0], device=dev)
        for s in range(0, uu.shape[0], 1 << 22):
            a_, b_ = base[uu[s:s + (1 << 22)]], base[vv[s:s + (1 << 22)]]
            dd[s:s + (1 << 22)] = ((a_ - b_).pow(2).sum(1) if metric == L2 else -(a_ * b_).sum(1))
            del a_, b_
        o = torch.argsort(dd, stable=True)
        uu, vv = uu[o], vv[o]
        del o, dd
        o = torch.argsort(uu, stable=True)
        uu, vv = uu[o], vv[o]
        del o
        start = torch.zeros(n + 1, dtype=torch.int64, device=dev)
        start[1:] = torch.cumsum(torch.bincount(uu, minlength=n), 0)
        rank = torch.arange(uu.shape[0], device=dev) - start[uu]
        keep = rank < max_degree
        nap = torch.full((n, max_degree), -1, dtype=torch.int32, device=dev)
        nap[uu[keep], rank[keep]] = vv[keep].to(torch.int32)
        del uu, vv, rank, keep, start

        # ---- base-space neighbours inside the coarse cell: cell_nb[N, R], closest first
        n_cells = max(1, n // cell_size)
        assign, cent = _coarse_assign(base, n_cells, metric, seed)
        cell_nb = _cell_knn(base, assign, n_cells, max_degree, metric)

        # ---- links between cells.  The representative of a cell is its member that appears in
        # the most training lists (closest to the centroid among equals); every node gets
        # `long_links` edges to representatives of cells near its own, and a representative
        # links to all of them, so that a search can walk from cell to cell.
        n_near = min(n_cells - 1, 16)
        if n_near > 0 and long_links > 0:
            pop = torch.bincount(train_knn.reshape(-1).long(), minlength=n).to(torch.float32)
            closeness = torch.empty(n, device=dev)
            for s in range(0, n, 1 << 20):
                closeness[s:s + (1 << 20)] = -(base[s:s + (1 << 20)] - cent[assign[s:s + (1 << 20)]]).pow(2).sum(1)
            o = torch.argsort(closeness, descending=True, stable=True)
            o = o[torch.argsort(pop[o], descending=True, stable=True)]
            o = o[torch.argsort(assign[o], stable=True)]             # per cell: most popular, then most central
            cell_of = assign[o]
            head = torch.ones_like(cell_of, dtype=torch.bool)
            head[1:] = cell_of[1:] != cell_of[:-1]
            rep = torch.full((n_cells,), -1, dtype=torch.int64, device=dev)
            rep[cell_of[head]] = o[head]
            live = rep >= 0
            cc = cent.clone()
            cc[~live] = float("inf")                                  # empty cells are nobody's neighbour
            dcell = torch.cdist(cent, cc)
            dcell.fill_diagonal_(float("inf"))
            near = torch.topk(dcell, n_near, dim=1, largest=False).indices      # [cells, n_near]
            # Nearest-cell lists are lopsided in high dimension (a few hub cells are everybody's
            # neighbour, others nobody's), so a cell also links back to every cell that lists it:
            # otherwise whole cells have no in-edge and cannot be reached from the entry points.
            src_c = torch.arange(n_cells, device=dev)[:, None].expand(-1, n_near).reshape(-1)
            dst_c = near.reshape(-1)
            # priority: back-links to the cells whose two nearest cells we are (their guaranteed
            # way in), then our own nearest cells, then the remaining back-links
            col_c = torch.arange(n_near, device=dev)[None, :].expand(n_cells, -1).reshape(-1)
            e_src = torch.cat([dst_c, src_c, dst_c])
            e_dst = torch.cat([src_c, dst_c, src_c])
            e_cls = torch.cat([torch.where(col_c < 2, 0, 3), torch.ones_like(col_c), torch.full_like(col_c, 2)])
            ok_e = live[e_src] & live[e_dst] & (e_cls < 3)
            e_src, e_dst, e_cls = e_src[ok_e], e_dst[ok_e], e_cls[ok_e]
            o_c = torch.argsort(e_cls, stable=True)
            e_src, e_dst, e_cls = e_src[o_c], e_dst[o_c], e_cls[o_c]
            o_c = torch.argsort(e_src * n_cells + e_dst, stable=True)           # duplicates: lowest class first
            e_src, e_dst, e_cls = e_src[o_c], e_dst[o_c], e_cls[o_c]
            first_c = torch.ones_like(e_src, dtype=torch.bool)
            first_c[1:] = (e_src[1:] != e_src[:-1]) | (e_dst[1:] != e_dst[:-1])
            e_src, e_dst, e_cls = e_src[first_c], e_dst[first_c], e_cls[first_c]
            o_c = torch.argsort(e_src * 4 + e_cls, stable=True)                 # per source: by class
            e_src, e_dst = e_src[o_c], e_dst[o_c]
            start_c = torch.zeros(n_cells + 1, dtype=torch.int64, device=dev)
            start_c[1:] = torch.cumsum(torch.bincount(e_src, minlength=n_cells), 0)
            rank_c = torch.arange(e_src.shape[0], device=dev) - start_c[e_src]
            width_c = 8 * n_near
            keep_c = rank_c < width_c
            near_sym = torch.full((n_cells, width_c), -1, dtype=torch.int64, device=dev)
            near_sym[e_src[keep_c], rank_c[keep_c]] = e_dst[keep_c]
            n_links = (near_sym >= 0).sum(1).clamp_(min=1)                         # [cells]
            near_rep = torch.where(near_sym >= 0, rep[near_sym.clamp(min=0)], torch.full_like(near_sym, -1))
            ll = min(long_links, n_near)
            node = torch.arange(n, device=dev)[:, None]
            pick = (node * 7 + torch.arange(ll, device=dev)[None, :] * 5) % n_links[assign][:, None]
            longs = near_rep[assign[:, None].expand(-1, ll), pick].to(torch.int32)        # [N, ll]
            rep_rows = near_rep[live][:, :max(1, max_degree // 2)].to(torch.int32)        # [live cells, <= R/2]
            rep_ids = rep[live]
        else:
            longs = torch.full((n, 0), -1, dtype=torch.int32, device=dev)
            rep_rows = rep_ids = None

        # ---- per node: links to other cells, projection edges, then cell edges; duplicates
        # of an earlier entry are dropped and the row cut to max_degree
        adj = torch.full((n, deg_pad), -1, dtype=torch.int32, device=dev)

        def pack_rows(parts):
            x = torch.cat(parts, 1)
            w = x.shape[1]
            eq = x[:, :, None] == x[:, None, :]
            eq &= torch.tril(torch.ones(w, w, dtype=torch.bool, device=dev), diagonal=-1)[None]
            x = torch.where(eq.any(2), torch.full_like(x, -1), x)
            o_ = torch.argsort((x < 0).to(torch.int8), dim=1, stable=True)
            return x.gather(1, o_)[:, :max_degree]

        width = longs.shape[1] + 2 * max_degree
        row_chunk = max(1, (1 << 27) // (width * width))
        for s in range(0, n, row_chunk):
            adj[s:s + row_chunk, :max_degree] = pack_rows(
                [longs[s:s + row_chunk], nap[s:s + row_chunk], cell_nb[s:s + row_chunk]])
        if rep_ids is not None:
            for s in range(0, rep_ids.shape[0], row_chunk):
                r_ = rep_ids[s:s + row_chunk]
                adj[r_, :max_degree] = pack_rows([rep_rows[s:s + row_chunk], nap[r_], cell_nb[r_]])
        del nap, cell_nb, longs

        # entry points and routers: k-means of the training queries; the base point closest
        # to each of `n_start` coarse centroids is an entry point, and the row of entry point
        # i is replaced by the base points closest to the i-th slice of n_start*max_degree
        # fine centroids, so that one expansion round fans out over the whole query space.
        def kmeans_nearest(kc, sd):
            g = _gen(sd, dev)
            kc = min(kc, train.shape[0])
            cent = train[torch.randperm(train.shape[0], generator=g, device=dev)[:kc]].clone()
            for _ in range(4):
                a = _scores(train, cent, L2).argmax(1)
                sums = torch.zeros_like(cent).index_add_(0, a, train)
                cnt = torch.bincount(a, minlength=cent.shape[0]).clamp_(min=1).to(train.dtype)
                cent = sums / cnt[:, None]
            if metric == IP:
                cent = _normalize_(cent)
            return exact_knn(base, cent, 1, metric)[:, 0].long(), cent

        start_ids = torch.unique(kmeans_nearest(4 * n_start, seed + 1)[0])[:n_start]
        if routers and n > 4 * n_start * max_degree:
            rt, rcent = kmeans_nearest(n_start * max_degree, seed + 2)
            # A router first points at cell representatives, then keeps what is left of its own
            # row.  Which representatives: for every training query, the routers the search would
            # rank best for it (query-to-base metric, as the kernel does) are pointed at the
            # representative of the cell holding that query's nearest base point; a router keeps
            # its most frequent targets and fills up with the cells closest to its query centroid.
            if rep_ids is not None:
                n_rep = min(max_degree // 2, rep_ids.shape[0])
                rt_vecs = base[rt]
                want = rep[assign[train_knn[:, 0].long()]]                      # [T] target representative
                r_l, t_l = [], []
                for s in range(0, train.shape[0], 8192):
                    top_r = torch.topk(_scores(train[s:s + 8192], rt_vecs, metric), min(3, rt.shape[0]), dim=1).indices
                    r_l.append(top_r.reshape(-1))
                    t_l.append(want[s:s + 8192, None].expand(-1, top_r.shape[1]).reshape(-1))
                pair = torch.cat(r_l) * n + torch.cat(t_l)
                pair = pair[torch.cat(t_l) >= 0]
                uniq, cnt_p = torch.unique(pair, return_counts=True)
                o_p = torch.argsort(cnt_p, descending=True, stable=True)
                uniq = uniq[o_p]
                o_p = torch.argsort(uniq // n, stable=True)
                uniq = uniq[o_p]
                r_of, t_of = uniq // n, uniq % n
                start_p = torch.zeros(rt.shape[0] + 1, dtype=torch.int64, device=dev)
                start_p[1:] = torch.cumsum(torch.bincount(r_of, minlength=rt.shape[0]), 0)
                rank_p = torch.arange(r_of.shape[0], device=dev) - start_p[r_of]
                keep_p = rank_p < n_rep
                learned = torch.full((rt.shape[0], n_rep), -1, dtype=torch.int64, device=dev)
                learned[r_of[keep_p], rank_p[keep_p]] = t_of[keep_p]
                nearest = rep_ids[torch.topk(_scores(rcent, base[rep_ids], metric), n_rep, dim=1).indices]
                for s in range(0, rt.shape[0], row_chunk):
                    r_ = rt[s:s + row_chunk]
                    links = pack_rows([learned[s:s + row_chunk].to(torch.int32),
                                       nearest[s:s + row_chunk].to(torch.int32)])[:, :n_rep]
                    adj[r_, :max_degree] = pack_rows([links, adj[r_, :max_degree]])
            rt = torch.unique(rt)
            rt = rt[~torch.isin(rt, start_ids)]
            rows = torch.full((start_ids.shape[0] * max_degree,), -1, dtype=torch.int32, device=dev)
            rows[:rt.shape[0]] = rt.to(torch.int32)[:rows.shape[0]]
            rows = rows.reshape(start_ids.shape[0], max_degree)
            adj[start_ids, :max_degree] = rows          # valid ids first: unused slots trail
            adj[start_ids, max_degree:] = -1
        return Graph(adj.contiguous(), start_ids.to(torch.int32), max_degree)
    finally:
        torch.backends.cuda.matmul.allow_tf32 = prev


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

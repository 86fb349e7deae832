"""K-NN graph construction sharded over the ranks of a ``torch.distributed`` group.

One process per GPU.  Every rank holds all points.  Trees are dealt round-robin
(rank g builds trees g, g+G, ...; tree t always uses seed ``seed + t``, so the
forest is the one a single GPU would build).  Each rank accumulates candidate
lists for all N rows from its own trees; one all-to-all (posted in a few pieces, so
that the merge of a piece runs behind the transfer of the next) then hands rank q
the G partial lists of the rows it owns and a G-way merge keeps the K best.  Before
each exploration sweep the owned index rows are all-gathered into the full
snapshot graph and every rank sweeps only its own rows.

The reference is single-GPU (device 0 hard-coded, reference src/rsfk.cu:679-684);
this module has no counterpart there.  The arithmetic is the engine's: on a GPU
``gpu_rsfk.device.DeviceForest`` (the CUDA kernels); the collectives are
``torch.distributed``'s (NCCL over NVLink on GPUs).
"""
import torch
import torch.distributed as dist


def tree_share(n_trees, rank, world):
    """Number of trees rank ``rank`` builds when ``n_trees`` are dealt round-robin."""
    return len(range(rank, n_trees, world))


def row_block(N, world):
    """Rows per rank: equal blocks of ceil(N/world); the last block may be short."""
    return (N + world - 1) // world


def owned_rows(N, rank, world):
    blk = row_block(N, world)
    begin = min(N, rank * blk)
    return begin, min(N, begin + blk)


def replicate_points(own_rows, N, group=None):
    """Every rank contributes its block of rows (``owned_rows``) and receives all N:
    the points cross the host link once in total and NVLink does the rest.
    ``own_rows`` is this rank's float32 [rows, D] device tensor."""
    world = dist.get_world_size(group) if dist.is_initialized() else 1
    if world == 1:
        return own_rows
    D = own_rows.shape[1]
    blk = row_block(N, world)
    if own_rows.shape[0] != blk:
        pad = torch.zeros((blk - own_rows.shape[0], D), dtype=own_rows.dtype, device=own_rows.device)
        own_rows = torch.cat([own_rows, pad])
    full = torch.empty((blk * world, D), dtype=own_rows.dtype, device=own_rows.device)
    dist.all_gather_into_tensor(full.view(-1), own_rows.contiguous().view(-1), group=group)
    return full[:N]


def _exchange_and_merge(engine, idx, dst, rows, K, world, rank, group, chunks):
    """Rank q receives every rank's partial lists of the rows it owns (block q of ``rows``
    padded to equal blocks) and merges them.  The exchange runs in ``chunks`` pieces of each
    block, all posted at once; the merge of piece c runs while the later pieces are still
    on the wire.  Returns the merged [blk, K] lists."""
    dev = idx.device
    blk = row_block(rows, world)
    pad = blk * world - rows
    if pad:
        pi, pd = engine.init_lists(pad, K, dev, False)
        idx = torch.cat([idx, pi])
        dst = torch.cat([dst, pd])
    recv_idx = torch.empty((world, blk, K), dtype=torch.int32, device=dev)
    recv_dst = torch.empty((world, blk, K), dtype=torch.float32, device=dev)
    own_idx = torch.empty((blk, K), dtype=torch.int32, device=dev)
    own_dst = torch.empty((blk, K), dtype=torch.float32, device=dev)
    chunks = max(1, min(int(chunks), blk))
    cb = (blk + chunks - 1) // chunks
    peer = (lambda g: dist.get_global_rank(group, g)) if group is not None else (lambda g: g)
    pieces, works = [], []
    for c0 in range(0, blk, cb):
        c1 = min(blk, c0 + cb)
        ops = []
        for g in range(world):
            if g == rank:
                continue
            ops.append(dist.P2POp(dist.isend, idx[g * blk + c0:g * blk + c1], peer(g), group))
            ops.append(dist.P2POp(dist.isend, dst[g * blk + c0:g * blk + c1], peer(g), group))
            ops.append(dist.P2POp(dist.irecv, recv_idx[g, c0:c1], peer(g), group))
            ops.append(dist.P2POp(dist.irecv, recv_dst[g, c0:c1], peer(g), group))
        pieces.append((c0, c1))
        works.append(dist.batch_isend_irecv(ops) if ops else [])
    for (c0, c1), ws in zip(pieces, works):
        for w in ws:
            w.wait()
        li = [idx[rank * blk + c0:rank * blk + c1] if g == rank else recv_idx[g, c0:c1] for g in range(world)]
        ld = [dst[rank * blk + c0:rank * blk + c1] if g == rank else recv_dst[g, c0:c1] for g in range(world)]
        engine.merge_lists(li, ld, own_idx[c0:c1], own_dst[c0:c1])
    return own_idx, own_dst


def build_knn_graph(engine, points, K, n_trees, min_children, max_children, max_depth=5000,
                    seed=0, sweeps=1, self_in_row=True, group=None, exchange_chunks=4, single=False):
    """Returns ``(idx_own, dist_own, row_begin, row_end)``: the canonical K-lists
    of this rank's rows ``[row_begin, row_end)``.

    ``engine`` supplies ``init_lists, forest, merge_lists, explore`` with the
    signatures of ``DeviceForest``; ``points`` is a float32 [N, D] tensor on the
    engine's device, identical on every rank.  ``single`` builds the whole graph on
    this rank alone, whatever the group (the graph a sharded build must reproduce).
    """
    world = dist.get_world_size(group) if dist.is_initialized() and not single else 1
    rank = dist.get_rank(group) if dist.is_initialized() and not single else 0
    N = points.shape[0]
    dev = points.device

    # 1. this rank's trees into full-N candidate lists
    idx, dst = engine.init_lists(N, K, dev, self_in_row)
    mine = tree_share(n_trees, rank, world)
    if mine > 0:
        engine.forest(points, idx, dst, mine, min_children, max_children, max_depth, seed,
                      first_tree=rank, tree_stride=world)
    begin, end = owned_rows(N, rank, world)
    if world == 1:
        own_idx, own_dst = idx, dst
    else:
        # 2. all-to-all: rank q receives every rank's rows [q*blk, (q+1)*blk) and merges them
        own_idx, own_dst = _exchange_and_merge(engine, idx, dst, N, K, world, rank, group, exchange_chunks)
        del idx, dst

    # 3. exploration sweeps over the owned rows against the gathered snapshot
    for _ in range(sweeps):
        if world == 1:
            snapshot = own_idx.clone()
        else:
            snapshot = torch.empty((row_block(N, world) * world, K), dtype=torch.int32, device=dev)
            dist.all_gather_into_tensor(snapshot.view(-1), own_idx.view(-1), group=group)
        if end > begin:
            engine.explore(points, snapshot, own_idx, own_dst, begin, end, list_row0=begin)
        del snapshot
    return own_idx[:end - begin], own_dst[:end - begin], begin, end


def search_queries(engine, points, queries, K, n_trees, min_children, max_children, max_depth=5000,
                   seed=0, group=None):
    """The query (base/query) search sharded like the graph build: every rank holds
    all base points and all queries, builds trees g, g+G, ... over the base points
    (tree t with seed ``seed + t``) and updates a list for every query from them;
    one all-to-all hands rank q the partial lists of the query rows it owns and a
    merge keeps the K best.  Returns ``(idx_own, dist_own, row_begin, row_end)``
    for this rank's query rows; the lists equal a single rank's bit for bit.

    ``engine`` supplies ``init_lists, forest_ann, merge_lists`` with the signatures
    of ``DeviceForest``.
    """
    world = dist.get_world_size(group) if dist.is_initialized() else 1
    rank = dist.get_rank(group) if dist.is_initialized() else 0
    NQ = queries.shape[0]
    dev = queries.device
    idx, dst = engine.init_lists(NQ, K, dev, False)
    mine = tree_share(n_trees, rank, world)
    if mine > 0:
        engine.forest_ann(points, queries, idx, dst, mine, min_children, max_children, max_depth, seed,
                          first_tree=rank, tree_stride=world)
    begin, end = owned_rows(NQ, rank, world)
    if world == 1:
        return idx, dst, begin, end
    own_idx, own_dst = _exchange_and_merge(engine, idx, dst, NQ, K, world, rank, group, 4)
    return own_idx[:end - begin], own_dst[:end - begin], begin, end


def gather_graph(idx_own, dist_own, N, group=None):
    """All ranks' owned rows concatenated into the full [N, K] graph (every rank)."""
    world = dist.get_world_size(group) if dist.is_initialized() else 1
    if world == 1:
        return idx_own, dist_own
    K = idx_own.shape[1]
    blk = row_block(N, world)
    dev = idx_own.device

    def padded(t, fill):
        if t.shape[0] == blk:
            return t.contiguous()
        extra = torch.full((blk - t.shape[0], K), fill, dtype=t.dtype, device=dev)
        return torch.cat([t, extra])

    full_i = torch.empty((blk * world, K), dtype=torch.int32, device=dev)
    full_d = torch.empty((blk * world, K), dtype=torch.float32, device=dev)
    dist.all_gather_into_tensor(full_i.view(-1), padded(idx_own, -1).view(-1), group=group)
    dist.all_gather_into_tensor(full_d.view(-1), padded(dist_own, float("inf")).view(-1), group=group)
    return full_i[:N], full_d[:N]

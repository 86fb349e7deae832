"""K-NN graph construction sharded over the ranks of a ``torch.distributed`` group.

One process per GPU.  Every rank holds all points.  Trees are dealt round-robin
(rank g builds trees g, g+G, ...; tree t always uses seed ``seed + t``, so the
forest is the one a single GPU would build).  Each rank accumulates candidate
lists for all N rows from its own trees; one all-to-all then hands rank q the G
partial lists of the rows it owns and a G-way merge keeps the K best.  Before
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


def build_knn_graph(engine, points, K, n_trees, min_children, max_children, max_depth=5000,
                    seed=0, sweeps=1, self_in_row=True, group=None):
    """Returns ``(idx_own, dist_own, row_begin, row_end)``: the canonical K-lists
    of this rank's rows ``[row_begin, row_end)``.

    ``engine`` supplies ``init_lists, forest, merge_lists, explore`` with the
    signatures of ``DeviceForest``; ``points`` is a float32 [N, D] tensor on the
    engine's device, identical on every rank.
    """
    world = dist.get_world_size(group) if dist.is_initialized() else 1
    rank = dist.get_rank(group) if dist.is_initialized() else 0
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
        # 2. all-to-all: rank q receives every rank's rows [q*blk, (q+1)*blk)
        blk = row_block(N, world)
        pad = blk * world - N
        if pad:
            pi, pd = engine.init_lists(pad, K, dev, False)
            idx = torch.cat([idx, pi])
            dst = torch.cat([dst, pd])
        recv_idx = torch.empty((world, blk, K), dtype=torch.int32, device=dev)
        recv_dst = torch.empty((world, blk, K), dtype=torch.float32, device=dev)
        dist.all_to_all_single(recv_idx.view(-1), idx.view(-1), group=group)
        dist.all_to_all_single(recv_dst.view(-1), dst.view(-1), group=group)
        del idx, dst
        own_idx = torch.empty((blk, K), dtype=torch.int32, device=dev)
        own_dst = torch.empty((blk, K), dtype=torch.float32, device=dev)
        engine.merge_lists([recv_idx[g] for g in range(world)], [recv_dst[g] for g in range(world)],
                           own_idx, own_dst)
        del recv_idx, recv_dst

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
    blk = row_block(NQ, world)
    pad = blk * world - NQ
    if pad:
        pi, pd = engine.init_lists(pad, K, dev, False)
        idx = torch.cat([idx, pi])
        dst = torch.cat([dst, pd])
    recv_idx = torch.empty((world, blk, K), dtype=torch.int32, device=dev)
    recv_dst = torch.empty((world, blk, K), dtype=torch.float32, device=dev)
    dist.all_to_all_single(recv_idx.view(-1), idx.view(-1), group=group)
    dist.all_to_all_single(recv_dst.view(-1), dst.view(-1), group=group)
    del idx, dst
    own_idx = torch.empty((blk, K), dtype=torch.int32, device=dev)
    own_dst = torch.empty((blk, K), dtype=torch.float32, device=dev)
    engine.merge_lists([recv_idx[g] for g in range(world)], [recv_dst[g] for g in range(world)],
                       own_idx, own_dst)
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

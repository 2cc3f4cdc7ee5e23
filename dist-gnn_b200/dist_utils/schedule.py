"""Stage schedules of the distributed SpMM: which sparse column block a rank multiplies at each stage and which
rank's feature block it needs for it.  Pure host logic shared by the CUDA stage loop and by the tests.

1D   (light_dist_gnn/models/gcn.py:21-29): P stages, stage s multiplies column block s by the block of rank s.
1.5D (1D_CAGNET/dist_15d.py:64-76, groups 1D_CAGNET/utils.py:36-49): P ranks = R row blocks x c replicas, rank ->
     (row block rank // c, replica rank % c).  Replica j handles P // c^2 consecutive column blocks starting at
     j * (P // c^2); the last replica also takes what is left.  The block of column block b comes from the rank that
     holds row block b in the same replica column, i.e. global rank b*c + j, inside the column group {j, j+c, ...}.
     Partial results are then summed over the row group {b*c .. b*c+c-1}.
"""
from collections import namedtuple

Stage = namedtuple('Stage', 'part root_global root_in_group')


def check_layout(world_size, rep):
    if rep < 1 or world_size % rep:
        raise ValueError(f'replication factor {rep} must divide the world size {world_size}')
    if rep > 1 and world_size // (rep * rep) < 1:
        raise ValueError(f'1.5D needs world_size >= rep^2 (got {world_size}, rep {rep})')


def row_groups(world_size, rep):
    """Replication groups: consecutive `rep` ranks share one row block."""
    return [list(range(i, i + rep)) for i in range(0, world_size, rep)]


def col_groups(world_size, rep):
    """Broadcast groups: ranks with the same replica index, one per row block."""
    return [list(range(j, world_size, rep)) for j in range(rep)]


def data_rank(rank, rep):
    """Row block a rank works on, and how many row blocks exist is world_size // rep."""
    return rank // rep


def stages_1d(world_size):
    return [Stage(s, s, s) for s in range(world_size)]


def stages_15d(rank, world_size, rep):
    check_layout(world_size, rep)
    replica = rank % rep
    basic = world_size // (rep * rep)
    count = basic if replica != rep - 1 else world_size // rep - (rep - 1) * basic
    return [Stage(replica * basic + i, (replica * basic + i) * rep + replica, replica * basic + i) for i in range(count)]


def stages(rank, world_size, rep=1):
    return stages_1d(world_size) if rep == 1 else stages_15d(rank, world_size, rep)


def pull_order(stage_list, me, size):
    """Order in which a rank of a `size`-rank communicator handles its stages when remote blocks are pulled from their
    owners (stage order 'peer_copy'): (own, remote) index lists into stage_list - the stages this rank roots itself, then
    the remote ones sorted by the distance of their root after this rank, so that in step j of a 1D loop every rank reads
    from rank me + j and no owner serves two readers at once."""
    own = [i for i, st in enumerate(stage_list) if st.root_in_group == me]
    remote = [i for i, st in enumerate(stage_list) if st.root_in_group != me]
    remote.sort(key=lambda i: ((stage_list[i].root_in_group - me) % size, i))
    return own, remote


def pack_layout(sizes, owner):
    """Where every reader's rows start inside `owner`'s send buffer in the 'peer_compact' stage order.  sizes[q][s] is the
    number of rows of block s that reader q's sparse block touches (0 for q == s: a rank reads its own block in place).
    Returns (offsets, total): offsets[q] = first row of reader q's list, lists laid out in ascending reader order."""
    offsets, total = [], 0
    for q in range(len(sizes)):
        offsets.append(total)
        if q != owner:
            total += int(sizes[q][owner])
    return offsets, total


def compact_layout(gathered, me, remote_roots):
    """Bookkeeping of the 'peer_compact' stage order for rank `me`, from the lists every rank asked for.
    gathered[q][s]   the ascending row ids of block s that reader q needs (absent or empty: nothing)
    remote_roots     the roots of this rank's remote stages, in the order it pulls them
    Returns a dict:  sizes (sizes[q][s]), packs [(reader q, first row of q's list inside this rank's send buffer)],
    stage_offsets / stage_rows per remote stage (where this rank's list starts inside the root's send buffer, its
    length), area_offsets / area_rows (where the pulled lists land on this rank, side by side in pull order) and
    send_rows (rows of the largest send buffer over all ranks: every rank allocates that much)."""
    size = len(gathered)
    sizes = [[len(gathered[q].get(s, ())) if q != s else 0 for s in range(size)] for q in range(size)]
    layouts = [pack_layout(sizes, s) for s in range(size)]
    packs = [(q, layouts[me][0][q]) for q in range(size) if q != me and sizes[q][me] > 0]
    stage_rows = [sizes[me][r] for r in remote_roots]
    area_offsets, total = [], 0
    for rows in stage_rows:
        area_offsets.append(total)
        total += rows
    return dict(sizes=sizes, packs=packs, stage_offsets=[layouts[r][0][me] for r in remote_roots], stage_rows=stage_rows,
                area_offsets=area_offsets, area_rows=total, send_rows=max(max(t for _, t in layouts), 1))


def join_packed_blocks(blocks, area_offsets, first, count):
    """The sparse block of ONE product that multiplies `count` consecutive arrivals of the compact peer loops.
    blocks[j] = (row ids, packed column ids, values, rows of the packed operand) of arrival j (torch tensors; the
    column ids are positions in that arrival's own list); area_offsets[j] = first row of arrival j in the landing area.
    Returns (row, col, val, operand rows): column ids re-based to the group's slice of the area (arrival `first` starts
    at 0), entries in row-major order and, inside a row, ascending (arrival, column) - the order a stage-by-stage loop
    would add them in."""
    import torch
    members = range(first, first + count)
    base = area_offsets[first]
    total = sum(blocks[j][3] for j in members)
    if count == 1:
        row, col, val, _ = blocks[first]
        return row, col, val, total
    row = torch.cat([blocks[j][0] for j in members])
    col = torch.cat([blocks[j][1] + (area_offsets[j] - base) for j in members])
    val = torch.cat([blocks[j][2] for j in members])
    order = torch.sort(row * total + col).indices
    return row[order], col[order], val[order], total


def default_stage_group(stage_order, rep, n_stages):
    """Stages (or arrivals) per product when the caller does not say.
    'reference', 1D: two products per distributed SpMM (half of the stages each): longer rows per product and one
        read-modify-write of the result instead of P-1, while the second half travels under the first.
    'peer_compact' / 'peer_gather', 1D, 8 ranks or more: one product per arrival, the last two arrivals joined
        (1,1,1,1,1,2 at 8 ranks).  By then the products run behind the transfers, so the joined block does not wait, and
        a pass over the result is saved: 15.7 ms per epoch on the benchmark graph with 0.77 of the transfer hidden at
        width 256, against 16.2 ms / 0.79 (all single), 15.5-15.7 ms / 0.70 (1,1,1,2,2), 15.8 ms / 0.54-0.61 (1,1,1,1,3 and
        1,1,2,3), 16.6 ms / 0.38 (4,2,1): joining more keeps shaving product time but exposes the transfer.  With fewer
        ranks the products dominate and waiting for a joined arrival costs what the join saves (4 ranks: 22.5 / 23.3 /
        25.2 ms for 1 / 2,1 / 3).
    Everything else: stage by stage."""
    if stage_order == 'reference' and rep == 1:
        return max(1, (n_stages + 1) // 2)
    if stage_order in ('peer_compact', 'peer_gather') and rep == 1 and n_stages >= 8:
        return tuple([1] * (n_stages - 1 - 2) + [2])
    return 1

"""A check of the distributed product that shares nothing with the code it checks.

``sampled_rows_check`` runs  z = sum_s A[rank, s] X_s  through the model's own stage loop (models.gcn.broadcast, whatever
schedule the environment selects) on seeded operand blocks, gathers all operand blocks with torch.distributed, and
recomputes a sample of rows of this rank's block of A - the longest row among them - in float64 with plain index
arithmetic on the row block's COO entries.  It pins what light_dist_gnn/models/gcn.py:16-30 computes (1.5D:
1D_CAGNET/dist_15d.py:61-106) for the graph and the schedule actually in use, on any number of ranks, and needs neither
the CPU oracle nor a second implementation of the kernels.  bench.py and spmm_sweep.py print its result.
"""
import torch

TOLERANCE = 1e-5
ROWS = 384


def sampled_rows_check(env, row_block, adj_parts, widths, rows=ROWS):
    """row_block: this rank's n x (n * blocks) coalesced COO block of A; adj_parts: its column blocks (what the stage
    loop multiplies).  Collective: every rank of the environment calls it.  Returns a dict with the worst relative
    errors over ranks and widths (max-abs and Frobenius, both relative to the exact rows) and `ok`."""
    from models.gcn import broadcast
    dev, n = env.device, row_block.size(0)
    idx, val = row_block.indices(), row_block.values()
    row = idx[0].contiguous()
    gen = torch.Generator(device='cpu').manual_seed(977 + env.rank // env.rep)
    counts = torch.bincount(row, minlength=n)
    sample = torch.cat((torch.randperm(n, generator=gen)[:max(rows - 1, 0)].to(dev), counts.argmax().view(1))).unique()
    lo = torch.searchsorted(row, sample)
    hi = torch.searchsorted(row, sample, right=True)
    lengths = hi - lo
    slot = torch.repeat_interleave(torch.arange(sample.numel(), device=dev), lengths)        # entry -> sampled row
    offsets = torch.arange(int(lengths.sum()), device=dev) - torch.repeat_interleave(lengths.cumsum(0) - lengths, lengths)
    entries = torch.repeat_interleave(lo, lengths) + offsets
    cols, vals = idx[1][entries], val[entries].double()
    worst = {'max_rel': 0.0, 'fro_rel': 0.0}
    for width in widths:
        x = torch.randn(n, width, generator=torch.Generator(device='cpu').manual_seed(31 * width + env.rank // env.rep)).to(dev)
        z = broadcast(adj_parts, x, f'selfcheck{width}')
        x_all = env.all_gather_then_cat(x) if env.world_size > 1 else x
        want = torch.zeros(sample.numel(), width, dtype=torch.float64, device=dev)
        for c0 in range(0, entries.numel(), 1 << 20):                                        # bounded temporaries
            sl = slice(c0, c0 + (1 << 20))
            want.index_add_(0, slot[sl], vals[sl, None] * x_all[cols[sl]].double())
        got = z[sample].double()
        worst['max_rel'] = max(worst['max_rel'], float((got - want).abs().max() / want.abs().max().clamp(min=1e-30)))
        worst['fro_rel'] = max(worst['fro_rel'], float((got - want).norm() / want.norm().clamp(min=1e-30)))
        del x, z, x_all
    every = env.all_gather_object(worst) if env.world_size > 1 else [worst]
    out = {'max_rel': max(w['max_rel'] for w in every), 'fro_rel': max(w['fro_rel'] for w in every),
           'rows': int(sample.numel()) * env.world_size, 'widths': list(widths), 'tolerance': TOLERANCE,
           'against': "float64 evaluation of sampled rows of every rank's row block on operands gathered with torch.distributed",
           'schedule': env.stage_order, 'stage_group': env.stage_group}
    out['ok'] = bool(out['max_rel'] <= TOLERANCE and out['fro_rel'] <= TOLERANCE)
    return out

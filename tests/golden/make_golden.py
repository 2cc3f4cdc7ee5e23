"""Generates the golden fixtures in this folder by running the REFERENCE code itself.

Run in the build container only (the reference tree does not exist anywhere else):

    python tests/golden/make_golden.py --reference /path/to/reference

The reference's light_dist_gnn/ is copied to a temporary folder (it writes data/ and logs beside
itself), imported from there unmodified, and driven through its own public functions:

  spmm_cases.npz   C.addmm_(A, B) - the CPU call of light_dist_gnn/models/gcn.py:13 - on small adversarial blocks
  graph_small.npz  graph_utils.preprocess / sym_normalization, COO_Graph.partition, Parted_COO_Graph at P=2 and 3
  gcn_small.npz    models.gcn.broadcast, DistGCNLayer and the shipped 3-layer GCN trained as dist_train.train
                   does, on 2 gloo ranks
  plumbing.npz     the 10,000-node / 2-layer / Glorot configuration on 2 gloo ranks, stored as digests

Shims applied from outside the reference files: torch.cuda.synchronize becomes a no-op in the
workers (light_dist_gnn/dist_utils/timer.py:17 calls it with no driver present), and
sym_normalization is called with faster_device='cpu' (graph_utils.py:24 defaults to cuda:0).

Inputs come from the product's synthetic generator (loaded by file path, its integer streams are
restated independently in oracle/ref_graph.py); small inputs are stored in the fixture, the larger
one is stored as a SHA-256 so a test can prove it regenerated the same bytes.
"""
import argparse
import functools
import hashlib
import importlib.util
import os
import shutil
import sys
import tempfile

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))


def load_synthetic():
    spec = importlib.util.spec_from_file_location('dg_synthetic', os.path.join(ROOT, 'dist-gnn_b200', 'coo_graph', 'synthetic.py'))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def sha(*arrays):
    h = hashlib.sha256()
    for a in arrays:
        h.update(np.ascontiguousarray(a).tobytes())
    return h.hexdigest()


def import_reference(ref_root):
    work = tempfile.mkdtemp(prefix='ref_ldg_')
    dst = os.path.join(work, 'light_dist_gnn')
    shutil.copytree(os.path.join(ref_root, 'light_dist_gnn'), dst)
    sys.path.insert(0, dst)
    return dst


# --------------------------------------------------------------------------------------------- spmm cases
def spmm_cases():
    rng = np.random.Generator(np.random.PCG64(7))
    out, names = {}, []

    def add(name, m, k, F, rows, cols, alpha=1.0, beta=1.0):
        rows, cols = np.asarray(rows, dtype=np.int64), np.asarray(cols, dtype=np.int64)
        vals = rng.standard_normal(rows.size, dtype=np.float32)
        A = torch.sparse_coo_tensor(torch.from_numpy(np.stack((rows, cols))), torch.from_numpy(vals), (m, k)).coalesce()
        B = rng.standard_normal((k, F), dtype=np.float32)
        C0 = rng.standard_normal((m, F), dtype=np.float32)
        C = torch.from_numpy(C0.copy())
        if alpha == 1.0 and beta == 1.0:
            C.addmm_(A, torch.from_numpy(B))                      # the reference's exact call
        else:
            C.addmm_(A, torch.from_numpy(B), beta=beta, alpha=alpha)
        idx = A.indices().numpy()
        for key, v in dict(row=idx[0].astype(np.int32), col=idx[1].astype(np.int32), val=A.values().numpy(),
                           dims=np.array([m, k, F], dtype=np.int64), ab=np.array([alpha, beta], dtype=np.float32),
                           B=B, C0=C0, C=C.numpy()).items():
            out[f'{name}/{key}'] = v
        names.append(name)

    def rand_pairs(m, k, nnz):
        flat = rng.choice(m * k, size=nnz, replace=False)
        return flat // k, flat % k

    add('empty', 5, 4, 3, [], [])
    add('one_entry', 1, 1, 1, [0], [0])
    r, c = rand_pairs(64, 48, 300)
    for F in (1, 3, 41, 47, 100, 256):
        add(f'rand_F{F}', 64, 48, F, r, c)
    add('alpha_beta', 64, 48, 20, r, c, alpha=0.5, beta=-2.0)
    add('beta_zero', 64, 48, 20, r, c, alpha=1.5, beta=0.0)
    # rows 0..9 empty, row 10 very heavy, the rest light
    hr = np.concatenate((np.full(1200, 10), rng.integers(11, 40, 200)))
    hc = np.concatenate((rng.choice(1500, 1200, replace=False), rng.integers(0, 1500, 200)))
    add('heavy_row', 40, 1500, 47, hr, hc)
    hr = np.concatenate((np.full(500, 3), rng.integers(4, 20, 100)))
    hc = np.concatenate((rng.choice(600, 500, replace=False), rng.integers(0, 600, 100)))
    add('heavy_row_F128', 20, 600, 128, hr, hc)
    r, c = rand_pairs(64, 48, 500)
    add('rand_F602', 64, 48, 602, r, c)
    add('last_rows_empty', 50, 30, 8, [0, 0, 3], [1, 29, 2])
    out['names'] = np.array(names)
    return out


# --------------------------------------------------------------------------------------------- graph fixtures
def small_dataset(syn, n=1000, edges=20000, F=32, classes=7, seed=1):
    return syn.make_dataset(num_nodes=n, directed_edges=edges, feat_dim=F, num_classes=classes,
                            split=(0.6, 0.2, 0.2), seed=seed)


def write_reference_dataset(name, d):
    from coo_graph import datasets
    datasets.save_dataset(d['edge_index'], d['features'], d['labels'], d['train_mask'], d['val_mask'], d['test_mask'],
                          d['num_nodes'], d['num_edges'], d['num_classes'], name)


def reference_full_graph(name):
    """COO_Graph(name) with normalisation forced onto the CPU."""
    import coo_graph.graph_utils as gu
    from coo_graph import COO_Graph
    if not getattr(gu.sym_normalization, '_cpu_shim', False):
        shim = functools.partial(gu.sym_normalization, faster_device='cpu')
        shim._cpu_shim = True
        gu.sym_normalization = shim
    return COO_Graph(name, full_graph_cache_enabled=False)


def graph_fixture(syn):
    from coo_graph import Parted_COO_Graph
    d = small_dataset(syn)
    write_reference_dataset('gsmall', d)
    g = reference_full_graph('gsmall')
    out = {'in/edge_index': d['edge_index'].numpy(), 'in/features': d['features'].numpy(), 'in/labels': d['labels'].numpy(),
           'in/masks': torch.stack((d['train_mask'], d['val_mask'], d['test_mask'])).numpy(),
           'in/meta': np.array([d['num_nodes'], d['num_edges'], d['num_classes']], dtype=np.int64),
           'full/adj_idx': g.adj.indices().numpy(), 'full/adj_val': g.adj.values().numpy(), 'full/features': g.features.numpy()}
    for P in (2, 3):
        g.partition(P)
        for r in range(P):
            pg = Parted_COO_Graph('gsmall', r, P)
            pre = f'P{P}/r{r}/'
            out[pre + 'adj_idx'], out[pre + 'adj_val'] = pg.adj.indices().numpy(), pg.adj.values().numpy()
            out[pre + 'adj_shape'] = np.array(pg.adj.shape, dtype=np.int64)
            out[pre + 'features'] = pg.features.numpy()
            out[pre + 'labels'], out[pre + 'train_mask'] = pg.labels.numpy(), pg.train_mask.numpy()
            out[pre + 'local_labels'], out[pre + 'local_train_mask'] = pg.local_labels.numpy(), pg.local_train_mask.numpy()
            out[pre + 'parts_nnz'] = np.array([p.values().numel() for p in pg.adj_parts], dtype=np.int64)
            out[pre + 'parts_idx'] = np.concatenate([p.indices().numpy() for p in pg.adj_parts], axis=1)
            out[pre + 'parts_val'] = np.concatenate([p.values().numpy() for p in pg.adj_parts])
            out[pre + 'parts_shape'] = np.array([list(p.shape) for p in pg.adj_parts], dtype=np.int64)
    return out


# --------------------------------------------------------------------------------------------- gloo workers
def _worker(rank, world, dataset, mode, weights, epochs, port, q):
    os.environ.update(MASTER_ADDR='127.0.0.1', MASTER_PORT=str(port))
    torch.cuda.synchronize = lambda *a, **k: None
    torch.set_num_threads(2)
    import dist_utils
    import models.gcn as ref_gcn
    from coo_graph import Parted_COO_Graph
    import torch.nn.functional as F
    env = dist_utils.DistEnv(rank, world, 'gloo')
    g = Parted_COO_Graph(dataset, rank, world, device=env.device)
    rec = {}
    calls = []
    inner = ref_gcn.broadcast

    def spy(adj_parts, feat, tag):
        z = inner(adj_parts, feat, tag)
        calls.append((tag, z.detach().clone()))
        return z
    ref_gcn.broadcast = spy

    if mode == 'shipped':            # the shipped 3-layer model, trained as dist_train.train does (dist_train.py:26-46)
        model = ref_gcn.GCN(g, env, hidden_dim=16)
        params = [model.weight1, model.weight2, model.weight3]
        forward = lambda: model(g.features)
    else:                            # the reference layer with injected weights (2-layer Glorot configuration)
        params = [torch.nn.Parameter(w.clone()) for w in weights]

        def forward():
            h = g.features
            for l, w in enumerate(params):
                h = ref_gcn.DistGCNLayer.apply(h, w, g.adj_parts, f'L{l + 1}')
                if l < len(params) - 1:
                    h = F.relu(h)
            return h
    rec['w0'] = [p.detach().clone() for p in params]
    opt = torch.optim.Adam(params, lr=0.01)
    loss_func = torch.nn.CrossEntropyLoss()
    losses = []
    for epoch in range(epochs):
        calls.clear()
        outputs = forward()
        opt.zero_grad()
        if g.local_labels[g.local_train_mask].size(0) > 0:
            loss = loss_func(outputs[g.local_train_mask], g.local_labels[g.local_train_mask])
        else:
            loss = (outputs * 0).sum()
        loss.backward()
        if epoch == 0:
            rec['outputs'] = outputs.detach().clone()
            rec['bcast'] = [(t, z) for t, z in calls]
            rec['dw'] = [p.grad.detach().clone() for p in params]
        opt.step()
        losses.append(float(loss.item()))
    rec['losses'] = losses
    rec['w_final'] = [p.detach().clone() for p in params]
    env.barrier_all()
    q.put((rank, {k: ([(t, z.numpy()) for t, z in v] if k == 'bcast' else
                      [x.numpy() for x in v] if isinstance(v, list) and k != 'losses' else
                      v.numpy() if torch.is_tensor(v) else v) for k, v in rec.items()}))


def run_reference_training(dataset, world, mode, weights, epochs, port):
    import torch.multiprocessing as mp
    store = os.path.join(tempfile.gettempdir(), 'torch-dist')
    if os.path.exists(store):
        os.remove(store)
    ctx = mp.get_context('spawn')
    q = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, world, dataset, mode, weights, epochs, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    got = dict(q.get(timeout=600) for _ in range(world))
    for p in procs:
        p.join()
    return [got[r] for r in range(world)]


def gcn_small_fixture():
    out = {}
    res = run_reference_training('gsmall', 2, 'shipped', None, 3, 29611)
    for r, rec in enumerate(res):
        pre = f'r{r}/'
        out[pre + 'losses'] = np.array(rec['losses'], dtype=np.float64)
        out[pre + 'outputs'] = rec['outputs']
        for i, w in enumerate(rec['w0']):
            out[pre + f'w0_{i}'] = w
        for i, w in enumerate(rec['w_final']):
            out[pre + f'wfinal_{i}'] = w
        for i, w in enumerate(rec['dw']):
            out[pre + f'dw_{i}'] = w
        out[pre + 'bcast_tags'] = np.array([t for t, _ in rec['bcast']])
        for i, (_, z) in enumerate(rec['bcast']):
            out[pre + f'bcast_{i}'] = z
    return out


def digest(a, rows):
    a = np.asarray(a)
    return dict(rows=a[rows], colsum=a.astype(np.float64).sum(axis=0), fro=np.array(np.sqrt((a.astype(np.float64) ** 2).sum())),
                absmax=np.array(np.abs(a).max()))


def plumbing_fixture(syn):
    cfg = syn.CONFIGS['plumbing']
    d = syn.make_dataset(seed=0, **cfg)
    write_reference_dataset('plumbing', d)
    g = reference_full_graph('plumbing')
    g.partition(2)
    dims = [cfg['feat_dim']] + [cfg['hidden']] * (cfg['layers'] - 1) + [cfg['num_classes']]
    weights = syn.glorot_weights(dims, seed=0)
    res = run_reference_training('plumbing', 2, 'injected', weights, 3, 29613)
    n = res[0]['outputs'].shape[0]
    rows = np.sort(np.random.Generator(np.random.PCG64(3)).choice(n, 48, replace=False))
    out = {'sample_rows': rows,
           'in/sha_edge_index': np.array(sha(d['edge_index'].numpy())),
           'in/sha_features': np.array(sha(d['features'].numpy())),
           'in/sha_labels_masks': np.array(sha(d['labels'].numpy(), d['train_mask'].numpy(), d['val_mask'].numpy(), d['test_mask'].numpy())),
           'in/sha_weights': np.array(sha(*[w.numpy() for w in weights])),
           'full/adj_nnz': np.array(g.adj.values().numel()),
           'full/sha_adj_idx': np.array(sha(g.adj.indices().numpy())),
           'full/adj_val_sum': np.array(g.adj.values().double().sum().item())}
    for r, rec in enumerate(res):
        pre = f'r{r}/'
        out[pre + 'losses'] = np.array(rec['losses'], dtype=np.float64)
        for k, v in digest(rec['outputs'], rows).items():
            out[pre + 'outputs/' + k] = v
        out[pre + 'bcast_tags'] = np.array([t for t, _ in rec['bcast']])
        for i, (_, z) in enumerate(rec['bcast']):
            for k, v in digest(z, rows).items():
                out[pre + f'bcast_{i}/' + k] = v
        for i, w in enumerate(rec['dw']):
            out[pre + f'dw_{i}'] = w
        for i, w in enumerate(rec['w_final']):
            for k, v in digest(w, np.arange(min(4, w.shape[0]))).items():
                out[pre + f'wfinal_{i}/' + k] = v
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument('--reference', required=True, help='root of the reference checkout (holds light_dist_gnn/)')
    args = ap.parse_args()
    syn = load_synthetic()
    import_reference(args.reference)
    np.savez_compressed(os.path.join(HERE, 'spmm_cases.npz'), **spmm_cases())
    np.savez_compressed(os.path.join(HERE, 'graph_small.npz'), **graph_fixture(syn))
    np.savez_compressed(os.path.join(HERE, 'gcn_small.npz'), **gcn_small_fixture())
    np.savez_compressed(os.path.join(HERE, 'plumbing.npz'), **plumbing_fixture(syn))
    for f in sorted(os.listdir(HERE)):
        if f.endswith('.npz'):
            print(f, os.path.getsize(os.path.join(HERE, f)), 'bytes')


if __name__ == '__main__':
    main()

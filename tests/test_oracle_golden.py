"""The CPU oracle against outputs of the reference code itself (tests/golden/*.npz)."""
import hashlib

import numpy as np
import pytest

from conftest import assert_close
from oracle import ref_gcn, ref_graph

TOL = 1e-5   # fp32 parity tolerance of the path: max-abs and Frobenius relative error


def _case(z, name):
    g = lambda k: z[f'{name}/{k}']
    m, k, F = (int(v) for v in g('dims'))
    return ref_graph.Coo(g('row').astype(np.int64), g('col').astype(np.int64), g('val'), (m, k)), g('B'), g('C0'), g('C'), g('ab')


def test_spmm_oracle_matches_reference_addmm(golden):
    z = golden('spmm_cases')
    for name in z['names']:
        A, B, C0, C, (alpha, beta) = _case(z, name)
        got = ref_gcn.spmm_coo(A, np.ascontiguousarray(B), C0.copy(), float(alpha), float(beta))
        assert_close(got, C, TOL, name)


def test_spmm_oracle_thread_count_does_not_change_bits(golden):
    z = golden('spmm_cases')
    A, B, C0, _, _ = _case(z, 'heavy_row')
    one = ref_gcn.spmm_coo(A, B, C0.copy(), threads=1)
    four = ref_gcn.spmm_coo(A, B, C0.copy(), threads=4)
    assert np.array_equal(one, four)


def test_generator_restatement_matches_fixture_inputs(golden):
    z = golden('graph_small')
    n, e, c = (int(v) for v in z['in/meta'])
    ei = ref_graph.rmat_edge_index(n, e, seed=1)
    assert np.array_equal(ei.astype(np.int32), z['in/edge_index'])
    assert np.array_equal(ref_graph.uniform_labels(n, c, 1).astype(np.int8), z['in/labels'])
    assert np.array_equal(ref_graph.random_split(n, (0.6, 0.2, 0.2), 1), z['in/masks'])


def test_normalisation_matches_reference(golden):
    z = golden('graph_small')
    n = int(z['in/meta'][0])
    A = ref_graph.sym_normalization(z['in/edge_index'], n)
    assert np.array_equal(np.stack((A.row, A.col)), z['full/adj_idx'])       # indices bit-exact
    assert_close(A.val, z['full/adj_val'], 1e-6, 'adj values')
    assert_close(ref_graph.preprocess_features(z['in/features']), z['full/features'], 1e-6, 'features')


def test_duplicate_edges_add_up_and_old_self_loops_go():
    ei = np.array([[0, 0, 1, 2, 2], [1, 1, 0, 2, 0]])      # (0,1) twice, a self loop at 2
    A = ref_graph.sym_normalization(ei, 3)
    dense = A.dense()
    deg = np.array([1 + 1 + 1, 2 + 1, 1.0])                # column sums of A+I with multiplicity
    want = np.array([[1, 2, 0], [1, 1, 0], [1, 0, 1]], dtype=np.float64) / np.sqrt(np.outer(deg, deg))
    assert np.allclose(dense, want, rtol=1e-6)


@pytest.mark.parametrize('P', [2, 3])
def test_partition_matches_reference(golden, P):
    z = golden('graph_small')
    n = int(z['in/meta'][0])
    A = ref_graph.Coo(z['full/adj_idx'][0], z['full/adj_idx'][1], z['full/adj_val'], (n, n))
    parts = ref_graph.partition(A, z['full/features'], z['in/labels'].astype(np.int64), z['in/masks'], P)
    for r, part in enumerate(parts):
        pre = f'P{P}/r{r}/'
        pg = ref_graph.parted_graph(part)
        assert tuple(z[pre + 'adj_shape']) == part['adj'].shape
        assert np.array_equal(np.stack((part['adj'].row, part['adj'].col)), z[pre + 'adj_idx'])
        assert np.array_equal(part['adj'].val, z[pre + 'adj_val'])
        assert np.array_equal(part['features'], z[pre + 'features'])
        assert np.array_equal(part['labels'], z[pre + 'labels'])
        assert np.array_equal(part['masks'][0], z[pre + 'train_mask'])
        assert np.array_equal(pg['local_labels'], z[pre + 'local_labels'])
        assert np.array_equal(pg['local_train_mask'], z[pre + 'local_train_mask'])
        assert np.array_equal([p.nnz for p in pg['adj_parts']], z[pre + 'parts_nnz'])
        assert np.array_equal(np.concatenate([np.stack((p.row, p.col)) for p in pg['adj_parts']], axis=1), z[pre + 'parts_idx'])
        assert np.array_equal(np.concatenate([p.val for p in pg['adj_parts']]), z[pre + 'parts_val'])
        assert np.array_equal([list(p.shape) for p in pg['adj_parts']], z[pre + 'parts_shape'])


def _parted_from_fixture(z, P):
    n = int(z['in/meta'][0])
    A = ref_graph.Coo(z['full/adj_idx'][0], z['full/adj_idx'][1], z['full/adj_val'], (n, n))
    parts = ref_graph.partition(A, z['full/features'], z['in/labels'].astype(np.int64), z['in/masks'], P)
    return [ref_graph.parted_graph(p) for p in parts]


def test_gcn_oracle_matches_reference_training_over_gloo(golden):
    """Shipped 3-layer model, 2 gloo ranks, 3 epochs: every broadcast-SpMM result of epoch 0 (3 forward,
    3 backward), outputs, dW after the all-reduce, losses and the weights after 3 Adam steps."""
    z, t = golden('graph_small'), golden('gcn_small')
    parted = _parted_from_fixture(z, 2)
    weights = [t[f'r0/w0_{i}'] for i in range(3)]
    model = ref_gcn.gcn_1d(parted, weights)
    feats = [p['features'] for p in parted]
    labels = [p['local_labels'] for p in parted]
    masks = [p['local_train_mask'] for p in parted]
    for epoch in range(3):
        losses, outputs, trace, btrace = model.epoch(feats, labels, masks)
        for r in range(2):
            assert abs(losses[r] - t[f'r{r}/losses'][epoch]) <= 2e-5 * max(1.0, abs(t[f'r{r}/losses'][epoch])), (epoch, r)
        if epoch == 0:
            for r in range(2):
                tags = list(t[f'r{r}/bcast_tags'])
                assert tags == ['ForwardL1', 'ForwardL2', 'ForwardL3', 'BackwardL3', 'BackwardL2', 'BackwardL1']
                got = [trace[l]['z'][r] for l in range(3)] + [btrace[l]['ag'][r] for l in (2, 1, 0)]
                for i, g in enumerate(got):
                    assert_close(g, t[f'r{r}/bcast_{i}'], TOL, f'rank {r} {tags[i]}')
                assert_close(outputs[r], t[f'r{r}/outputs'], TOL, f'outputs r{r}')
                for l in range(3):
                    assert_close(btrace[l]['dw'][r], t[f'r{r}/dw_{l}'], TOL, f'dW{l} r{r}')
    for l in range(3):
        assert_close(model.weights[l], t[f'r0/wfinal_{l}'], 1e-4, f'weights after 3 steps, layer {l}')


def test_plumbing_config_oracle_matches_reference_digests(golden):
    """10,000-node / 2-layer / Glorot configuration on 2 ranks: inputs regenerated from the seed must
    hash to the stored SHA-256, then every stage-loop result matches the reference's digests."""
    import torch
    from coo_graph import synthetic
    t = golden('plumbing')
    cfg = synthetic.CONFIGS['plumbing']
    d = synthetic.make_dataset(seed=0, **cfg)
    sha = lambda *a: hashlib.sha256(b''.join(np.ascontiguousarray(x).tobytes() for x in a)).hexdigest()
    assert sha(d['edge_index'].numpy()) == str(t['in/sha_edge_index'])
    assert sha(d['features'].numpy()) == str(t['in/sha_features'])
    dims = [cfg['feat_dim'], cfg['hidden'], cfg['num_classes']]
    weights = [w.numpy() for w in synthetic.glorot_weights(dims, seed=0)]
    assert sha(*weights) == str(t['in/sha_weights'])
    n = cfg['num_nodes']
    # vectorised normalisation for this size: no duplicates by construction, so coalesce is a sort
    ei = ref_graph.add_self_loops(d['edge_index'].numpy().astype(np.int64), n)
    A0 = ref_graph.fast_coalesce_sorted(ei[0], ei[1], np.ones(ei.shape[1], dtype=np.float32), (n, n))
    deg = np.bincount(A0.col, minlength=n).astype(np.float32)
    dr = np.power(deg, np.float32(-0.5), dtype=np.float32)
    A = ref_graph.Coo(A0.row, A0.col, ((dr[A0.row] * A0.val) * dr[A0.col]).astype(np.float32), (n, n))
    assert A.nnz == int(t['full/adj_nnz'])
    assert sha(np.stack((A.row, A.col))) == str(t['full/sha_adj_idx'])
    assert abs(A.val.astype(np.float64).sum() - float(t['full/adj_val_sum'])) < 1e-3
    feats = ref_graph.preprocess_features(d['features'].numpy())
    masks = torch.stack((d['train_mask'], d['val_mask'], d['test_mask'])).numpy()
    parts = [ref_graph.parted_graph(p) for p in ref_graph.partition(A, feats, d['labels'].numpy().astype(np.int64), masks, 2)]
    model = ref_gcn.gcn_1d(parts, weights)
    rows = t['sample_rows']
    for epoch in range(3):
        losses, outputs, trace, btrace = model.epoch([p['features'] for p in parts], [p['local_labels'] for p in parts],
                                                     [p['local_train_mask'] for p in parts])
        for r in range(2):
            assert abs(losses[r] - t[f'r{r}/losses'][epoch]) <= 2e-5 * max(1.0, abs(t[f'r{r}/losses'][epoch]))
        if epoch == 0:
            for r in range(2):
                got = [trace[0]['z'][r], trace[1]['z'][r], btrace[1]['ag'][r], btrace[0]['ag'][r]]
                for i, g in enumerate(got):
                    scale = float(t[f'r{r}/bcast_{i}/absmax'])
                    assert np.abs(g[rows] - t[f'r{r}/bcast_{i}/rows']).max() <= TOL * scale
                    assert np.abs(g.astype(np.float64).sum(0) - t[f'r{r}/bcast_{i}/colsum']).max() <= 1e-4 * scale * np.sqrt(g.shape[0])
                    assert abs(np.sqrt((g.astype(np.float64) ** 2).sum()) - float(t[f'r{r}/bcast_{i}/fro'])) <= TOL * float(t[f'r{r}/bcast_{i}/fro'])
                for l in range(2):
                    assert_close(btrace[l]['dw'][r], t[f'r{r}/dw_{l}'], TOL, f'dW{l}')

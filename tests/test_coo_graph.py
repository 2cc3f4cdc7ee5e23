"""The product's graph preparation (coo_graph/) against the reference's outputs and the oracle: bit-exact indices."""
import os

import numpy as np
import pytest
import torch

from conftest import assert_close
from oracle import ref_graph
from coo_graph import COO_Graph, Parted_COO_Graph, datasets, graph_utils, synthetic


def _dataset_from_fixture(z):
    n, e, c = (int(v) for v in z['in/meta'])
    m = torch.from_numpy(z['in/masks'])
    return dict(edge_index=torch.from_numpy(z['in/edge_index']), features=torch.from_numpy(z['in/features']),
                labels=torch.from_numpy(z['in/labels']), train_mask=m[0], val_mask=m[1], test_mask=m[2],
                num_nodes=n, num_edges=e, num_classes=c)


def test_generator_is_the_fixture_generator(golden):
    z = golden('graph_small')
    d = synthetic.make_dataset(num_nodes=1000, directed_edges=20000, feat_dim=32, num_classes=7, split=(0.6, 0.2, 0.2), seed=1)
    assert np.array_equal(d['edge_index'].numpy(), z['in/edge_index'])
    assert np.array_equal(d['features'].numpy(), z['in/features'])
    assert np.array_equal(d['labels'].numpy(), z['in/labels'])


def test_generated_graph_is_symmetric_loop_free_and_distinct():
    ei = synthetic.rmat_edge_index(5000, 60000, seed=3)
    assert ei.shape == (2, 60000)
    keys = ei[0] * 5000 + ei[1]
    assert keys.unique().numel() == 60000 and bool((ei[0] != ei[1]).all())
    assert torch.equal(torch.sort(keys).values, torch.sort(ei[1] * 5000 + ei[0]).values)
    # prefix property: a smaller target is the set of earliest distinct draws of a larger one
    lo_s, hi_s = synthetic.rmat_undirected(5000, 20000, seed=3)
    lo_l, hi_l = synthetic.rmat_undirected(5000, 60000, seed=3)
    assert set(zip(lo_s.tolist(), hi_s.tolist())) <= set(zip(lo_l.tolist(), hi_l.tolist()))


def test_normalisation_matches_reference(golden):
    z = golden('graph_small')
    A = graph_utils.sym_normalization(torch.from_numpy(z['in/edge_index']), 1000)
    assert A.is_coalesced()
    assert np.array_equal(A.indices().numpy(), z['full/adj_idx'])
    assert_close(A.values().numpy(), z['full/adj_val'], 1e-6, 'adj values')


def test_normalisation_with_duplicates_matches_oracle():
    g = torch.Generator().manual_seed(5)
    ei = torch.randint(0, 50, (2, 600), generator=g)       # many duplicates and self loops
    got = graph_utils.sym_normalization(ei, 50)
    want = ref_graph.sym_normalization(ei.numpy(), 50)
    assert np.array_equal(got.indices().numpy(), np.stack((want.row, want.col)))
    assert_close(got.values().numpy(), want.val, 1e-6, 'values')


@pytest.mark.parametrize('P', [2, 3])
def test_partition_files_and_loader_match_reference(golden, P, tmp_path, monkeypatch):
    z = golden('graph_small')
    monkeypatch.setattr(datasets, 'data_root', str(tmp_path))
    datasets.save_dataset(name='gsmall', **_dataset_from_fixture(z))
    full = COO_Graph('gsmall')
    assert os.path.exists(tmp_path / 'gsmall_GCN_full.coo_graph')
    assert_close(full.features.numpy(), z['full/features'], 1e-6, 'features')
    full.partition(P)
    in_memory = COO_Graph.from_dict('gsmall', _dataset_from_fixture(z))
    for r in range(P):
        pre = f'P{P}/r{r}/'
        assert os.path.exists(tmp_path / f'gsmall_GCN_{P}_parts' / f'part_{r}_of_{P}.coo_graph')
        for pg in (Parted_COO_Graph('gsmall', r, P), Parted_COO_Graph.from_full(in_memory, r, P)):
            assert tuple(pg.adj.shape) == tuple(z[pre + 'adj_shape'])
            assert np.array_equal(pg.adj.indices().numpy(), z[pre + 'adj_idx'])
            assert_close(pg.adj.values().numpy(), z[pre + 'adj_val'], 1e-6, 'adj values')
            assert_close(pg.features.numpy(), z[pre + 'features'], 1e-6, 'features')
            assert pg.labels.dtype == torch.long and np.array_equal(pg.labels.numpy(), z[pre + 'labels'])
            assert np.array_equal(pg.train_mask.numpy(), z[pre + 'train_mask'])
            assert np.array_equal(pg.local_labels.numpy(), z[pre + 'local_labels'])
            assert np.array_equal(pg.local_train_mask.numpy(), z[pre + 'local_train_mask'])
            assert pg.local_num_nodes == z[pre + 'adj_shape'][0] and pg.local_num_edges == z[pre + 'adj_val'].size
            assert np.array_equal([p.values().numel() for p in pg.adj_parts], z[pre + 'parts_nnz'])
            assert all(p.is_coalesced() for p in pg.adj_parts)
            assert np.array_equal(np.concatenate([p.indices().numpy() for p in pg.adj_parts], axis=1), z[pre + 'parts_idx'])
            assert np.array_equal([list(p.shape) for p in pg.adj_parts], z[pre + 'parts_shape'])


def test_partition_refuses_block_counts_the_reference_cannot_fill(tmp_path, monkeypatch):
    # 9 nodes in 4 parts: blocks of 3 rows only fill 3 parts; the reference fails with IndexError too
    d = synthetic.make_dataset(num_nodes=9, directed_edges=16, feat_dim=4, num_classes=2, split=(0.6, 0.2, 0.2), seed=0)
    g = COO_Graph.from_dict('tiny', d)
    with pytest.raises(IndexError):
        g.part_dict(3, 4)


def test_missing_dataset_is_generated_or_refused(tmp_path, monkeypatch):
    monkeypatch.setattr(datasets, 'data_root', str(tmp_path))
    with pytest.raises(FileNotFoundError):
        datasets.load_dataset('reddit')
    d = datasets.load_dataset('rmat_plumbing')
    assert d['edge_index'].dtype == torch.int32 and d['labels'].dtype == torch.int8 and d['features'].shape == (10000, 128)
    assert d['num_edges'] == 200000

"""On-disk dataset dict, same keys, dtypes and file name as the reference
(light_dist_gnn/coo_graph/datasets.py:15-38): ``data/{name}.torch`` holding edge_index int32 [2,E],
features fp32 [N,d], labels int8, three bool masks and the three counts.

The reference fetches missing datasets from DGL / PyG / OGB (datasets.py:41-108); none of those
packages or the network exist here, so a missing file is built from the synthetic R-MAT generator
when the name is ``rmat_<config>[_seed<k>][_noperm]`` and is an error otherwise.
"""
import os
import re

import torch

from . import synthetic

data_root = os.environ.get('DIST_GNN_DATA_ROOT', os.path.join(os.path.dirname(__file__), '..', 'data'))


def _ensure_root():
    os.makedirs(data_root, exist_ok=True)


def dataset_path(name):
    return os.path.join(data_root, name + '.torch')


def save_dataset(edge_index, features, labels, train_mask, val_mask, test_mask, num_nodes, num_edges, num_classes, name):
    _ensure_root()
    if name.startswith('a_quarter'):  # the reference's quarter-size cut (datasets.py:16-27)
        keep_nodes = num_nodes // 4
        inside = (edge_index[0] < keep_nodes) & (edge_index[1] < keep_nodes)
        edge_index = edge_index[:, inside].clone()
        features, labels = features[:keep_nodes].clone(), labels[:keep_nodes].clone()
        train_mask, val_mask, test_mask = (m[:keep_nodes].clone() for m in (train_mask, val_mask, test_mask))
        num_nodes, num_edges = keep_nodes, edge_index.size(1)
    torch.save({'edge_index': edge_index.int(), 'features': features, 'labels': labels.char(),
                'train_mask': train_mask.bool(), 'val_mask': val_mask.bool(), 'test_mask': test_mask.bool(),
                'num_nodes': num_nodes, 'num_edges': num_edges, 'num_classes': num_classes}, dataset_path(name))


def prepare_dataset(name):
    m = re.fullmatch(r'rmat_([a-z0-9]+?)(?:_seed(\d+))?(_noperm)?', name)
    if not m or m.group(1) not in synthetic.CONFIGS:
        raise FileNotFoundError(
            f'dataset {name!r} is not on disk and cannot be downloaded here; '
            f'synthetic names are rmat_<{"|".join(synthetic.CONFIGS)}>[_seed<k>][_noperm]')
    cfg = synthetic.CONFIGS[m.group(1)]
    d = synthetic.make_dataset(seed=int(m.group(2) or 0), permute=m.group(3) is None, **cfg)
    save_dataset(name=name, **d)


def load_dataset(name):
    if not os.path.exists(dataset_path(name)):
        prepare_dataset(name)
    return torch.load(dataset_path(name))

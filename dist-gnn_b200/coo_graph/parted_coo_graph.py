"""Full and partitioned graph objects with the attributes, file names and file contents of the
reference's light_dist_gnn/coo_graph/parted_coo_graph.py.

``COO_Graph(name).partition(P)`` writes ``data/{name}_GCN_{P}_parts/part_{r}_of_{P}.coo_graph``;
``Parted_COO_Graph(name, r, P, device=...)`` loads one of them and column-splits the local row
block into the P ``adj_parts`` the broadcast stage loop multiplies by.  Added on top of the
reference surface: ``COO_Graph.from_dict`` and ``Parted_COO_Graph.from_full`` build the same objects
in memory (the benchmark regenerates its graph from a seed on every rank, nothing to read from
disk), and ``Parted_COO_Graph.plan(s)`` caches the device-side CSR plan of ``adj_parts[s]``.
"""
import datetime
import os

import torch

from . import datasets, graph_utils


class BasicGraph:
    """Moves a cached attribute dict to the device (parted_coo_graph.py:9-16)."""

    def __init__(self, d, name, device):
        self.name, self.device, self.attr_dict = name, device, d
        self.adj = d['adj'].to(device)
        self.features = d['features'].to(device)
        labels = d['labels'].to(device)
        self.labels = labels.to(torch.float if labels.dim() == 2 else torch.long)
        self.train_mask, self.val_mask, self.test_mask = (
            d[k].bool().to(device) for k in ('train_mask', 'val_mask', 'test_mask'))
        self.num_nodes, self.num_edges, self.num_classes = d['num_nodes'], d['num_edges'], d['num_classes']

    def __repr__(self):
        counts = ','.join(str(int(m.sum())) for m in (self.train_mask, self.val_mask, self.test_mask))
        return f'<COO Graph: {self.name}, |V|: {self.num_nodes}, |E|: {self.num_edges}, masks: {counts}>'


class GraphCache:
    """Cache file naming and (de)serialisation (parted_coo_graph.py:23-48)."""

    @staticmethod
    def full_graph_path(name, preprocess_for, root=None):
        return os.path.join(root or datasets.data_root, f'{name}_{preprocess_for}_full.coo_graph')

    @staticmethod
    def parted_graph_path(name, preprocess_for, rank, num_parts, root=None):
        folder = os.path.join(root or datasets.data_root, f'{name}_{preprocess_for}_{num_parts}_parts')
        os.makedirs(folder, exist_ok=True)
        return os.path.join(folder, f'part_{rank}_of_{num_parts}.coo_graph')

    @staticmethod
    def save_dict(d, path):
        if os.path.exists(path):
            print(f'warning: cache file {path} is overwritten.')
        # plain tensors are cloned so views do not drag their whole storage into the file
        torch.save({k: (v.clone() if type(v) is torch.Tensor and not v.is_sparse else v) for k, v in d.items()}, path)

    @staticmethod
    def load_dict(path):
        d = torch.load(path)
        for k, v in list(d.items()):
            if type(v) is torch.Tensor and v.is_sparse:
                d[k] = v.coalesce()
        return d


def _zero_pad(t, pad):
    return torch.cat((t, torch.zeros((pad,) + tuple(t.shape[1:]), dtype=t.dtype, device=t.device)))


class COO_Graph(BasicGraph):
    def __init__(self, name, preprocess_for='GCN', full_graph_cache_enabled=True, device='cpu'):
        self.preprocess_for = preprocess_for
        self.cache_path = GraphCache.full_graph_path(name, preprocess_for)
        if full_graph_cache_enabled and os.path.exists(self.cache_path):
            attr = GraphCache.load_dict(self.cache_path)
        else:
            attr = graph_utils.preprocess(name, datasets.load_dataset(name), preprocess_for)
            GraphCache.save_dict(attr, self.cache_path)
        super().__init__(attr, name, device)

    @classmethod
    def from_dict(cls, name, dataset_dict, preprocess_for='GCN', device='cpu', normalize_features=True):
        """Same object as the constructor, from an in-memory dataset dict (keys of save_dataset);
        nothing is read or written on disk.  ``normalize_features=False`` skips the feature row
        normalisation of ``preprocess`` for callers that feed already-prepared features."""
        self = cls.__new__(cls)
        self.preprocess_for, self.cache_path = preprocess_for, None
        d = dict(dataset_dict)
        if normalize_features:
            attr = graph_utils.preprocess(name, d, preprocess_for)
        else:
            attr = d
            attr['adj'] = graph_utils.sym_normalization(attr.pop('edge_index'), attr['num_nodes'])
        BasicGraph.__init__(self, attr, name, device)
        return self

    def part_dict(self, rank, num_parts, padding=True):
        """The dict ``partition`` stores for one rank (parted_coo_graph.py:63-93): row block of adj
        re-shaped to (n, n*P), feature block zero-padded to n rows, GLOBAL labels and masks padded to n*P."""
        n = (self.num_nodes + num_parts - 1) // num_parts
        pad = n * num_parts - self.num_nodes
        if (self.num_nodes + n - 1) // n < num_parts:
            raise IndexError(f'{self.num_nodes} nodes cannot fill {num_parts} blocks of {n} rows')
        idx, val = self.adj.indices(), self.adj.values()
        lo, hi = torch.searchsorted(idx[0].contiguous(), torch.tensor([n * rank, n * (rank + 1)], device=idx.device)).tolist()
        sub_idx = idx[:, lo:hi].clone()
        sub_idx[0] -= n * rank
        rows = min(n, self.num_nodes - n * rank)
        feats = self.features[n * rank:n * rank + rows]
        d = dict(self.attr_dict)
        d['labels'], d['train_mask'], d['val_mask'], d['test_mask'] = \
            self.labels.to(self.attr_dict['labels'].dtype), self.train_mask, self.val_mask, self.test_mask
        if padding and pad > 0:
            if rows < n:
                feats = _zero_pad(feats, n - rows)
            for k in ('labels', 'train_mask', 'val_mask', 'test_mask'):
                d[k] = _zero_pad(d[k], pad)
            shape = (n, n * num_parts)
        else:
            shape = (rows, self.num_nodes)
        d['adj'] = graph_utils._coo(sub_idx, val[lo:hi], shape)
        d['features'] = feats
        return d

    def partition(self, num_parts, padding=True):
        begin = datetime.datetime.now()
        print(self.name, num_parts, 'partition begin', begin)
        for r in range(num_parts):
            GraphCache.save_dict(self.part_dict(r, num_parts, padding),
                                 GraphCache.parted_graph_path(self.name, self.preprocess_for, r, num_parts))
            print(Parted_COO_Graph(self.name, r, num_parts, self.preprocess_for))
        print(self.name, num_parts, 'partition done', datetime.datetime.now() - begin)


class Parted_COO_Graph(BasicGraph):
    def __init__(self, name, rank, num_parts, preprocess_for='GCN', device='cpu'):
        path = GraphCache.parted_graph_path(name, preprocess_for, rank, num_parts)
        if not os.path.exists(path):
            raise Exception('Not parted yet. Run COO_Graph.partition() first.', path)
        self._finish(GraphCache.load_dict(path), name, rank, num_parts, device)

    @classmethod
    def from_full(cls, full_graph, rank, num_parts, device=None):
        """The object the constructor would load after ``full_graph.partition(num_parts)``, built in memory."""
        self = cls.__new__(cls)
        self._finish(full_graph.part_dict(rank, num_parts), full_graph.name, rank, num_parts,
                     device if device is not None else full_graph.device)
        return self

    def _finish(self, d, name, rank, num_parts, device):
        self.rank, self.num_parts = rank, num_parts
        BasicGraph.__init__(self, d, name, device)
        n = self.local_num_nodes = self.adj.size(0)
        self.local_num_edges = self.adj.values().size(0)
        self.local_labels = self.labels[n * rank:n * (rank + 1)]
        self.local_train_mask = self.train_mask[n * rank:n * (rank + 1)].bool()
        self.adj_parts = graph_utils.sparse_2d_split(self.adj, n, split_dim=1)

    def plan(self, s):
        """Device CSR plan of ``adj_parts[s]``, built on first use and cached for the life of that block."""
        import spmm_cpp
        return spmm_cpp.plan_for(self.adj_parts[s])

    def __repr__(self):
        return super().__repr__() + f'<Local: {self.rank}, |V|: {self.local_num_nodes}, |E|: {self.local_num_edges}>'

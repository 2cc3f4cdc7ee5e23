"""Training flow with the surface of light_dist_gnn/dist_train.py: train(g, env, total_epoch) and main(env, args)."""
import numpy as np
import torch
import torch.nn as nn

import spmm_cpp

from coo_graph import Parted_COO_Graph
from dist_utils import DistEnv
from models import GCN


def f1(y_true, y_pred, multilabel=True):
    from sklearn.metrics import f1_score
    y_true, y_pred = y_true.cpu().numpy(), y_pred.cpu().numpy()
    if multilabel:
        y_pred = (y_pred > 0.5).astype(np.float32)
    else:
        y_pred = np.argmax(y_pred, axis=1)
    return f1_score(y_true, y_pred, average='micro'), f1_score(y_true, y_pred, average='macro')


def local_loss(g, outputs, loss_func):
    """Mean loss over this rank's LOCAL train rows (dist_train.py:39-43); a rank without train rows still
    back-propagates a zero so that it takes part in every collective."""
    cached = getattr(g, '_train_rows', None)
    if cached is None:      # the mask never changes: find the rows once instead of a host sync per epoch
        rows = g.local_train_mask.nonzero().squeeze(1)
        cached = g._train_rows = (rows, g.local_labels[rows])
    rows, labels = cached
    if rows.numel() > 0:
        return loss_func(outputs.index_select(0, rows), labels)
    DistEnv.env.logger.log('Warning: no training nodes in this partition! Backward fake loss.')
    return (outputs * 0).sum()


def train(g, env, total_epoch, hidden_dim=256, num_layers=3, weights=None, log_every=10, **model_options):
    """The reference's epoch loop (dist_train.py:26-55).  model_options go to GCN (cache_input_product,
    input_gradient_shortcut); the defaults recompute everything every epoch, as the reference does."""
    model = GCN(g, env, hidden_dim=hidden_dim, num_layers=num_layers, weights=weights, **model_options)
    optimizer = torch.optim.Adam(model.parameters(), lr=0.01)
    loss_func = nn.CrossEntropyLoss() if g.labels.dim() == 1 else nn.BCEWithLogitsLoss(reduction='mean')
    losses = []
    for epoch in range(total_epoch):
        with env.timer.timing('epoch'):
            outputs = model(g.features)
            optimizer.zero_grad()
            loss = local_loss(g, outputs, loss_func)
            loss.backward()
            optimizer.step()
            losses.append(loss.item())
            if outputs.is_cuda:         # the device is idle after loss.item(): the cheapest place for both
                spmm_cpp.check_dense_status()
                env.timer.resolve(synchronize=False)
            env.logger.log('Epoch {:05d} | Loss {:.4f}'.format(epoch, losses[-1]), rank=0)
        if epoch % log_every == 0 or epoch == total_epoch - 1:
            all_outputs = env.all_gather_then_cat(outputs)
            if g.labels.dim() > 1:
                mask = g.train_mask
                env.logger.log(f'Epoch: {epoch:03d}', f1(g.labels[mask], torch.sigmoid(all_outputs[mask])), rank=0)
            else:
                acc = lambda mask: all_outputs[mask].max(1)[1].eq(g.labels[mask]).sum().item() / max(mask.sum().item(), 1)
                env.logger.log(f'Epoch: {epoch:03d}, Train: {acc(g.train_mask):.4f}, Val: {acc(g.val_mask):.4f}, '
                               f'Test: {acc(g.test_mask):.4f}', rank=0)
    return model, losses


def main(env, args):
    env.logger.log('proc begin:', env)
    with env.timer.timing('total'):
        parts = env.world_size // env.rep
        g = Parted_COO_Graph(args.dataset, rank=env.rank // env.rep, num_parts=parts, device=env.device)
        env.logger.log('graph loaded', g)
        train(g, env, total_epoch=args.epoch, hidden_dim=getattr(args, 'hidden', 256), num_layers=getattr(args, 'layers', 3))
    env.logger.log(env.timer.summary_all(), rank=0)

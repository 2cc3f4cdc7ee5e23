"""Per-rank logger: prints and appends to logs_{P}/all_log_{rank}.txt (light_dist_gnn/dist_utils/logger.py:5-20)."""
import datetime as dt
import os


class DistLogger:
    def __init__(self, env):
        self.env = env
        root = os.environ.get('DIST_GNN_LOG_ROOT', os.path.join(os.path.dirname(__file__), '..'))
        self.log_root = os.path.join(root, f'logs_{env.world_size}')
        os.makedirs(self.log_root, exist_ok=True)
        self.log_fname = os.path.join(self.log_root, f'all_log_{env.rank}.txt')

    def log(self, *args, oneline=False, rank=-1):
        if rank != -1 and self.env.rank != rank:
            return
        line = f'{dt.datetime.now().time()} [{self.env.rank:1d}] ' + ' '.join(map(str, args)) + ('\r' if oneline else '\n')
        print(line, end='', flush=True)
        with open(self.log_fname, 'a+') as f:
            f.write(line)

from .gcn import GCN

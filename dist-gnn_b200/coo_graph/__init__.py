from .parted_coo_graph import COO_Graph, Parted_COO_Graph

"""Process-wide configuration store.

Mirrors the role of the reference's ``axonn/config.py:7-10``: a module whose
attributes hold the grid sizes and this rank's coordinates after
``axonn_b200.axonn.init``.  Unlike the reference, every name that ``init`` and
``create_dataloader`` may set is declared here so readers can see the schema.
"""

# grid sizes
G_inter = 1
G_data = 1
G_intra = 1
G_intra_r = 1
G_intra_c = 1
G_intra_d = 1

# this rank's coordinates
inter_layer_parallel_rank = 0
data_parallel_rank = 0
intra_layer_parallel_rank = 0
intra_layer_row_parallel_rank = 0
intra_layer_column_parallel_rank = 0
intra_layer_depth_parallel_rank = 0

# set by create_dataloader
micro_batch_size = None
batch_size = None
batch_size_per_gpu = None

# device string used for parameters / staging ("cuda" or "cpu")
device = "cpu"


def reset():
    """Restore defaults (used by tests that call ``init`` repeatedly)."""
    g = globals()
    for k in ("G_inter", "G_data", "G_intra", "G_intra_r", "G_intra_c", "G_intra_d"):
        g[k] = 1
    for k in (
        "inter_layer_parallel_rank",
        "data_parallel_rank",
        "intra_layer_parallel_rank",
        "intra_layer_row_parallel_rank",
        "intra_layer_column_parallel_rank",
        "intra_layer_depth_parallel_rank",
    ):
        g[k] = 0
    g["micro_batch_size"] = g["batch_size"] = g["batch_size_per_gpu"] = None
    g["device"] = "cpu"

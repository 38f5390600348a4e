"""axonn_b200: a Blackwell-native 4-D hybrid-parallel training framework.

Public surface (same names as the ``axonn`` package it mirrors)::

    from axonn_b200 import axonn as ax          # ax.init(G_inter, G_data, r, c, d)
    from axonn_b200.intra_layer import Linear, Conv2d, Embedding, auto_parallelize,
        optimize_communication, sync_gradients, clip_grad_norm_, no_grad_sync
    from axonn_b200.inter_layer import AxoNN_Inter_Layer_Engine
    from axonn_b200 import checkpoint, optim, models
"""

__version__ = "0.1.0"

from . import config  # noqa: F401
from . import axonn  # noqa: F401
from . import ops  # noqa: F401
from . import intra_layer  # noqa: F401
from . import checkpoint  # noqa: F401

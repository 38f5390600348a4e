"""axonn_b200: a Blackwell-native 4-D hybrid-parallel training framework.

Public surface (same names as the ``axonn`` package it mirrors)::

    from axonn_b200 import axonn as ax          # ax.init(G_inter, G_data, r, c, d)
    from axonn_b200.intra_layer import Linear, Conv2d, Embedding, auto_parallelize,
        optimize_communication, sync_gradients, clip_grad_norm_, no_grad_sync
    from axonn_b200.inter_layer import AxoNN_Inter_Layer_Engine
    from axonn_b200 import checkpoint, optim, models
"""

__version__ = "0.1.0"

import os as _os

# A pipeline stage keeps several blocking NCCL point-to-point kernels in flight (one communicator per neighbour and
# direction) next to its compute stream.  With the default of 8 hardware work queues per device two of those streams
# can share a queue, and a send queued behind a receive that still waits for its peer cannot start.  Asking for the
# maximum number of queues (before the CUDA context exists) makes such false dependencies less likely; it did not by
# itself cure the stall of the message-driven schedule on four NCCL stages, which is why the pipeline engine also
# posts its receives in a fixed order there.
_os.environ.setdefault("CUDA_DEVICE_MAX_CONNECTIONS", "32")

from . import config  # noqa: F401
from . import axonn  # noqa: F401
from . import ops  # noqa: F401
from . import intra_layer  # noqa: F401
from . import checkpoint  # noqa: F401

"""Run code written against the upstream ``axonn`` package on this one without editing its imports.

``install_as_axonn()`` registers this package and its modules in ``sys.modules`` under the upstream names, so that

    import axonn_b200.compat; axonn_b200.compat.install_as_axonn()
    from axonn import axonn as ax
    from axonn.intra_layer import Linear, auto_parallelize, sync_gradients
    from axonn.inter_layer import AxoNN_Inter_Layer_Engine
    from axonn.lightning import AxonnStrategy
    from axonn.models.transformers import parallelize

resolve to the modules of ``axonn_b200`` (the public names and call shapes are the same: upstream
``axonn/__init__.py``, ``axonn/intra_layer/__init__.py:10-23``, ``axonn/lightning/__init__.py``).  It is a run-time
alias on request, not a package called ``axonn`` on disk, so it cannot shadow a real installation by accident; if
the real package has been imported already the call refuses.
"""

import importlib
import sys

_MODULES = (
    "axonn", "config", "communication", "timers", "checkpoint", "optim", "inter_layer", "utils",
    "intra_layer", "intra_layer.fully_connected", "intra_layer.conv", "intra_layer.embedding",
    "intra_layer.communication", "intra_layer.asym_communication", "intra_layer.overlap_communication",
    "intra_layer.automatic_parallelism", "intra_layer.gradient_normalization",
    "lightning", "lightning.axonn_strategy", "models", "models.transformers",
)


def install_as_axonn() -> None:
    """Alias ``axonn`` and ``axonn.<module>`` to this package's modules (idempotent)."""
    import axonn_b200

    present = sys.modules.get("axonn")
    if present is not None and present is not axonn_b200:
        raise RuntimeError(f"a different 'axonn' package is already imported from {getattr(present, '__file__', '?')}")
    sys.modules["axonn"] = axonn_b200
    for name in _MODULES:
        sys.modules["axonn." + name] = importlib.import_module("axonn_b200." + name)

"""Lightning Fabric integration (``AxonnStrategy``)."""

from .axonn_strategy import AxonnStrategy, LIGHTNING_AVAILABLE  # noqa: F401

"""pegaflow_b200: B200-native KV-cache save/load path behind PegaFlow's engine interface.

The package is a thin Python layer over ``libpegaflow_b200.so`` (C ABI in
``include/pegaflow_b200.h``).  Importing it without the built library raises; there is no
CPU fallback.
"""
from ._native import PegaFlowError, PegaflowInternal, PegaflowInvalidArgument  # noqa: F401
from .backend import (HostRun, LayerXfer, PinnedPool, TransferBackend, enable_peer_access,  # noqa: F401
                      numa_node_of_device, save_blocks_noalloc)
from .engine import Block, Completion, PegaEngine, PyLoadState  # noqa: F401
from .connector import InProcEngineClient, QueryLoading, QueryReady, TransferStats  # noqa: F401,E402

"""b200fw: a Blackwell (sm_100a) native train / RL / inference framework."""
__version__ = "0.1.0"

import os as _os

# More hardware work queues than the default 8: the framework runs compute, optimizer communication, pipeline
# transfers and NCCL's own streams side by side, and streams that share a queue serialise (a kernel that waits for a
# peer then holds back unrelated work queued behind it).  Read by the CUDA driver when the context is created, so it
# only takes effect when this package is imported before the first CUDA call; an explicit setting wins.
_os.environ.setdefault("CUDA_DEVICE_MAX_CONNECTIONS", "32")

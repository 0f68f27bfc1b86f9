"""Trainer -> inference-engine weight synchronisation: SwiftSync LoRA deltas with a double buffer, the
NVLink peer-write path, the NCCL broadcast baseline, and the vLLM / IPC compatibility layer."""
from .double_buffer import DoubleBufferedLoRA
from .swift_sync import DeltaComputer, DeltaVersion, SwiftSyncConfig, SwiftSyncStats, SwiftSyncTransfer, SyncStats
from .nccl_transfer import (NCCLWeightTransfer, RayObjectStoreTransfer, TransferStats, WeightTransferManager,
                            WeightVersion)
from .ipc_transfer import (IPCHandle, IPCWeightTransfer, NonRetriableError, VLLMClient, WeightUpdateManager, classify_error)
from .peer_write import PeerWeightSync, VersionedWeightBuffer, fletcher_checksum

__all__ = [
    "DoubleBufferedLoRA", "DeltaComputer", "SwiftSyncConfig", "SwiftSyncStats", "SwiftSyncTransfer",
    "NCCLWeightTransfer", "RayObjectStoreTransfer", "TransferStats", "WeightTransferManager",
    "IPCWeightTransfer", "NonRetriableError", "VLLMClient", "WeightUpdateManager", "classify_error",
    "PeerWeightSync", "VersionedWeightBuffer", "fletcher_checksum", "DeltaVersion", "SyncStats", "WeightVersion",
    "IPCHandle",
]

"""KV-cache page migration over peer memory (push path)."""
from .copy import canonicalize_block_runs
from .lifecycle import TransferLedger, TransferRecord, TransferState
from .manager import CompiledKVTransferManager, KVPoolLayout
from .profile import (B200_NVLINK_KV_TARGET_PROFILE, GENERIC_KV_TARGET_PROFILE,
                      H200_NVLINK_KV_TARGET_PROFILE, KVRuntimeOverrides, KVTargetProfile,
                      select_kv_target_profile)

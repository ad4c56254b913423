"""aboleth_b200: GPU-initiated communication for B200 (sm_100a) over NVLink peer memory.

The public names follow the reference package's ``__all__`` (python/aboleth/__init__.py:126-227)
wherever the concept exists here; ``aboleth_b200.compiler`` replaces its Triton language
module, ``aboleth_b200.ops`` / ``parallel`` / ``models`` hold what the reference has no
counterpart for (tcgen05 GEMMs, fused TP collectives, the serving model).
"""
from . import abi  # noqa: F401
from .bootstrap import (Bootstrap, LocalBootstrap, PipeBootstrap, PipeBootstrapCoordinator,
                        TcpStoreBootstrap, TorchDistributedBootstrap, decode_bundle, encode_bundle)
from .compiler import (Artifact, CompileError, CompiledProgram, ProgramBuilder, build_artifact,
                       compilation, compile_program)
from .device_library import DeviceLibrary, device_library
from .endpoint_profiles import EndpointProfile
from .execution import (CapacityContract, ExecutionContract, ExecutionDecision, ExecutionFallback,
                        PaddingSemantics, RankControl, RuntimeGuard, compile_execution_plan)
from .pattern import (CommunicationStage, CompiledPattern, CompiledPatternPlan, KernelBinding,
                      OpaqueCapabilities, OpaqueStage, P2PRealizationProfile, Pattern, PhaseResources,
                      PhaseSchedule, RegionRequirement, Workset)
from .phase import CompiledPhase, PhaseBinding, compile_phase
from .planning import (CommunicationDataflow, CommunicationRegion, RegionEffect,
                       SimplifiedCommunicationDataflow, TransportPhase, plan_endpoint_work, plan_storage,
                       plan_transport, plan_transport_partitions, simplify_communication_dataflow)
from .runtime import (AllocationHandle, AllocationProvider, Endpoint, EndpointTable, LocalBuffer,
                      LocalEndpoint, Provider, RegisteredBuffer, RemoteBuffer, RemoteHandle, Runtime,
                      Transport, available_transports, connection_info_from_bytes, connection_transport,
                      provider_caps)
from .shapes import ShapeFamilyPlan, plan_shape_family
from .world import AutoTransportPolicy, LocalRegion, PeerRegionTable, TopologyInfo, World

FragmentArtifact = Artifact
StandaloneKernel = CompiledProgram
TransportPlan = dict

from . import moe, ops, parallel  # noqa: E402,F401
from .kv import (GENERIC_KV_TARGET_PROFILE, H200_NVLINK_KV_TARGET_PROFILE,  # noqa: E402
                 CompiledKVTransferManager, KVPoolLayout, KVRuntimeOverrides, KVTargetProfile,
                 select_kv_target_profile)

from .patterns import (CompiledKVCacheMigrationPlan, KVCacheLayoutContract,  # noqa: E402
                       KVCacheMigrationSpec, KVCachePhysicalization, MoEPatternSpec,
                       build_kv_cache_migration_pattern, build_moe_pattern, compile_kv_cache_migration)

__version__ = "0.1.0"

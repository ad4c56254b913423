"""aboleth_b200: GPU-initiated communication for B200 (sm_100a) over NVLink peer memory.

The public names follow the reference package's ``__all__`` (python/aboleth/__init__.py:126-227)
wherever the concept exists here; ``aboleth_b200.compiler`` replaces its Triton language
module, ``aboleth_b200.ops`` / ``parallel`` / ``models`` hold what the reference has no
counterpart for (tcgen05 GEMMs, fused TP collectives, the serving model).
"""
from . import abi  # noqa: F401
from .bootstrap import (Bootstrap, LocalBootstrap, PipeBootstrap, PipeBootstrapCoordinator,
                        TcpStoreBootstrap, TorchDistributedBootstrap, decode_bundle, encode_bundle)
from .compiler import (CompileError, CompiledProgram, LoadedKernel, ProgramBuilder, build_artifact,
                       compilation, compile_program)
from .compiler.artifact import (FragmentArtifact, StandaloneKernel, compile_fragment_artifact,
                                realize_bindable_epilogue, realize_standalone_kernel)
from .compiler.driver import install_compiler
from .device_library import DeviceLibrary, device_library
from .endpoint_profiles import EndpointProfile
from .execution import (CapacityContract, CompiledExecutionPlan, ExecutionContract, ExecutionDecision, ExecutionFallback,
                        PaddingSemantics, RankControl, RuntimeGuard, compile_execution_plan)
from .pattern import (CommunicationStage, CompiledPattern, CompiledPatternPlan, KernelBinding,
                      OpaqueCapabilities, OpaqueStage, P2PRealizationProfile, Pattern, PhaseResources,
                      PhaseSchedule, RegionRequirement, Workset)
from .language import (drain, invoke_transport_program, planned_wait, put, signal, token, token_type, wait,
                       wait_signal)
from .phase import CompiledPhase, PhaseLaunch, compile_phase
from .physicalization import (Artifact, PhaseBinding, PhysicalizedPattern, RuntimeBindings,
                              RuntimeBufferBinding, physicalize_pattern)
from .planning import (CommunicationDataflow, CommunicationDataflowOperation, CommunicationRegion,
                       OutputLifetimePlan, RegionAccess, RegionEffect, SimplifiedCommunicationDataflow,
                       TransportKernel, TransportPhase, TransportPlan, plan_endpoint_work,
                       plan_output_lifetimes, plan_storage, plan_transport, plan_transport_facts,
                       plan_transport_partitions, plan_transport_program, simplify_communication_dataflow)
from .runtime import (AllocationHandle, AllocationProvider, Endpoint, EndpointMesh, EndpointPair,
                      EndpointTable, LocalBuffer,
                      LocalEndpoint, Provider, RegisteredBuffer, RemoteBuffer, RemoteHandle, Runtime,
                      Transport, available_transports, connection_info_from_bytes, connection_transport,
                      PortAddress, probe_providers, provider_caps, query_port_address, select_device,
                      select_gid_index)
from .shapes import ShapeFamilyPlan, plan_shape_family
from .world import AutoTransportPolicy, LocalRegion, PeerRegionTable, TopologyInfo, World


from . import frontends, moe, ops, parallel  # noqa: E402,F401
from .kv import (GENERIC_KV_TARGET_PROFILE, H200_NVLINK_KV_TARGET_PROFILE,  # noqa: E402
                 CompiledKVTransferManager, KVPoolLayout, KVRuntimeOverrides, KVTargetProfile,
                 select_kv_target_profile)

from .patterns import (CompiledKVCacheMigrationPlan, KVCacheLayoutContract,  # noqa: E402
                       KVCacheMigrationSpec, KVCachePhysicalization, MoEPatternSpec,
                       build_kv_cache_migration_pattern, build_moe_pattern, compile_kv_cache_migration)

from .transport_binding import InvokeManifest, KernelTransportReduction  # noqa: E402

__version__ = "0.1.0"

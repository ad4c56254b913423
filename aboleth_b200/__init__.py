"""B200-native GPU-initiated communication framework with Aboleth's capabilities."""
from .bootstrap import (Bootstrap, LocalBootstrap, PipeBootstrap, PipeBootstrapCoordinator,
                        TcpStoreBootstrap, TorchDistributedBootstrap, decode_bundle, encode_bundle)
from .runtime import (AllocationHandle, AllocationProvider, Endpoint, EndpointTable, LocalBuffer,
                      LocalEndpoint, Provider, RegisteredBuffer, RemoteBuffer, RemoteHandle,
                      Runtime, Transport, available_transports, connection_info_from_bytes,
                      connection_transport, provider_caps)
from .world import AutoTransportPolicy, LocalRegion, PeerRegionTable, TopologyInfo, World

from . import abi, moe, ops, parallel  # noqa: E402,F401

__version__ = "0.1.0"

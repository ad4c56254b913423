"""Serving-engine integration: modular MoE prepare/finalize, the all2all backend, KV migration."""
from .compiled_vllm import AbolethMoERuntimeManager, ModularMoERuntime, PreparedExperts
from .vllm_all2all import AbolethAll2AllManager, AbolethPrepareAndFinalize, register_with_vllm
from .vllm_kv import KVCachePullTicket, VLLMKVPeerRuntime

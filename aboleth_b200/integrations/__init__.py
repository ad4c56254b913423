"""Serving-engine integration: modular MoE prepare/finalize and the all2all backend."""
from .compiled_vllm import AbolethMoERuntimeManager, ModularMoERuntime, PreparedExperts
from .vllm_all2all import AbolethAll2AllManager, AbolethPrepareAndFinalize, register_with_vllm

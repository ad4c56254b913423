"""Expert-parallel MoE: spec, fused dispatch/combine executor, CPU oracle."""
from .native import (PHASE_RECV, PHASE_SEND, DispatchResult, LocalMoEGroup, MoEBuffers,
                     NativeMoESlot)
from .spec import MoESpec
from .compiled_plan import CompiledMoEPlan, build_dataflow, compile_moe_plan
from .family import NativeMoEFamily, uniform_token_bound

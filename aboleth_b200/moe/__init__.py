"""Expert-parallel MoE: spec, fused dispatch/combine executor, CPU oracle."""
from .native import (PHASE_RECV, PHASE_SEND, DispatchResult, LocalMoEGroup, MoEBuffers,
                     NativeMoESlot)
from .spec import MoESpec

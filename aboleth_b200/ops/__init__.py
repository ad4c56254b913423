"""Python entry points of the hand-written sm_100a kernels."""
from .comm import alltoall, check_payload, fill_payload, pingpong, tier1_exercise
from .moe_ops import expert_offsets, permute, quant_fp8, router_topk, standin_expert, unpermute
from .gemm import (check_gemm_status, dequant_block_scaled, gemm_bf16, gemm_e4m3, gemm_e4m3_block_scaled,
                   gemm_e4m3_mx, gemm_status, grouped_gemm_bf16, grouped_gemm_e4m3_mx, pack_scales_mx)
from ._kernels import launch_count

"""B200-native EXL3 projection engine: hand-written sm_100a kernels behind turboexl3's projection entry points.

The product is libt3.so (C ABI: include/t3.h); this package is its Python host layer, mirroring the reference's module
API (src/root.zig). Importing the package does not load the library; the first call does, and fails loudly if it has not
been built (`python -m turboexl3_b200.build`).
"""
from .api import (last_kernel_symbol, plan_linear, plan_moe, EP_WORLD_MAX, ep_plan, BANKED_ROWS_MAX, BANKED_SKIP_ID, CLAMP_GATE_IN, CLAMP_SILU_OUT, DECODE_ROWS_MAX, MCG, MUL1, REDUCE_MAX_TOPK, Bank, Decode, Exl3Error,
                  Proj, codebook_table, configure, dequantize, device_error, engines_held, launch_count, lib, linear, linear_resident, linear_unrot, moe,
                  moe_clamped_banked, unrot_build,
                  moe_clamped, moe_merge, moe_swiglu, moe_swiglu_rows, moe_with_shared, parse_expert_quant, release_engines, resident_build,
                  status_name, trellis_admitted)

__all__ = ["last_kernel_symbol", "plan_linear", "plan_moe", "EP_WORLD_MAX", "ep_plan", "BANKED_ROWS_MAX", "BANKED_SKIP_ID", "linear_unrot", "moe_clamped_banked", "unrot_build", "CLAMP_GATE_IN", "CLAMP_SILU_OUT", "DECODE_ROWS_MAX", "MCG", "MUL1", "REDUCE_MAX_TOPK", "Bank", "Decode",
           "Exl3Error", "Proj", "codebook_table", "configure", "dequantize", "device_error", "engines_held", "launch_count", "lib", "linear_resident", "resident_build",
           "linear", "moe", "moe_clamped", "moe_merge", "moe_swiglu", "moe_swiglu_rows", "moe_with_shared", "parse_expert_quant", "release_engines",
           "status_name",
           "trellis_admitted"]

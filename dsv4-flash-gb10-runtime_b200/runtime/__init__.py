"""Host-side operators: the reference's three bindings under their own names, and the routed-MoE helpers."""
from .mxfp4_gemv_binding import mxfp4_gemv                                   # noqa: F401
from .fp8_e4m3_gemv_binding import (fp8_e4m3_gemv, fp8_e4m3_gemv_batched, fp8_e4m3_gemv_f32scale,     # noqa: F401
                                    fp8_shared_swiglu)
from .mxfp4_grouped_gemv_binding import (                                    # noqa: F401
    mxfp4_grouped_gemv, mxfp4_grouped_gemv_static, mxfp4_grouped_gemv_ids, mxfp4_dequant_bf16, moe_route_topk, device_status,
    moe_decode_layer, decode_workspace_bytes, decode_picks)
from .moe_batched import moe_forward, forward_workspace_bytes, moe_device_status, mma_clocks, stage_timing, stage_times, STAGES   # noqa: F401
from .bank_loader import load_expert_bank, load_shared_expert_fp8, SnapshotReader   # noqa: F401

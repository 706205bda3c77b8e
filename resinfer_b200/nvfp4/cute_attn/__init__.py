"""ResAttn decode under the reference's ``nvfp4.cute_attn`` name."""
from .kv_layout import PAGE_SIZE, SF_VEC, NvFp4PagedKVPool
from .plan import select_decode_plan, static_compile_plans, validate_decode_plan

__all__ = ["NvFp4PagedKVPool", "PAGE_SIZE", "SF_VEC", "select_decode_plan", "static_compile_plans",
           "validate_decode_plan"]

"""Hand-written sm_100a kernels (csrc/sm100) behind autograd functions, with PyTorch oracles on CPU."""
from . import _lib  # noqa: F401
from .attention import (attention_merge, attention_reference, flash_attention, flash_attention_packed,  # noqa: F401
                        flash_backward)
from .fused import (activation, apply_mrope, cross_entropy, embedding, mrope_angles, norm, rope_packed,  # noqa: F401
                    rope_tables, router_topk)
from .gemm import gemm, grouped_gemm, grouped_wgrad, linear  # noqa: F401
from .optim import adamw_step, cast_bf16, clip_coefficient, scale_, sumsq  # noqa: F401

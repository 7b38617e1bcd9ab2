"""Hot-path operators.  Each op has a PyTorch oracle (``*_ref``) and an sm_100a kernel."""
from . import backend  # noqa: F401
from .activations import glu, swiglu, swiglu_packed, oss_swiglu_ref  # noqa: F401
from .attention import attention, attention_ref, pointwise_attention  # noqa: F401
from .conv1d import causal_conv1d, causal_conv1d_ref  # noqa: F401
from .cross_entropy import (FusedCrossEntropyLoss, FusedLinearCrossEntropyLoss, cross_entropy, cross_entropy_ref,  # noqa: F401
                            fused_linear_cross_entropy, fused_linear_cross_entropy_ref)
from .gated_delta_rule import gated_delta_rule, gated_delta_rule_recurrent_ref  # noqa: F401
from .gemm import linear, linear_swiglu, matmul_nn, matmul_nt, matmul_tn  # noqa: F401
from .moe import (load_balance_loss, moe_ffn, moe_ffn_ref, router_topk_softmax, routing_metadata,  # noqa: F401
                  stable_topk)
from .newton_schulz import newton_schulz, newton_schulz_ref  # noqa: F401
from .norm import add_rms_norm, add_rms_norm_ref, gated_rms_norm, layer_norm, rms_norm, rms_norm_ref, layer_norm_ref, gated_rms_norm_ref  # noqa: F401
from .rope import apply_rotary_emb, build_rope_cache, qk_norm_rope, qkv_norm_rope, qkv_norm_rope_supported  # noqa: F401
from .selective_scan import selective_scan, selective_scan_ref  # noqa: F401
from .ssd import ssd_scan, ssd_scan_ref  # noqa: F401
from .diff_attn import diff_combine, diff_combine_ref  # noqa: F401,E402

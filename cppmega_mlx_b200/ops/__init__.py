"""Operator layer: each op has a PyTorch restatement (oracle / CPU path) and an sm_100a kernel path."""
from ._backend import check_status, has_library, kernels_enabled, load_library, set_kernels_enabled, use_kernels
from .activations import squared_relu, swiglu, swiglu_reference
from .conv import causal_conv1d_silu, packed_split_conv_silu
from .attention import masked_attention, masked_attention_reference
from .cce import linear_cross_entropy, linear_cross_entropy_reference
from .gemm import gemm_batched, gemm_raw, linear, linear_relu2, matmul_nt
from .m2rnn_post import m2rnn_post_gate, m2rnn_post_gate_reference
from .m2rnn_scan import broadcast_m2rnn_heads, m2rnn_scan, m2rnn_scan_reference
from .mamba3_scan import mamba3_scan, mamba3_scan_chunked, mamba3_scan_sequential
from .norm import add_rms_norm, layer_norm_ref, rms_norm, rms_norm_ref
from .rope import RopeScaling, apply_rope, apply_rope_reference, rope_inv_freq, rope_tables, rope_tables_at, yarn_attention_factor
from .sparse_mla import indices_to_mask, sparse_mla_attention, sparse_mla_masked_dense, sparse_mla_reference
from .fp8_scale import fp8_amax, fp8_pack, fp8_quantize, linear_with_amax
from .sparse_mla_blockscaled import mxfp8_roundtrip_ste, sparse_mla_blockscaled
from . import decode_attention  # module: decode_attention.decode_attention(...) / .decode_attention_reference(...)
from .topk import topk_select, topk_select_reference

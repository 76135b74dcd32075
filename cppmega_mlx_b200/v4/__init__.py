from .blocks import (CSAHCAConfig, CSAHCAHybridV4, EngramV4Block, EngramV4Config, KimiDeltaAttentionBlock, KimiDeltaAttentionConfig,
                     LinearAttentionBlock, LinearAttentionConfig, NativeSparseAttentionV4, NSAConfig, StreamingPoolCache)
from .delta_rule import chunked_gated_delta_rule, gated_delta_rule, recurrent_gated_delta_rule
from .moe_fp8 import FP8FeedForwardExpert, FP8GroupedExperts, FP8Linear, convert_moe_to_fp8, fp8_roundtrip_ste, quantize_linear_to_fp8
from .mtp_adapter import MTPSpeculativeAdapter
from .run_template import BlockSpec, MTPSpec, RunTemplate, dump_template, dumps_template, load_template, loads_template
from .superblock import UnifiedLMV4, UnifiedSuperblockV4

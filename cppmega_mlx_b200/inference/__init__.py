from .engine import DecodeSession, HybridKVCache, PromptCacheEntry, make_kv_cache, supports_incremental_decode
from .generation import (GenerationChunk, build_prompt_cache, generate_from_prompt_cache, generate_tokens,
                         generate_tokens_with_kv_cache, next_token_logits, stream_generate_tokens)
from .graph_decode import GraphDecodeSession, StaticStepRunner
from .static_cache import PagedDecodeCache, StaticDecodeCache
from .serving_engine import ServingEngine, ServingRequest
from .infilling import build_infilling_prompt, splice_infill
from .sampling import apply_top_k, apply_top_p, sample_next_token
from .serving import (ContinuousBatchScheduler, PagedKVBlockManager, build_paged_block_table, paged_decode_attention,
                      paged_latent_decode_attention)
from .speculative_decode import leviathan_accept, speculative_generate, typical_accept

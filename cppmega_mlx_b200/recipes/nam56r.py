"""NAM56R recipe: the validated model description, its expanded layer plan, and the bridge to the runnable hybrid LM.

Counterpart of ``cppmega_mlx/recipes/nam56r.py`` (``:52`` build config, ``:70`` pattern, ``:90-111`` parity contract,
``:114`` route lookup, ``:121`` DSA rank override, ``:130-197`` hybrid config bridge).  The parity contract stays honest
about what the layer plan covers: A/E/M/R placement is native here, the upstream-only pattern symbols ``D``, ``G`` and
``|`` are not supported, so ``require_fully_native_megatron_parity`` always refuses.
"""
from __future__ import annotations

from dataclasses import dataclass, replace
from typing import NoReturn

from ..config.model import (DEFAULT_ATTENTION_HEADS, DEFAULT_DSA_A_LAYER_RANKS, DEFAULT_HIDDEN_SIZE, DEFAULT_NAM56R_DEPTH,
                            DEFAULT_NAM56R_PATTERN, M2RNNConfig, Mamba3Config, Nam56RModelConfig)
from .pattern import ExpandedNamPattern, expand_nam_pattern, parse_rank_list

UNSUPPORTED_MEGATRON_PARITY_SYMBOLS = ("D", "G", "|")
CUSTOM_MEGATRON_LAYER_ROLES = ("mamba3", "m2rnn")


@dataclass(frozen=True)
class Nam56RParityContract:
    pattern: ExpandedNamPattern
    locally_covered_roles: tuple[str, ...]
    custom_megatron_roles: tuple[str, ...]
    unsupported_megatron_symbols: tuple[str, ...]
    megatron_fully_native: bool

    @property
    def reason(self) -> str:
        return ("the NAM56R layer plan covers A/E/M/R route placement but does not claim fully native Megatron parity: "
                f"{', '.join(self.custom_megatron_roles)} are custom seams and the upstream-only symbols "
                f"{', '.join(self.unsupported_megatron_symbols)} are unsupported")


def build_nam56r_config(**overrides) -> Nam56RModelConfig:
    hidden = overrides.get("hidden_size", DEFAULT_HIDDEN_SIZE)
    heads = overrides.get("num_attention_heads", DEFAULT_ATTENTION_HEADS)
    if hidden % heads:
        raise ValueError("hidden_size must be divisible by num_attention_heads")
    overrides.setdefault("m2rnn", M2RNNConfig(d_model=hidden))
    overrides.setdefault("mamba3", Mamba3Config(d_model=hidden))
    return Nam56RModelConfig(**overrides)


def default_nam56r_config() -> Nam56RModelConfig:
    return build_nam56r_config()


def build_nam56r_pattern(config: Nam56RModelConfig | None = None, *, pattern: str | None = None, depth: int | None = None,
                         dsa_a_layer_ranks=None) -> ExpandedNamPattern:
    config = config or build_nam56r_config()
    ranks = config.dsa.a_layer_ranks if dsa_a_layer_ranks is None else parse_rank_list(dsa_a_layer_ranks)
    return expand_nam_pattern(pattern if pattern is not None else config.pattern, depth if depth is not None else config.depth,
                              dsa_a_layer_ranks=ranks)


def build_nam56r_parity_contract(config: Nam56RModelConfig | None = None) -> Nam56RParityContract:
    ex = build_nam56r_pattern(config)
    roles = tuple(dict.fromkeys(l.role for l in ex.layers))
    return Nam56RParityContract(ex, roles, CUSTOM_MEGATRON_LAYER_ROLES, UNSUPPORTED_MEGATRON_PARITY_SYMBOLS, False)


def require_fully_native_megatron_parity(config: Nam56RModelConfig | None = None) -> NoReturn:
    raise NotImplementedError(build_nam56r_parity_contract(config).reason)


def attention_route_for_layer(layer_number: int, config: Nam56RModelConfig | None = None):
    for l in build_nam56r_pattern(config).layers:
        if l.number == layer_number:
            return l.attention_route
    raise ValueError(f"layer {layer_number} is outside the pattern")


def with_dsa_a_layer_ranks(config: Nam56RModelConfig, ranks) -> Nam56RModelConfig:
    return replace(config, dsa=replace(config.dsa, a_layer_ranks=parse_rank_list(ranks)))


def build_hybrid_tiny_config_from_nam56r(config: Nam56RModelConfig | None = None, **overrides):
    """The runnable ``HybridTinyConfig`` for a NAM56R description; ``overrides`` shrink it for smoke runs."""
    from ..models.hybrid_lm import HybridTinyConfig
    config = config or build_nam56r_config()
    st = config.structure
    env = config.source_structure_env
    if env.enabled:
        st = replace(st, active_components=env.active_components, bottleneck_dim=env.bottleneck_dim, max_ast_depth=env.max_ast_depth,
                     max_sibling_index=env.max_sibling_index, num_node_types=env.num_node_types)
    nh = config.ngram_hash
    params = dict(
        vocab_size=config.vocab_size, hidden_size=config.hidden_size, pattern=config.pattern, depth=config.depth,
        dsa_a_layer_ranks=config.dsa.a_layer_ranks, num_attention_heads=config.num_attention_heads, max_seq_length=config.seq_len,
        structure_components=st.active_components, structure_bottleneck_dim=st.bottleneck_dim, structure_num_categories=st.num_categories,
        structure_max_dep_level=st.max_dep_level, structure_max_ast_depth=st.max_ast_depth,
        structure_max_sibling_index=st.max_sibling_index, structure_num_node_types=st.num_node_types,
        moe_num_experts=config.moe.num_experts, moe_top_k=config.moe.top_k, moe_expert_hidden_size=config.moe.ffn_hidden_size,
        moe_shared_expert_hidden_size=config.moe.shared_expert_intermediate_size, mamba_expand=config.mamba3.expand,
        mamba_head_dim=config.mamba3.head_dim, mamba_state_dim=config.mamba3.state_dim, mamba_groups=config.mamba3.num_groups,
        mamba_mimo_rank=config.mamba3.mimo_rank, mamba_is_mimo=config.mamba3.is_mimo, mamba_chunk_size=config.mamba3.chunk_size,
        mamba_rope_fraction=config.mamba3.rope_fraction, m2rnn_k_head_dim=config.m2rnn.k_head_dim,
        m2rnn_v_head_dim=config.m2rnn.v_head_dim, m2rnn_chunk_size=config.m2rnn.runtime_bwd_chunk_size,
        ngram_hash_enabled=nh.enabled, ngram_hash_orders=nh.orders, ngram_hash_heads=nh.num_heads, ngram_hash_table_size=nh.table_size,
        ngram_hash_embed_dim=nh.embed_dim, ngram_hash_dropout=nh.dropout, ngram_hash_seed=nh.seed)
    params.update(overrides)
    return HybridTinyConfig(**params)


REFERENCE_PATTERN = DEFAULT_NAM56R_PATTERN
REFERENCE_DEPTH = DEFAULT_NAM56R_DEPTH
REFERENCE_DSA_A_LAYER_RANKS = DEFAULT_DSA_A_LAYER_RANKS

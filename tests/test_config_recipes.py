"""Typed configuration tree, layer-pattern expansion, the NAM56R recipe and the model-factory profiles (CPU, no model weights
beyond a tiny derived model)."""
import dataclasses

import pytest
import torch

from cppmega_mlx_b200.config import model as C
from cppmega_mlx_b200.recipes import model_factory as mf
from cppmega_mlx_b200.recipes import nam56r as N
from cppmega_mlx_b200.recipes import pattern as P


# ----------------------------------------------------------------------------------------------- pattern
def test_pattern_expansion_numbers_layers_and_routes_attention():
    ex = P.expand_nam_pattern("AEMR", 10, dsa_a_layer_ranks=(0, 2))
    assert ex.symbols == tuple("AEMRAEMRAE") and ex.depth == 10 and ex.layer_numbers == tuple(range(1, 11))
    assert ex.a_layer_numbers == (1, 5, 9) and ex.r_layer_numbers == (4, 8) and ex.mamba3_layer_numbers == (3, 7)
    assert ex.moe_layer_numbers == (2, 6, 10) and ex.engram_layer_numbers == () and ex.concept_layer_numbers == ()
    assert ex.dsa_layer_numbers == (1, 9) and ex.mla_layer_numbers == (5,)               # A ranks 0 and 2 are sparse, rank 1 dense
    assert [l.a_rank for l in ex.layers if l.symbol == "A"] == [0, 1, 2]
    assert ex.counts == {"A": 3, "E": 3, "M": 2, "R": 2, "N": 0, "C": 0}
    assert ex.role_counts["attention"] == 3 and ex.layer_numbers_for_role("m2rnn") == (4, 8)
    assert ex.attention_route_for_layer(5) == "mla" and ex.attention_route_for_layer(2) is None
    with pytest.raises(ValueError, match="outside expanded depth"):
        ex.attention_route_for_layer(11)
    with pytest.raises(ValueError, match="unsupported NAM layer role"):
        ex.layer_numbers_for_role("conv")
    assert P.layer_numbers_for_symbol("AEMR", 10, "E") == (2, 6, 10)
    assert P.a_layer_numbers("AEMR", 10) == (1, 5, 9) and P.r_layer_numbers("AEMR", 10) == (4, 8)
    assert P.expand_symbols("AM", 5) == tuple("AMAMA")
    assert P.parse_nam_pattern(" ame ") == ("A", "M", "E")       # case-insensitive, surrounding blanks ignored
    with pytest.raises(ValueError, match="invalid NAM pattern chars"):
        P.parse_nam_pattern("A|M")                               # the upstream separators are not part of the alphabet
    with pytest.raises(TypeError):
        P.parse_nam_pattern(7)


def test_pattern_rejects_bad_input():
    with pytest.raises(ValueError):
        P.parse_nam_pattern("AXM")                            # X is not in the alphabet
    with pytest.raises(ValueError):
        P.parse_nam_pattern("")
    with pytest.raises(ValueError):
        P.expand_symbols("AM", 0)
    with pytest.raises(ValueError):
        P.expand_nam_pattern("AM", 4, dsa_a_layer_ranks=(5,))     # only two A layers exist
    assert P.parse_rank_list("0, 2,3") == (0, 2, 3) and P.parse_rank_list([1, 4]) == (1, 4) and P.parse_rank_list("") == ()
    with pytest.raises(ValueError):
        P.parse_rank_list("1,1")
    with pytest.raises(ValueError):
        P.parse_rank_list("-1")


# ----------------------------------------------------------------------------------------------- config tree
def test_config_tree_round_trips_through_a_dict():
    cfg = N.build_nam56r_config(hidden_size=512, num_attention_heads=8, depth=12, seq_len=256, max_position_embeddings=512,
                                mamba3=C.Mamba3Config(d_model=512, num_groups=4), moe=C.MoeConfig(num_experts=8, top_k=2),
                                dsa=C.DSAConfig(a_layer_ranks=(0,), indexer_topk=64), ngram_hash=C.NgramHashConfig(enabled=True, orders=(2, 4)))
    d = cfg.to_dict()
    assert d["mamba3"]["num_groups"] == 4 and d["dsa"]["a_layer_ranks"] == (0,) and d["m2rnn"]["d_model"] == 512
    import json
    again = C.config_from_dict(C.Nam56RModelConfig, json.loads(json.dumps(d)))        # tuples come back from JSON as lists
    assert again == cfg and isinstance(again.ngram_hash.orders, tuple) and isinstance(again.moe, C.MoeConfig)
    assert cfg.head_dim == 64 and cfg.vocab_size == cfg.vocab.default_model_vocab_size
    assert cfg.mamba3.native_num_heads == 8 and cfg.mamba3.author_num_heads == 16
    with pytest.raises(dataclasses.FrozenInstanceError):
        cfg.depth = 3


@pytest.mark.parametrize("build,match", [
    (lambda: C.MoeConfig(top_k=32, num_experts=16), "top_k must be <= num_experts"),
    (lambda: C.MoeConfig(token_dispatcher_type="ring"), "token_dispatcher_type"),
    (lambda: C.MoeConfig(token_dispatcher_type="flex", router_dtype=None), "requires router_dtype"),
    (lambda: C.MoeConfig(num_experts=10, expert_model_parallel_size=4), "divisible by expert_model_parallel_size"),
    (lambda: C.M2RNNConfig(runtime_kernel="metal"), "runtime_kernel"),
    (lambda: C.M2RNNConfig(a_init_min=2.0, a_init_max=1.0), "a_init_min"),
    (lambda: C.M2RNNConfig(gradient_clipping=0.0), "gradient_clipping"),
    (lambda: C.Mamba3Config(d_model=100, head_dim=64), "divisible by Mamba3 head_dim"),
    (lambda: C.Mamba3Config(rope_fraction=1.5), "rope_fraction"),
    (lambda: C.Mamba3Config(dt_min=1.0, dt_max=0.1), "dt_min"),
    (lambda: C.MLAConfig(q_lora_rank=0), "must be positive"),
    (lambda: C.DSAConfig(a_layer_ranks=(1, 1)), "unique"),
    (lambda: C.DSAConfig(a_layer_ranks=(-1,)), "non-negative"),
    (lambda: C.DSAConfig(indexer_dtype="fp8"), "indexer_dtype"),
    (lambda: C.NgramHashConfig(orders=()), "at least one order"),
    (lambda: C.NgramHashConfig(dropout=1.0), "dropout"),
    (lambda: C.StructureConfig(active_components="structure,bogus"), "unknown structure components"),
    (lambda: C.VocabMetadata(default_model_vocab_size=123), "preserved vocab contract"),
    (lambda: C.Nam56RModelConfig(hidden_size=100, num_attention_heads=8), "divisible by num_attention_heads"),
    (lambda: C.Nam56RModelConfig(seq_len=4096, max_position_embeddings=1024), "max_position_embeddings"),
    (lambda: C.Nam56RModelConfig(m2rnn=C.M2RNNConfig(d_model=8)), "M2RNN d_model"),
])
def test_config_validation_messages(build, match):
    with pytest.raises(ValueError, match=match):
        build()


def test_structure_component_parsing():
    assert C.parse_structure_components("core") == ("structure", "dep_level")
    assert len(C.parse_structure_components("all")) == 5
    assert C.parse_structure_components(" ast_depth , structure ") == ("structure", "ast_depth")     # canonical order
    with pytest.raises(TypeError):
        C.parse_structure_components(3)
    with pytest.raises(ValueError, match="at least one"):
        C.parse_structure_components(" , ")
    assert C.StructureConfig(active_components="all").component_names[-1] == "ast_node_type"
    assert C.SourceStructureEnvConfig().component_names == ("structure", "dep_level")


# ----------------------------------------------------------------------------------------------- NAM56R recipe
def test_nam56r_recipe_contract_and_derived_model_config():
    cfg = N.default_nam56r_config()
    ex = N.build_nam56r_pattern(cfg)
    assert ex.depth == cfg.depth and set(ex.symbols) <= set("AEMR")
    contract = N.build_nam56r_parity_contract(cfg)
    assert contract.megatron_fully_native is False and "m2rnn" in contract.custom_megatron_roles
    with pytest.raises(NotImplementedError, match="does not claim fully native"):
        N.require_fully_native_megatron_parity(cfg)
    first_a = ex.a_layer_numbers[0]
    assert N.attention_route_for_layer(first_a, cfg) in ("dsa", "mla")
    with pytest.raises(ValueError, match="outside the pattern"):
        N.attention_route_for_layer(cfg.depth + 1, cfg)
    moved = N.with_dsa_a_layer_ranks(cfg, "0,1")
    assert moved.dsa.a_layer_ranks == (0, 1) and cfg.dsa.a_layer_ranks != (0, 1)             # a copy, the original is frozen
    assert N.build_nam56r_pattern(moved).dsa_layer_numbers == ex.a_layer_numbers[:2]
    short = N.build_nam56r_pattern(N.with_dsa_a_layer_ranks(cfg, (1,)), pattern="AM", depth=4)
    assert short.symbols == tuple("AMAM") and short.dsa_layer_numbers == (3,)
    with pytest.raises(ValueError, match="exceed zero-based A-layer range"):
        N.build_nam56r_pattern(cfg, pattern="AM", depth=4)                                    # the default ranks name A layers this short stack lacks
    tiny = N.build_hybrid_tiny_config_from_nam56r(N.build_nam56r_config(hidden_size=64, num_attention_heads=4, depth=4, seq_len=32,
                                                                        max_position_embeddings=32, pattern="AMER",
                                                                        mamba3=C.Mamba3Config(d_model=64, head_dim=16, num_groups=2, state_dim=8,
                                                                                              chunk_size=8),
                                                                        m2rnn=C.M2RNNConfig(d_model=64, k_head_dim=8, v_head_dim=8),
                                                                        moe=C.MoeConfig(num_experts=4, top_k=2, ffn_hidden_size=16,
                                                                                        shared_expert_intermediate_size=16),
                                                                        dsa=C.DSAConfig(a_layer_ranks=())), vocab_size=128)
    assert tiny.hidden_size == 64 and tiny.depth == 4 and tiny.pattern == "AMER" and tiny.vocab_size == 128
    assert tiny.moe_num_experts == 4 and tiny.mamba_groups == 2 and tiny.m2rnn_k_head_dim == 8
    with pytest.raises(ValueError, match="divisible by num_attention_heads"):
        N.build_nam56r_config(hidden_size=100, num_attention_heads=8)


# ----------------------------------------------------------------------------------------------- model factory
def test_model_factory_profiles_are_consistent():
    names = mf.list_model_profiles()
    assert {"local_gb10_quarter", "hybrid_1b", "moe_hybrid_ep8", "nam56r_56l"} <= set(names)
    with pytest.raises(ValueError, match="unknown model factory profile"):
        mf.get_model_profile("does_not_exist")
    for name in names:
        prof = mf.get_model_profile(name)
        cfg = prof.hybrid_config()
        assert cfg.hidden_size % cfg.num_attention_heads == 0
        assert len(cfg.expanded_pattern().symbols) == cfg.depth
        smaller = prof.hybrid_config(depth=2, max_seq_length=64, dsa_a_layer_ranks=())      # ranks pinned to A layers a short stack lacks are refused
        assert smaller.depth == 2 and smaller.max_seq_length == 64 and smaller.hidden_size == cfg.hidden_size
    one_b = mf.get_model_profile("hybrid_1b").hybrid_config()
    assert one_b.pattern.count("M") == 3 * one_b.pattern.count("A") and one_b.hidden_size == 2048 and one_b.vocab_size == 65536


def test_tiny_smoke_model_builds_and_steps_on_cpu():
    m = mf.build_local_gb10_quarter_tiny_smoke_model()
    ids = torch.randint(0, m.config.vocab_size, (2, 9))
    out = m(ids)
    assert out.shape[:2] == (2, 9) and torch.isfinite(out).all()
    assert m.num_parameters() == sum(p.numel() for p in m.parameters())
    assert m.num_parameters(trainable_only=True) <= m.num_parameters()

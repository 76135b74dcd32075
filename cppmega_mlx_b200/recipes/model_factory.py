"""Named model profiles and the factory that turns them into models.

Reference profiles (``cppmega_mlx/recipes/model_factory.py:27-58``): ``local_gb10_quarter`` (pattern
AEMEAEMEAEMR, depth 13, hidden 3584, 28 heads × 128, vocab 65536, DSA ranks (1,2,3), MTP depth 2) and
``nam56r_full`` (depth 52, hidden 4096).  Production-shaped profiles for the B200 benchmarks:

* ``hybrid_1b``      — 24 layers ``[M,M,M,A]``, d_model 2048, sparse MLA (16 heads, q_lora 1536, kv_lora 512,
                        rope 64, indexer 4×64, top-2048), Mamba3 (state 128, head 64, expand 2, chunk 256),
                        SwiGLU 5632 in every layer, MTP depth 1, vocab 65536;
* ``moe_hybrid_ep8`` — 16 layers ``[M,E,A,E]``, 64 routed experts top-6 + 2 shared, hidden 1408, sigmoid
                        aux-free router;
* ``nam56r_56l``     — 56 layers ``[M,M,M,A,M,E,M,R]``×7, d_model 3584, vocab 131072.
"""
from __future__ import annotations

from dataclasses import dataclass, field, replace
from typing import Any

import torch

from ..config.model import DSAConfig, MLAConfig, Mamba3Config, M2RNNConfig, MoeConfig, Nam56RModelConfig, VocabMetadata
from ..data.tokenizer_contract import REQUIRED_SPECIAL_TOKEN_IDS
from ..models.hybrid_lm import HybridTinyConfig, HybridTinyLM
from .pattern import ExpandedNamPattern, expand_nam_pattern

LOCAL_GB10_QUARTER_PROFILE = "local_gb10_quarter"
NAM56R_FULL_PROFILE = "nam56r_full"
HYBRID_1B_PROFILE = "hybrid_1b"
MOE_HYBRID_EP8_PROFILE = "moe_hybrid_ep8"
NAM56R_56L_PROFILE = "nam56r_56l"


@dataclass(frozen=True)
class MTPProfile:
    enabled: bool = True
    depth: int = 2
    beta: float = 0.6
    loss_weight: float = 0.3


@dataclass(frozen=True)
class TokenizerContractStatus:
    required_specials: tuple[tuple[str, int], ...] = tuple(REQUIRED_SPECIAL_TOKEN_IDS.items())
    vocab_size: int = 65_536


@dataclass(frozen=True)
class ModelFactoryProfile:
    name: str
    pattern: str
    depth: int
    hidden_size: int
    ffn_hidden_size: int
    num_attention_heads: int
    head_dim: int
    vocab_size: int
    max_seq_length: int = 4096
    dsa_a_layer_ranks: tuple[int, ...] = (1, 2, 3)
    dsa_indexer_n_heads: int | None = 32
    dsa_indexer_head_dim: int | None = 64
    dsa_topk: int = 256
    moe_num_experts: int = 16
    moe_top_k: int = 4
    moe_expert_hidden_size: int = 896
    moe_shared_expert_hidden_size: int = 1024
    mtp: MTPProfile = MTPProfile()
    tokenizer_contract: TokenizerContractStatus = TokenizerContractStatus()
    model_kind: str = "hybrid_tiny"
    upstream_recipe_module: str = "cppmega.recipes.run_profiles"
    upstream_recipe_name: str | None = None
    hybrid_overrides: tuple[tuple[str, Any], ...] = ()

    def __post_init__(self) -> None:
        for n in ("depth", "hidden_size", "ffn_hidden_size", "num_attention_heads", "head_dim", "vocab_size",
                  "max_seq_length", "moe_num_experts", "moe_top_k", "moe_expert_hidden_size",
                  "moe_shared_expert_hidden_size"):
            if getattr(self, n) <= 0:
                raise ValueError(f"{n} must be positive")
        if self.moe_top_k > self.moe_num_experts:
            raise ValueError("moe_top_k must be <= moe_num_experts")
        if self.dsa_a_layer_ranks and (not self.dsa_indexer_n_heads or not self.dsa_indexer_head_dim):
            raise ValueError("DSA A-layer ranks require DSA indexer dimensions")
        if self.model_kind != "hybrid_tiny":
            raise ValueError(f"unsupported model_kind={self.model_kind!r}")
        self.expanded_pattern

    @property
    def expanded_pattern(self) -> ExpandedNamPattern:
        return expand_nam_pattern(self.pattern, self.depth, dsa_a_layer_ranks=self.dsa_a_layer_ranks)

    def nam56r_config(self) -> Nam56RModelConfig:
        vs = self.vocab_size
        vocab = VocabMetadata(local_profile_vocab_size=vs if vs != 131_072 else 65_536,
                              megacpp_tokenizer_vocab_size=131_072 if vs != 131_072 or True else vs,
                              default_model_vocab_size=vs if vs in (65_536, 131_072) else vs) \
            if vs in (65_536, 131_072) else VocabMetadata(local_profile_vocab_size=vs, default_model_vocab_size=vs)
        return Nam56RModelConfig(
            pattern=self.pattern, depth=self.depth, hidden_size=self.hidden_size, ffn_hidden_size=self.ffn_hidden_size,
            num_attention_heads=self.num_attention_heads, seq_len=self.max_seq_length,
            max_position_embeddings=self.max_seq_length, vocab=vocab,
            moe=MoeConfig(num_experts=self.moe_num_experts, top_k=self.moe_top_k, ffn_hidden_size=self.moe_expert_hidden_size,
                          shared_expert_intermediate_size=self.moe_shared_expert_hidden_size),
            m2rnn=M2RNNConfig(d_model=self.hidden_size), mamba3=Mamba3Config(d_model=self.hidden_size),
            mla=MLAConfig(), dsa=DSAConfig(a_layer_ranks=self.dsa_a_layer_ranks,
                                           indexer_n_heads=self.dsa_indexer_n_heads or 32,
                                           indexer_head_dim=self.dsa_indexer_head_dim or 64, indexer_topk=self.dsa_topk))

    def hybrid_config(self, **overrides) -> HybridTinyConfig:
        base = dict(
            vocab_size=self.vocab_size, hidden_size=self.hidden_size, pattern=self.pattern, depth=self.depth,
            dsa_a_layer_ranks=self.dsa_a_layer_ranks, num_attention_heads=self.num_attention_heads,
            attention_sparse_topk=self.dsa_topk, max_seq_length=self.max_seq_length,
            moe_num_experts=self.moe_num_experts, moe_top_k=self.moe_top_k,
            moe_expert_hidden_size=self.moe_expert_hidden_size,
            moe_shared_expert_hidden_size=self.moe_shared_expert_hidden_size,
            mamba_head_dim=64, mamba_state_dim=64, mamba_groups=8, mamba_conv_kernel=4, mamba_chunk_size=64,
            m2rnn_k_head_dim=64, m2rnn_v_head_dim=16, m2rnn_num_v_heads=4, m2rnn_num_f_heads=4, m2rnn_num_g_heads=4,
            mtp_enabled=self.mtp.enabled, mtp_depth=self.mtp.depth, mtp_decay=self.mtp.beta,
            mtp_loss_weight=self.mtp.loss_weight, dsa_indexer_heads=self.dsa_indexer_n_heads or 4,
            dsa_indexer_head_dim=self.dsa_indexer_head_dim or 64)
        base.update(dict(self.hybrid_overrides))
        base.update(overrides)
        return HybridTinyConfig(**base)

    def tiny_smoke_config(self, **overrides) -> HybridTinyConfig:
        """Same routing (pattern, DSA ranks, MTP) at toy width, for CPU tests."""
        small = dict(vocab_size=128, hidden_size=64, depth=min(self.depth, len(self.pattern)), num_attention_heads=4,
                     max_seq_length=64, attention_sparse_topk=8, moe_num_experts=4, moe_top_k=2, moe_expert_hidden_size=32,
                     moe_shared_expert_hidden_size=16, mamba_head_dim=16, mamba_state_dim=8, mamba_groups=2,
                     mamba_chunk_size=8, m2rnn_k_head_dim=8, m2rnn_v_head_dim=4, ffn_hidden_size=0,
                     mla_q_lora_rank=32, mla_kv_lora_rank=32, mla_qk_nope_head_dim=16, mla_qk_rope_head_dim=8,
                     mla_v_head_dim=16, dsa_indexer_head_dim=16, dsa_indexer_heads=2)
        small["dsa_a_layer_ranks"] = tuple(r for r in self.dsa_a_layer_ranks
                                           if r < expand_nam_pattern(self.pattern, small["depth"]).symbols.count("A"))
        small.update(overrides)
        return self.hybrid_config(**small)

    def build_model(self, *, dtype: torch.dtype | None = torch.bfloat16, device=None, ep_group=None, **overrides) -> HybridTinyLM:
        cfg = self.hybrid_config(**overrides)
        if device is not None:
            with torch.device(device):
                model = HybridTinyLM(cfg, ep_group=ep_group)
        else:
            model = HybridTinyLM(cfg, ep_group=ep_group)
        return model.to(dtype) if dtype is not None else model


def local_gb10_quarter_profile() -> ModelFactoryProfile:
    return ModelFactoryProfile(LOCAL_GB10_QUARTER_PROFILE, "AEMEAEMEAEMR", 13, 3584, 18_944, 28, 128, 65_536,
                               upstream_recipe_name="local_gb10_quarter")


def nam56r_full_profile() -> ModelFactoryProfile:
    return ModelFactoryProfile(NAM56R_FULL_PROFILE, "AEMEAEMEAEMR", 52, 4096, 21_504, 32, 128, 65_536,
                               dsa_a_layer_ranks=(1, 2, 3, 5, 6, 7, 9, 10, 11), upstream_recipe_name="h200_dsa_9_4_m")


_MLA = (("mla_low_rank", True), ("mla_q_lora_rank", 1536), ("mla_kv_lora_rank", 512), ("mla_qk_nope_head_dim", 128),
        ("mla_qk_rope_head_dim", 64), ("mla_v_head_dim", 128), ("dsa_all_a_layers", True), ("position_embedding", False),
        ("mamba_state_dim", 128), ("mamba_head_dim", 64), ("mamba_expand", 2), ("mamba_chunk_size", 256), ("mamba_groups", 8))


def hybrid_1b_profile() -> ModelFactoryProfile:
    return ModelFactoryProfile(HYBRID_1B_PROFILE, "MMMA", 24, 2048, 5632, 16, 128, 65_536, dsa_a_layer_ranks=(),
                               dsa_indexer_n_heads=4, dsa_indexer_head_dim=64, dsa_topk=2048,
                               mtp=MTPProfile(True, 1, 0.6, 0.3),
                               hybrid_overrides=_MLA + (("ffn_hidden_size", 5632),))


def moe_hybrid_ep8_profile() -> ModelFactoryProfile:
    return ModelFactoryProfile(MOE_HYBRID_EP8_PROFILE, "MEAE", 16, 2048, 5632, 16, 128, 65_536, dsa_a_layer_ranks=(),
                               dsa_indexer_n_heads=4, dsa_indexer_head_dim=64, dsa_topk=2048, moe_num_experts=64, moe_top_k=6,
                               moe_expert_hidden_size=1408, moe_shared_expert_hidden_size=1408, mtp=MTPProfile(False, 1),
                               hybrid_overrides=_MLA + (("moe_scoring", "sigmoid"), ("moe_aux_loss_free", True),
                                                        ("moe_num_shared_experts", 2), ("moe_activation", "swiglu")))


def nam56r_56l_profile() -> ModelFactoryProfile:
    return ModelFactoryProfile(NAM56R_56L_PROFILE, "MMMAMEMR", 56, 3584, 18_944, 28, 128, 131_072, max_seq_length=8192,
                               dsa_a_layer_ranks=(), dsa_indexer_n_heads=4, dsa_indexer_head_dim=64, dsa_topk=2048,
                               moe_num_experts=32, moe_top_k=4, moe_expert_hidden_size=2048, moe_shared_expert_hidden_size=2048,
                               mtp=MTPProfile(True, 1, 0.6, 0.3),
                               hybrid_overrides=_MLA + (("m2rnn_k_head_dim", 64), ("m2rnn_v_head_dim", 128),
                                                        ("m2rnn_num_v_heads", 28), ("m2rnn_num_f_heads", 28),
                                                        ("m2rnn_num_g_heads", 28), ("m2rnn_num_q_heads", 28),
                                                        ("m2rnn_num_k_heads", 28)))


_PROFILES = {LOCAL_GB10_QUARTER_PROFILE: local_gb10_quarter_profile, NAM56R_FULL_PROFILE: nam56r_full_profile,
             HYBRID_1B_PROFILE: hybrid_1b_profile, MOE_HYBRID_EP8_PROFILE: moe_hybrid_ep8_profile,
             NAM56R_56L_PROFILE: nam56r_56l_profile}


def get_model_profile(name: str) -> ModelFactoryProfile:
    if name not in _PROFILES:
        raise ValueError(f"unknown model factory profile {name!r}; supported: {', '.join(_PROFILES)}")
    return _PROFILES[name]()


def list_model_profiles() -> tuple[str, ...]:
    return tuple(_PROFILES)


def local_gb10_quarter(*, dtype: torch.dtype | None = torch.bfloat16, device=None, **hybrid_config_overrides) -> HybridTinyLM:
    """Allocates the full ~2 B-parameter model; tests should use ``tiny_smoke_config`` instead."""
    return local_gb10_quarter_profile().build_model(dtype=dtype, device=device, **hybrid_config_overrides)


def build_local_gb10_quarter_tiny_smoke_model(**overrides) -> HybridTinyLM:
    return HybridTinyLM(local_gb10_quarter_profile().tiny_smoke_config(**overrides))

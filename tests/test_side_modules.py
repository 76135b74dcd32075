"""Side modules of the model stack and the measurement / sweep helpers, on CPU: structure embedding, n-gram hash embedding,
concept block, the byte-fallback tokenizer, the MTP speculative adapter, the clock sampler's parser and the sweep summary."""
import json
import math

import pytest
import torch


# ----------------------------------------------------------------------------------------------- structure embedding
def test_structure_embedding_channels_offsets_and_absent_inputs():
    from cppmega_mlx_b200.nn.structure_embedding import StructureEmbedding
    torch.manual_seed(0)
    se = StructureEmbedding(hidden_size=24, num_categories=5, max_dep_level=4, active_components="all", bottleneck_dim=8)
    assert se.active_component_names == StructureEmbedding.ALL_COMPONENTS
    assert se._comp_offsets.tolist() == [0, 5, 9, 73, 137] and se.stacked_emb.weight.shape[0] == 137 + 256
    # both tables start at zero: the module adds nothing before training
    ids = torch.randint(0, 4, (2, 7))
    assert float(se(structure_ids=ids, dep_levels=ids).abs().max()) == 0.0
    assert se().dim() == 0                                    # no channel given: a scalar zero that broadcasts in `h + …`
    with torch.no_grad():
        se.stacked_emb.weight.normal_()
        se.up_proj.weight.normal_()
    full = se(structure_ids=ids, dep_levels=ids)
    only_structure = se(structure_ids=ids)
    only_dep = se(dep_levels=ids)
    assert full.shape == (2, 7, 24)
    assert torch.allclose(full, only_structure + only_dep, atol=1e-5)          # channels are blended linearly
    # ids are clamped to the channel's range: 99 reads the last dependency level, negatives the first
    hi = se(dep_levels=torch.full((1, 3), 99))
    last = se(dep_levels=torch.full((1, 3), 3))
    assert torch.equal(hi, last)
    assert torch.equal(se(dep_levels=torch.full((1, 3), -5)), se(dep_levels=torch.zeros(1, 3, dtype=torch.long)))
    # manual evaluation of one position
    row = se.stacked_emb.weight[5 + 3] * se.component_scales[1]
    assert torch.allclose(last[0, 0], row @ se.up_proj.weight.t(), atol=1e-5)


def test_structure_embedding_validation():
    from cppmega_mlx_b200.nn.structure_embedding import StructureEmbedding
    with pytest.raises(ValueError, match="unknown structure components"):
        StructureEmbedding(hidden_size=8, active_components="structure,nope")
    with pytest.raises(ValueError, match="at least one"):
        StructureEmbedding(hidden_size=8, active_components=" , ")
    with pytest.raises(ValueError, match="positive"):
        StructureEmbedding(hidden_size=0)
    se = StructureEmbedding(hidden_size=8, active_components="structure,ast_depth")
    assert se.active_component_names == ("structure", "ast_depth")
    with pytest.raises(ValueError, match="rank 2"):
        se(structure_ids=torch.zeros(3, dtype=torch.long))
    with pytest.raises(ValueError, match="does not match"):
        se(structure_ids=torch.zeros(2, 3, dtype=torch.long), ast_depth_ids=torch.zeros(2, 4, dtype=torch.long))


# ----------------------------------------------------------------------------------------------- n-gram hash embedding
def test_ngram_hash_is_causal_deterministic_and_in_range():
    from cppmega_mlx_b200.nn.ngram_hash import NgramHashEmbedding, pick_primes
    assert len(set(pick_primes(16, 500_000))) == 16
    assert pick_primes(3, 100) == (100, 101, 102)             # no listed prime near the target: consecutive sizes
    a = NgramHashEmbedding(hidden_size=16, orders=(2, 3), num_heads=2, table_size=500_000, embed_dim=4, seed=7)
    b = NgramHashEmbedding(hidden_size=16, orders=(2, 3), num_heads=2, table_size=500_000, embed_dim=4, seed=7)
    c = NgramHashEmbedding(hidden_size=16, orders=(2, 3), num_heads=2, table_size=500_000, embed_dim=4, seed=8)
    ids = torch.randint(0, 65536, (2, 11))
    ha, hb, hc = a._hash_all(ids), b._hash_all(ids), c._hash_all(ids)
    assert ha.shape == (2, 4, 11) and torch.equal(ha, hb) and not torch.equal(ha, hc)
    lo = a.table_offsets[None, :, None]
    assert bool(((ha >= lo) & (ha < lo + a.table_sizes_t[None, :, None])).all())
    # a position's rows depend on the last `order` tokens only: changing token 0 leaves positions ≥ 3 alone (orders 2 and 3)
    ids2 = ids.clone()
    ids2[:, 0] += 1
    h2 = a._hash_all(ids2)
    assert torch.equal(ha[:, :, 3:], h2[:, :, 3:]) and not torch.equal(ha[:, :, 0], h2[:, :, 0])
    # the order-2 tables ignore the token two places back, the order-3 tables see it
    ids3 = ids.clone()
    ids3[:, 4] += 1
    h3 = a._hash_all(ids3)
    assert torch.equal(ha[:, :2, 6], h3[:, :2, 6]) and not torch.equal(ha[:, 2:, 6], h3[:, 2:, 6])
    out = a(ids)
    assert out.shape == (2, 11, 16) and float(out.abs().max()) == 0.0          # zero-initialised projection
    with pytest.raises(ValueError):
        NgramHashEmbedding(hidden_size=16, orders=())
    with pytest.raises(ValueError):
        a._hash_all(torch.zeros(5, dtype=torch.long))


# ----------------------------------------------------------------------------------------------- concept block
def test_concept_block_matches_manual_cross_attention():
    from cppmega_mlx_b200.nn.concept import ConceptBlock, ConceptBlockConfig
    torch.manual_seed(0)
    cfg = ConceptBlockConfig(hidden_size=16, num_concepts=5, concept_dim=12, num_heads=4)
    blk = ConceptBlock(cfg)
    x = torch.randn(2, 6, 16)
    assert float(blk(x).abs().max()) == 0.0                   # zero-initialised output projection
    with torch.no_grad():
        blk.out_proj.weight.normal_(std=0.3)
    y = blk(x)
    xn = x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + cfg.eps)
    q = (xn @ blk.q_proj.weight.t()).view(2, 6, 4, 4)
    bank = blk.concept_bank.weight
    k = (bank @ blk.k_proj.weight.t()).view(5, 4, 4)
    v = (bank @ blk.v_proj.weight.t()).view(5, 4, 4)
    out = torch.zeros(2, 6, 4, 4)
    for h in range(4):
        w = torch.softmax(q[:, :, h] @ k[:, h].t() / math.sqrt(4), -1)         # [2, 6, 5]: no causal mask, concepts are global
        out[:, :, h] = w @ v[:, h]
    assert torch.allclose(y, out.reshape(2, 6, 16) @ blk.out_proj.weight.t(), atol=1e-5)
    # permuting the sequence permutes the output: positions do not interact
    perm = torch.randperm(6)
    assert torch.allclose(blk(x[:, perm]), y[:, perm], atol=1e-6)
    with pytest.raises(ValueError, match="divisible"):
        ConceptBlockConfig(hidden_size=10, num_heads=4)
    with pytest.raises(ValueError, match="shaped"):
        blk(torch.randn(2, 6, 8))


# ----------------------------------------------------------------------------------------------- tokenizer
def test_byte_fallback_tokenizer_contract_and_round_trip():
    from cppmega_mlx_b200.data.tokenizer_contract import REQUIRED_SPECIAL_TOKEN_IDS
    from cppmega_mlx_b200.tokenizer.cpp_tokenizer import CppMegaTokenizer, TokenizerContractError, build_byte_fallback_tokenizer
    tok = build_byte_fallback_tokenizer()
    for name, want in REQUIRED_SPECIAL_TOKEN_IDS.items():
        assert tok.id_for_token(name) == want
    assert tok.bos_token_id == REQUIRED_SPECIAL_TOKEN_IDS["<BOS>"] and tok.nl_token_id == REQUIRED_SPECIAL_TOKEN_IDS["<NL>"]
    src = "int main() {\n\n    return 0;\n}"
    ids = tok.encode(src)
    # runs of newlines / blanks collapse to one sentinel each, so decoding gives the normalised text
    assert tok.decode(ids) == "int main() {\n return 0;\n}"
    assert ids.count(tok.nl_token_id) == 2 and ids.count(tok.space_token_id) == 4
    wrapped = tok.encode("x", prepend="<BOS>", append=tok.eos_token_id)
    assert wrapped[0] == tok.bos_token_id and wrapped[-1] == tok.eos_token_id and len(wrapped) == 3
    assert tok.encode(["a", "b c"]) == [tok.encode("a"), tok.encode("b c")]
    assert tok.encode_batch(["a b"]) == [tok.encode("a b")]
    assert tok("a") == tok.encode("a")
    assert tok.token_for_id(tok.id_for_token("a")) == "a" and tok.id_for_token("no such token") is None
    with pytest.raises(TokenizerContractError, match="unknown special token"):
        tok.encode("x", prepend="<NOPE>")
    with pytest.raises(TypeError):
        tok.encode(5)
    with pytest.raises(TokenizerContractError, match="vocab size"):
        tok.validate_contract(check_vocab_size=True)

    class Broken:                                              # a vocabulary whose <BOS> sits at the wrong id
        def get_vocab(self):
            v = dict(tok._vocab)
            v["<BOS>"] = 47
            return v

        def get_vocab_size(self, with_added_tokens=True):
            return 10
    with pytest.raises(TokenizerContractError, match="<BOS>"):
        CppMegaTokenizer(Broken())
    assert CppMegaTokenizer(Broken(), strict=False).vocab_size == 10


def test_tokenizer_loader_reads_a_saved_file(tmp_path):
    from cppmega_mlx_b200.tokenizer.cpp_tokenizer import build_byte_fallback_tokenizer, load_cppmega_tokenizer
    tok = build_byte_fallback_tokenizer()
    tok._tok.save(str(tmp_path / "tokenizer.json"))
    again = load_cppmega_tokenizer(tmp_path)                  # a directory resolves to its tokenizer.json
    assert again.encode("a+b") == tok.encode("a+b") and again.path == tmp_path / "tokenizer.json"
    with pytest.raises(FileNotFoundError):
        load_cppmega_tokenizer(tmp_path / "missing")


# ----------------------------------------------------------------------------------------------- MTP speculative adapter
def test_mtp_adapter_drafts_depth_tokens_greedily():
    from cppmega_mlx_b200.v4.mtp_adapter import MTPSpeculativeAdapter

    class Head:
        class config:
            depth = 3

        def __init__(self):
            self.calls = []

        def draft_step(self, k, h, tok):
            # logits that make token (previous token + k + 1) mod 11 the arg-max, hidden passed on unchanged
            self.calls.append((k, tuple(tok[:, 0].tolist())))
            lg = torch.zeros(tok.shape[0], 1, 11)
            lg[torch.arange(tok.shape[0]), 0, (tok[:, 0] + k + 1) % 11] = 5.0
            return lg, h

    class Model:
        pass
    m = Model()
    with pytest.raises(ValueError, match="no sequential MTP head"):
        MTPSpeculativeAdapter(m)
    m.mtp_head = Head()
    ad = MTPSpeculativeAdapter(m)
    toks, logits = ad.draft(torch.randn(2, 8), torch.tensor([1, 9]))
    assert ad.depth == 3 and toks.shape == (2, 3) and logits.shape == (2, 3, 11)
    assert toks.tolist() == [[2, 4, 7], [10, 1, 4]]           # each draft feeds the next depth
    assert [c[0] for c in m.mtp_head.calls] == [0, 1, 2] and m.mtp_head.calls[1][1] == (2, 10)


# ----------------------------------------------------------------------------------------------- measurement helpers
def test_clock_sampler_parses_samples_and_reasons():
    from cppmega_mlx_b200.utils.measure import ClockSampler, measured_peaks

    class Done:
        def terminate(self):
            pass

        def wait(self, timeout=None):
            return 0
    s = ClockSampler(0)
    assert s.stop()["reasons"] == ["nvidia-smi unavailable"]   # never started (no nvidia-smi on this machine)
    s.proc = Done()
    s.lines = ["1500, 1965, 990.1, 0x4, Not Active, Not Active, Not Active, Active",
               "1700, 1965, 995.0, 0x4, Not Active, Not Active, Not Active, Active",
               "1600, 1965, 700.0, 0x0, Not Active, Not Active, Not Active, Not Active",
               "garbage line", "N/A, 1965, 1, 0, Not Active, Active, Not Active, Not Active"]
    out = s.stop()
    assert out == {"sm_mhz": 1600.0, "sm_max_mhz": 1965.0, "reasons": ["sw_power_cap"], "samples": 3}
    pk = measured_peaks()
    assert pk["hbm_gbs"] > 1000 and pk["bf16_tflops"] > 100


def test_throughput_sweep_summary_and_error_rows():
    from cppmega_mlx_b200.cli.bench_throughput_sweep import summarise
    steps = [{"tokens_per_second": v, "seconds": 4096 / v} for v in (10.0, 50.0, 100.0, 110.0, 90.0, 120.0)]
    ok = summarise({"status": "ok", "steps": steps, "memory": {"after": {"peak_bytes": 123}}, "final_loss": 2.5,
                    "throughput_claim_gate": {"status": "pass"}, "kernel_dispatch": {"total_calls": 7}}, warmup=2)
    assert ok["status"] == "ok" and ok["timed_steps"] == 4
    assert ok["tokens_per_second"] == {"median": 105.0, "p10": 90.0, "p90": 120.0}
    assert ok["peak_memory_bytes"] == 123 and ok["throughput_claim_gate"] == "pass" and ok["kernel_calls"] == 7
    assert abs(ok["seconds_per_step_median"] - 4096 / 105.0) < 2.0
    err = summarise({"status": "error", "error": "out of memory", "error_type": "OutOfMemoryError", "steps": steps}, warmup=2)
    assert err == {"status": "error", "error": "out of memory", "error_type": "OutOfMemoryError"}
    assert summarise({"status": "ok", "steps": steps[:2]}, warmup=2)["error"] == "no timed steps"


def test_throughput_sweep_runs_a_cell_end_to_end(tmp_path):
    """One tiny (optimizer, batch) cell through the receipt harness in a fresh process, and a cell that fails stays in the table."""
    from cppmega_mlx_b200.cli import bench_throughput_sweep as sweep
    out = tmp_path / "sweep.json"
    rc = sweep.main(["--model-profile", "custom", "--optimizers", "adamw,not_an_optimizer", "--batch-sizes", "1", "--seq-len", "32",
                     "--steps", "3", "--warmup-steps", "1", "--dtype", "float32", "--loss-backend", "cross_entropy", "--depth", "2", "--vocab-size", "128",
                     "--hidden-size", "32", "--num-attention-heads", "2", "--pattern", "AM", "--cell-timeout", "600", "--output", str(out)])
    doc = json.loads(out.read_text())
    assert rc == 0 and doc["format"] == "cppmega_b200_throughput_sweep_v1" and len(doc["rows"]) == 2
    good, bad = doc["rows"]
    assert good["status"] == "ok" and good["timed_steps"] == 2 and good["tokens_per_second"]["median"] > 0
    assert bad["status"] == "error" and bad["optimizer"] == "not_an_optimizer"
    assert doc["best"]["optimizer"] == "adamw"

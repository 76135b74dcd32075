"""Property-style checks of the data layer over many random inputs: packing never loses or reorders a document's tokens, masks keep
documents apart, FIM transforms are permutations of the input plus sentinels, dataset cursors resume exactly, batches validate."""
import random

import numpy as np
import pytest
import torch

EOS, BOS, PAD = 3, 2, 0


def _random_docs(rng, n, max_len, vocab=50):
    return [[rng.randrange(4, vocab) for _ in range(rng.randint(1, max_len))] for _ in range(n)]


def _split_row_into_docs(tokens, mask):
    docs, cur = [], []
    for t, m in zip(tokens, mask):
        if not m:
            break
        if t == BOS and not cur:
            continue
        cur.append(int(t))
        if t == EOS:
            docs.append(cur)
            cur = []
    return docs, cur


@pytest.mark.parametrize("seed", range(6))
@pytest.mark.parametrize("bos", [None, BOS])
def test_best_fit_packing_keeps_every_document_whole(seed, bos):
    from cppmega_mlx_b200.data.packing import pack_bos_aligned_best_fit
    rng = random.Random(seed)
    seq_len = rng.choice([16, 24, 33])
    docs = _random_docs(rng, rng.randint(1, 30), seq_len - 3)
    p = pack_bos_aligned_best_fit(docs, seq_len=seq_len, eos_token_id=EOS, bos_token_id=bos, pad_token_id=PAD)
    assert p.tokens.shape[1] == seq_len and p.tokens.dtype == np.int32
    got = []
    for r in range(p.tokens.shape[0]):
        row_docs, rest = _split_row_into_docs(p.tokens[r], p.token_mask[r])
        assert rest == []                                      # no document straddles a row
        got += row_docs
        if bos is not None:
            assert p.tokens[r, 0] == BOS
        assert not p.token_mask[r, int(p.token_mask[r].sum()):].any()          # padding is a suffix
        assert (p.tokens[r][~p.token_mask[r]] == PAD).all()
    assert sorted(got) == sorted(d + [EOS] for d in docs)     # a permutation of the input documents, each closed by EOS
    # the real positions are exactly the documents (with their EOS) plus one BOS per row
    assert p.token_mask.sum() == sum(len(d) + 1 for d in docs) + (p.tokens.shape[0] if bos is not None else 0)


@pytest.mark.parametrize("seed", range(6))
def test_sequential_packing_is_the_concatenation(seed):
    from cppmega_mlx_b200.data.packing import pack_documents_with_eos
    rng = random.Random(100 + seed)
    seq_len = rng.choice([8, 13, 32])
    docs = _random_docs(rng, rng.randint(1, 20), seq_len * 2) if seed % 2 else _random_docs(rng, 12, seq_len - 1)
    p = pack_documents_with_eos(docs, seq_len=seq_len, eos_token_id=EOS, oversized="truncate")
    flat = p.tokens[p.token_mask].tolist()
    want = []
    for d in docs:
        d = d + [EOS]
        if len(d) > seq_len:
            d = d[:seq_len - 1] + [EOS]                        # truncated documents still end in EOS
        want += d
    assert flat == want
    assert p.token_mask[:-1].all()                             # only the last row may be short
    # document ids count the EOS tokens strictly before a position, restarting in every row
    for r in range(p.tokens.shape[0]):
        n = int(p.token_mask[r].sum())
        ids = p.doc_ids[r, :n].tolist()
        expect, k = [], 0
        for t in p.tokens[r, :n]:
            expect.append(k)
            k += int(t == EOS)
        assert ids == expect and (p.doc_ids[r, n:] == -1).all()


def test_packing_refuses_what_it_cannot_represent():
    from cppmega_mlx_b200.data.packing import pack_documents_with_eos
    with pytest.raises(ValueError, match="does not fit"):
        pack_documents_with_eos([[5] * 10], seq_len=8, eos_token_id=EOS)
    with pytest.raises(ValueError, match="negative"):
        pack_documents_with_eos([[5, -1]], seq_len=8, eos_token_id=EOS)
    with pytest.raises(TypeError):
        pack_documents_with_eos([[0.5, 1.5]], seq_len=8, eos_token_id=EOS)
    with pytest.raises(ValueError, match="one-dimensional"):
        pack_documents_with_eos([[[1, 2]]], seq_len=8, eos_token_id=EOS)
    with pytest.raises(ValueError, match="strategy"):
        pack_documents_with_eos([[5]], seq_len=8, eos_token_id=EOS, strategy="random")
    with pytest.raises(ValueError, match="at least 2"):
        pack_documents_with_eos([[5]], seq_len=1, eos_token_id=EOS, bos_token_id=BOS)
    with pytest.raises(ValueError, match="non-negative integer"):
        pack_documents_with_eos([[5]], seq_len=8, eos_token_id=True)
    empty = pack_documents_with_eos([[]], seq_len=4, eos_token_id=EOS)          # an empty document is just its EOS
    assert empty.tokens[0].tolist() == [EOS, PAD, PAD, PAD]


@pytest.mark.parametrize("seed", range(4))
def test_boundary_masks_numpy_and_torch_agree_and_separate_documents(seed):
    from cppmega_mlx_b200.data.packing import (cumulative_doc_ids_from_eos, document_boundary_mask, torch_cumulative_doc_ids_from_eos,
                                               torch_document_boundary_mask)
    g = np.random.default_rng(seed)
    tokens = g.integers(3, 9, size=(3, 17))                    # EOS (3) appears often
    mask = np.ones_like(tokens, dtype=bool)
    mask[1, 11:] = False
    ids = cumulative_doc_ids_from_eos(tokens, eos_token_id=EOS, token_mask=mask)
    tids = torch_cumulative_doc_ids_from_eos(torch.from_numpy(tokens), eos_token_id=EOS, token_mask=torch.from_numpy(mask))
    assert np.array_equal(ids, tids.numpy())
    for causal in (False, True):
        m_np = document_boundary_mask(ids, token_mask=mask, causal=causal)
        m_t = torch_document_boundary_mask(tids, token_mask=torch.from_numpy(mask), causal=causal)
        assert np.array_equal(m_np, m_t.numpy())
    m = document_boundary_mask(ids, causal=True)
    for b in range(3):
        for i in range(17):
            for j in range(17):
                same = ids[b, i] >= 0 and ids[b, i] == ids[b, j]
                assert bool(m[b, i, j]) == bool(same and j <= i)
    assert document_boundary_mask(torch.from_numpy(ids)).dtype == torch.bool                 # torch input: causal by default
    assert document_boundary_mask(torch.from_numpy(ids), expand_heads=True).shape == (3, 1, 17, 17)
    assert not document_boundary_mask(ids)[1, 12:, :].any() and not document_boundary_mask(ids)[1, :, 12:].any()   # padded positions see nothing
    with pytest.raises(ValueError, match="two-dimensional"):
        cumulative_doc_ids_from_eos(tokens[0], eos_token_id=EOS)
    with pytest.raises(ValueError, match="token_mask shape"):
        cumulative_doc_ids_from_eos(tokens, eos_token_id=EOS, token_mask=mask[:, :5])


@pytest.mark.parametrize("seed", range(8))
def test_fim_transform_is_a_permutation_with_sentinels(seed):
    from cppmega_mlx_b200.data.fim import FIM_SPECIAL_TOKEN_IDS as S
    from cppmega_mlx_b200.data.fim import apply_fim_permutation, apply_fim_transform, apply_ifim_transform, sample_middle_span
    rng = random.Random(seed)
    doc = [rng.randrange(100, 200) for _ in range(rng.randint(3, 40))]
    out = apply_fim_transform(doc, fim_rate=1.0, spm_rate=0.5, seed=seed)
    sent = {S.fim_prefix, S.fim_suffix, S.fim_middle, S.eot}
    assert sorted(t for t in out if t not in sent) == sorted(doc)               # nothing lost, nothing invented
    assert out[0] == S.fim_prefix and out[-1] == S.eot and len(out) == len(doc) + 4
    assert apply_fim_transform(doc, fim_rate=1.0, seed=seed) == out             # a seed fixes the sample
    assert apply_fim_transform(doc, fim_rate=0.0, seed=seed) == doc
    # the original order can be rebuilt from either layout
    start, end = sample_middle_span(len(doc), rng=random.Random(seed + 1))
    assert 0 < start < end < len(doc)
    psm = apply_fim_permutation(doc, span=(start, end), mode="psm")
    i_s, i_m = psm.index(S.fim_suffix), psm.index(S.fim_middle)
    assert psm[1:i_s] + psm[i_m + 1:-1] + psm[i_s + 1:i_m] == doc               # prefix + middle + suffix
    spm = apply_fim_permutation(doc, span=(start, end), mode="spm")
    assert spm[:2] == [S.fim_prefix, S.fim_suffix]
    i_m = spm.index(S.fim_middle)
    assert spm[i_m + 1:-1] + spm[2:i_m] == doc                                  # (prefix + middle) + suffix
    instr = [7, 8, 9]
    ifim = apply_ifim_transform(doc, instruction_token_ids=instr, fim_rate=1.0, seed=seed)
    assert ifim[0] == S.fim_instruction and ifim[1:4] == instr and ifim[4:] == out
    with pytest.raises(ValueError, match="either seed or rng"):
        apply_fim_transform(doc, seed=1, rng=random.Random(1))
    with pytest.raises(ValueError, match="between 0.0 and 1.0"):
        apply_fim_transform(doc, fim_rate=1.5)
    with pytest.raises(ValueError, match="must satisfy"):
        apply_fim_permutation(doc, span=(0, 2), mode="psm")
    with pytest.raises(ValueError, match="psm"):
        apply_fim_permutation(doc, span=(1, 2), mode="xyz")
    with pytest.raises(ValueError, match="not be empty"):
        apply_ifim_transform(doc, instruction_token_ids=[], fim_rate=1.0, seed=0)
    assert apply_fim_transform([1, 2], fim_rate=1.0, seed=0) == [1, 2]          # too short to split: returned unchanged


@pytest.mark.parametrize("shuffle", [False, True])
def test_dataset_cursor_resumes_the_exact_stream(tmp_path, shuffle):
    from cppmega_mlx_b200.data.token_dataset import TokenNpzDataset
    tokens = np.arange(10 * 8 + 5, dtype=np.int32)             # 10 windows of 8 and a dropped tail
    np.savez(tmp_path / "t.npz", tokens=tokens)
    mk = lambda **kw: TokenNpzDataset(tmp_path / "t.npz", seq_len=8, batch_size=3, shuffle=shuffle, seed=11, pin_memory=False, **kw)
    ds = mk(loop=True)
    assert ds.num_samples == 10 and ds.num_batches == 3 and ds.dropped_samples == 1 and len(ds) == 3
    it = ds.iter_batches()
    stream = [next(it).tokens.clone() for _ in range(8)]       # more than two epochs
    for consumed in (0, 1, 3, 4, 7):
        cur = ds.cursor_after(consumed)
        assert (cur.epoch, cur.batch_offset, cur.global_batch_offset) == (consumed // 3, consumed % 3, consumed)
        resumed = mk(loop=True).iter_batches(resume_batch=cur.batch_offset, epoch=cur.epoch)
        for k in range(consumed, 8):
            assert torch.equal(next(resumed).tokens, stream[k]), (consumed, k)
    if shuffle:
        assert not torch.equal(stream[0], stream[3])           # another epoch, another order
        assert sorted(ds.sample_order(epoch=2).tolist()) == list(range(10))
    else:
        assert torch.equal(stream[0], stream[3])
        assert stream[0][0].tolist() == list(range(8))
    once = list(mk().iter_batches())                           # without loop: one pass, the remainder sample dropped
    assert len(once) == 3 and list(mk().iter_batches(resume_batch=3)) == []
    assert ds.token_id_range() == (0, 79)
    with pytest.raises(ValueError, match="non-negative"):
        ds.cursor_after(-1)


def test_lm_batch_views_and_validation():
    from cppmega_mlx_b200.data.batch import LMTokenBatch, ensure_lm_batch, synthetic_token_batch
    t = torch.arange(24).reshape(2, 12)
    am = torch.ones(2, 12)
    am[1, 8:] = 0
    b = LMTokenBatch(tokens=t, attention_mask=am, structure_ids=t % 5, document_ids=t // 6)
    assert torch.equal(b.inputs, t[:, :-1]) and torch.equal(b.targets, t[:, 1:])
    assert b.num_target_tokens == 11 + 7 and torch.equal(b.target_mask, am[:, 1:])
    side = b.side_inputs()
    assert set(side) == {"structure_ids", "document_ids"} and side["structure_ids"].shape == (2, 11)
    half = b.slice_rows(1, 2)
    assert half.tokens.shape == (1, 12) and torch.equal(half.attention_mask, am[1:2]) and half.dep_levels is None
    assert set(b.as_dict()) == {"tokens", "attention_mask", "structure_ids", "document_ids"}
    assert torch.equal(b.to("cpu").tokens, t)
    assert ensure_lm_batch(b) is b
    assert torch.equal(ensure_lm_batch({"tokens": t, "unknown_key": 1}).tokens, t)
    assert torch.equal(ensure_lm_batch(t.numpy()).tokens, t)
    with pytest.raises(ValueError, match="must contain 'tokens'"):
        ensure_lm_batch({"ids": t})
    with pytest.raises(ValueError, match=r"\(B, S\)"):
        LMTokenBatch(tokens=torch.arange(5))
    with pytest.raises(ValueError, match="at least two positions"):
        LMTokenBatch(tokens=torch.zeros(2, 1, dtype=torch.long))
    with pytest.raises(ValueError, match="must match tokens"):
        LMTokenBatch(tokens=t, dep_levels=torch.zeros(2, 5, dtype=torch.long))
    s1, s2 = synthetic_token_batch(2, 16, 100, seed=3), synthetic_token_batch(2, 16, 100, seed=3)
    assert torch.equal(s1.tokens, s2.tokens) and s1.tokens.shape == (2, 17) and int(s1.tokens.max()) < 100

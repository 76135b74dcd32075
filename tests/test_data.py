"""Data pipeline: NPZ / Megatron / Parquet readers, packing, FIM, tokenizer contract, DataLoader bridge."""
import numpy as np
import pytest
import torch

from cppmega_mlx_b200.data import fim, packing
from cppmega_mlx_b200.data.batch import LMTokenBatch, synthetic_token_batch
from cppmega_mlx_b200.data.megatron_indexed import MegatronIndexedDataset, parse_mmididx, write_mmididx
from cppmega_mlx_b200.data.token_dataset import TokenNpzDataset, fixed_windows, open_token_dataset
from cppmega_mlx_b200.data.tokenizer_contract import EXPECTED_VOCAB_SIZE, tokenizer_contract_metadata, validate_special_tokens


def test_synthetic_batch_is_seeded_and_shifted():
    a = synthetic_token_batch(2, 9, vocab_size=50, seed=3)
    b = synthetic_token_batch(2, 9, vocab_size=50, seed=3)
    assert torch.equal(a.tokens, b.tokens) and a.tokens.shape == (2, 10)
    assert torch.equal(a.inputs, a.tokens[:, :-1]) and torch.equal(a.targets, a.tokens[:, 1:])
    assert int(a.tokens.max()) < 50


def test_fixed_windows_drop_tail():
    w = fixed_windows(np.arange(23), 5)
    assert w.shape == (4, 5) and w[3, 4] == 19


def test_npz_dataset_cursor_and_shuffle(tmp_path):
    p = tmp_path / "t.npz"
    np.savez(p, tokens=np.arange(8 * 6, dtype=np.int32) % 97)
    ds = TokenNpzDataset(p, seq_len=6, batch_size=2, shuffle=True, seed=4)
    assert ds.num_samples == 8 and ds.num_batches == 4
    e0 = [b.tokens.clone() for b in ds.iter_batches(epoch=0)]
    e0b = [b.tokens.clone() for b in ds.iter_batches(epoch=0)]
    e1 = [b.tokens.clone() for b in ds.iter_batches(epoch=1)]
    assert all(torch.equal(x, y) for x, y in zip(e0, e0b))
    assert not all(torch.equal(x, y) for x, y in zip(e0, e1))
    resumed = [b.tokens for b in ds.iter_batches(epoch=0, resume_batch=2)]
    assert len(resumed) == 2 and torch.equal(resumed[0], e0[2])
    cur = ds.cursor_after(5)
    assert (cur.epoch, cur.batch_offset) == (1, 1)


def test_npz_rejects_short_and_bad_args(tmp_path):
    p = tmp_path / "s.npz"
    np.savez(p, tokens=np.arange(3, dtype=np.int32))
    with pytest.raises(ValueError):
        TokenNpzDataset(p, seq_len=8, batch_size=1)
    with pytest.raises(ValueError):
        TokenNpzDataset(p, seq_len=1, batch_size=1)


def test_megatron_round_trip_and_validation(tmp_path):
    seqs = [np.arange(10, dtype=np.int32), np.arange(100, 107, dtype=np.int32), np.arange(5, dtype=np.int32)]
    bin_path, idx_path = write_mmididx(tmp_path / "corp", seqs)
    idx = parse_mmididx(idx_path)
    assert list(idx.sequence_lengths) == [10, 7, 5] and idx.dtype == np.int32
    ds = MegatronIndexedDataset(tmp_path / "corp", seq_len=4, batch_size=2)
    flat = np.concatenate(seqs)
    first = next(iter(ds.iter_batches()))
    assert first.tokens.shape == (2, 4)
    assert first.tokens.flatten().tolist() == flat[:8].tolist()
    same = open_token_dataset(str(bin_path), seq_len=4, batch_size=2)
    assert same.num_samples == ds.num_samples
    raw = bytearray(idx_path.read_bytes())
    raw[0:4] = b"XXXX"
    bad = tmp_path / "bad.idx"
    bad.write_bytes(raw)
    with pytest.raises((ValueError, NotImplementedError)):
        parse_mmididx(bad)


def test_parquet_tokens_and_text(tmp_path):
    pa = pytest.importorskip("pyarrow")
    import pyarrow.parquet as pq
    from cppmega_mlx_b200.data.parquet_dataset import TokenParquetDataset
    p = tmp_path / "a.parquet"
    pq.write_table(pa.table({"tokens": [[1, 2, 3, 4, 5], [6, 7, 8], [9, 10, 11, 12]]}), p)
    ds = TokenParquetDataset(p, seq_len=4, batch_size=1)
    assert ds.num_samples == 3
    assert next(iter(ds)).tokens.tolist() == [[1, 2, 3, 4]]
    q = tmp_path / "b.parquet"
    pq.write_table(pa.table({"text": ["ab", "cd"]}), q)

    class Tok:
        def encode(self, s):
            return [ord(c) for c in s]
    dt = TokenParquetDataset(q, seq_len=2, batch_size=1, text_key="text", tokenizer=Tok(), eos_token_id=3)
    assert next(iter(dt)).tokens.tolist() == [[97, 98]]
    with pytest.raises(ValueError):
        TokenParquetDataset(q, seq_len=2, batch_size=1)


def test_packing_sequential_and_best_fit():
    docs = [[5, 6, 7], [8, 9], [10, 11, 12, 13, 14]]
    out = packing.pack_documents_with_eos(docs, seq_len=8, eos_token_id=3)
    assert out.tokens.shape[1] == 8
    flat = out.tokens[out.token_mask.astype(bool)].tolist()
    assert flat == [5, 6, 7, 3, 8, 9, 3, 10, 11, 12, 13, 14, 3][:len(flat)] or sorted(flat) == sorted([5, 6, 7, 3, 8, 9, 3, 10, 11, 12, 13, 14, 3])
    bf = packing.pack_documents_with_eos(docs, seq_len=8, eos_token_id=3, strategy="best_fit")
    assert bf.tokens.shape[1] == 8
    with pytest.raises(ValueError):
        packing.pack_documents_with_eos([[1] * 20], seq_len=8, eos_token_id=3)
    tr = packing.pack_documents_with_eos([[1] * 20], seq_len=8, eos_token_id=3, oversized="truncate")
    assert tr.tokens.shape == (1, 8)


def test_doc_ids_and_boundary_mask():
    toks = np.array([[5, 6, 3, 7, 8, 3, 9, 0]])
    ids = packing.cumulative_doc_ids_from_eos(toks, eos_token_id=3)
    assert ids.tolist() == [[0, 0, 0, 1, 1, 1, 2, 2]]
    m = packing.document_boundary_mask(ids, causal=True)
    assert m[0, 3, 2] == False and m[0, 4, 3] == True and m[0, 3, 4] == False  # noqa: E712
    tids = packing.torch_cumulative_doc_ids_from_eos(torch.from_numpy(toks), eos_token_id=3)
    assert tids.tolist() == ids.tolist()
    tm = packing.torch_document_boundary_mask(tids, causal=True)
    assert np.array_equal(tm.numpy().astype(bool).reshape(m.shape), m.astype(bool))


def test_fim_modes():
    doc = list(range(100, 110))
    psm = fim.apply_fim_permutation(doc, span=(3, 6), mode="psm")
    assert psm == [4] + doc[:3] + [6] + doc[6:] + [5] + doc[3:6] + [3]
    spm = fim.apply_fim_permutation(doc, span=(3, 6), mode="spm")
    assert spm[0] in (4, 6) and spm[-1] == 3 and sorted(t for t in spm if t >= 100) == doc
    assert fim.apply_fim_transform(doc, fim_rate=0.0, seed=1) == doc
    a = fim.apply_fim_transform(doc, fim_rate=1.0, seed=7)
    assert a == fim.apply_fim_transform(doc, fim_rate=1.0, seed=7) and len(a) == len(doc) + 4
    i = fim.apply_ifim_permutation(doc, instruction_token_ids=[50, 51], span=(2, 4), mode="psm")
    assert i[:3] == [45, 50, 51]
    with pytest.raises(ValueError):
        fim.apply_fim_transform(doc, fim_rate=1.5)


def test_tokenizer_contract():
    meta = tokenizer_contract_metadata()
    assert EXPECTED_VOCAB_SIZE == 65536
    good = {"<BOS>": 2, "<EOT>": 3, "<FIM_PREFIX>": 4, "<FIM_MIDDLE>": 5, "<FIM_SUFFIX>": 6}
    assert isinstance(meta, dict)
    problems = validate_special_tokens({"<EOT>": 9})
    assert problems


def test_dataloader_bridge(tmp_path):
    from cppmega_mlx_b200.data.dataloader_bridge import iterate_lm_batches, make_dataloader
    p = tmp_path / "t.npz"
    np.savez(p, tokens=np.arange(40, dtype=np.int32))
    ds = TokenNpzDataset(p, seq_len=5, batch_size=2, pin_memory=False)
    direct = [b.tokens for b in ds.iter_batches()]
    viadl = [b.tokens for b in iterate_lm_batches(make_dataloader(ds, num_workers=0))]
    assert len(direct) == len(viadl) and all(torch.equal(a, b) for a, b in zip(direct, viadl))


def test_byte_fallback_tokenizer_round_trip():
    from cppmega_mlx_b200.tokenizer import build_byte_fallback_tokenizer
    tok = build_byte_fallback_tokenizer()
    s = "int main()\n{ return 0; }"
    ids = tok.encode(s)
    assert tok.decode(ids) == s

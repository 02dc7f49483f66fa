import numpy as np
import pytest
import torch

from nmtgminor_b200.data.dataset import Dataset, allocate_batches, allocate_batches_python, collate
from nmtgminor_b200.data.iterator import DataIterator, MultiDataIterator
from nmtgminor_b200.data.mmap_dataset import (IndexedDataset, IndexedDatasetBuilder, MMapIndexedDataset, write_dataset)
from nmtgminor_b200.data.synthetic import synthetic_dataset, synthetic_pairs, token_budget_batches


@pytest.mark.parametrize("unbalanced", [False, True])
@pytest.mark.parametrize("multiplier", [1, 8])
def test_cpp_allocator_matches_python(unbalanced, multiplier):
    rng = np.random.RandomState(3)
    n = 3000
    src, tgt = rng.randint(1, 120, n), rng.randint(1, 120, n)
    lengths = np.maximum(src, tgt)
    order = np.lexsort((src, tgt))
    kw = dict(batch_size_words=1500, batch_size_frames=2500, batch_size_sents=64, multiplier=multiplier, max_src_len=110,
              max_tgt_len=110, min_src_len=2, min_tgt_len=2, cleaning=True, unbalanced=unbalanced, cut_off_size=100,
              smallest_batch_size=4)
    a = allocate_batches(order, lengths, src, tgt, **kw)
    b = allocate_batches_python(list(order), lengths, src, tgt, **kw)
    assert a == b
    for batch in a:
        assert len(batch) <= 64
        if not unbalanced and len(batch) > 1:
            assert max(lengths[i] for i in batch) * len(batch) <= 1500
    kept = {i for bt in a for i in bt}
    assert all(2 <= src[i] < 110 and 2 <= tgt[i] < 110 for i in kept)


def test_collate_keys_layout_and_packing():
    src, tgt = synthetic_pairs(5, 100, 3, 9, seed=2)
    b = collate(src, tgt, round_to=16)
    T_s, T_t = max(len(s) for s in src), max(len(t) for t in tgt)
    assert b.get("source").shape == (T_s, 5) and b.get("target").shape == (T_t, 5)
    assert b.get("target_input").shape == (T_t - 1, 5) and b.get("target_output").shape == (T_t - 1, 5)
    assert torch.equal(b.get("target_input"), b.get("target")[:-1]) and torch.equal(b.get("target_output"), b.get("target")[1:])
    assert b.get("src_selfattn_mask").shape == (5, T_s) and b.get("target_input_selfattn_mask").shape == (5, T_t - 1)
    assert b.tgt_size == sum(len(t) - 1 for t in tgt) and b.src_size == sum(len(s) for s in src) and b.size == 5
    ps, pt, lab = b.packed_source(), b.packed_target_input(), b.packed_target_output()
    assert ps.tokens.numel() % 16 == 0 and pt.tokens.numel() == lab.numel()
    assert torch.equal(ps.tokens[:b.src_size], torch.cat(src))
    assert torch.equal(pt.tokens[:b.tgt_size], torch.cat([t[:-1] for t in tgt]))
    assert torch.equal(lab[:b.tgt_size], torch.cat([t[1:] for t in tgt]))
    assert (lab[b.tgt_size:] == 0).all() and ps.cu.tolist()[-1] == b.src_size
    # packed rows agree with the padded layout
    padded = ps.pad(ps.tokens[:, None].float()).squeeze(-1).long()
    assert torch.equal(padded, b.get("source"))


def test_audio_collate_has_padding_channel():
    feats = [torch.randn(n, 40) for n in (7, 3)]
    tgt = [torch.tensor([2, 5, 6, 3]), torch.tensor([2, 7, 3])]
    b = collate(feats, tgt, src_type="audio")
    assert b.get("source").shape == (7, 2, 41)
    assert b.get("source")[:, 1, 0].tolist() == [1, 1, 1, 0, 0, 0, 0]
    assert b.get("src_selfattn_mask")[1].tolist() == [False] * 3 + [True] * 4


def test_dataset_token_budget_and_static_batches():
    ds = synthetic_dataset(500, 200, 5, 40, 600, multiplier=4)
    sizes = ds.batch_sizes()
    assert sum(sizes) == 500
    assert all(s % 4 == 0 for s in sizes[:-1] if s >= 4)
    b = ds.get_batch(0)
    assert b.get("target").shape[0] * b.size <= 600 + b.get("target").shape[0]
    static = token_budget_batches(200, 5, 40, 512, 3, static=True)
    sig = {(x.packed_source().tokens.numel(), x.packed_target_input().tokens.numel(), x.packed_source().cu.numel()) for x in static}
    assert len(sig) == 1
    assert all(x.tgt_size <= 512 for x in static)


def test_iterator_shards_evenly_and_resumes():
    ds = synthetic_dataset(300, 100, 5, 20, 200)
    n = len(ds)
    its = [DataIterator(ds, seed=5, num_shards=3, shard_id=r, epoch=1) for r in range(3)]
    orders = [it._order_for_epoch(1) for it in its]
    assert len({len(o) for o in orders}) == 1 and len(orders[0]) == (n + 2) // 3
    assert set(range(n)) <= set(orders[0]) | set(orders[1]) | set(orders[2])
    assert DataIterator(ds, seed=5, num_shards=3, shard_id=0)._order_for_epoch(2) != orders[0]
    it = DataIterator(ds, seed=1)
    e = it.next_epoch_itr()
    first = [next(e).get("indices").tolist() for _ in range(4)]
    state = it.state_dict()
    assert state["iterations_in_epoch"] == 4 and state["epoch"] == 1
    it2 = DataIterator(ds, seed=1)
    it2.load_state_dict(state)
    e2 = it2.next_epoch_itr()
    full = DataIterator(ds, seed=1).next_epoch_itr()
    expect = [b.get("indices").tolist() for b in full]
    assert first == expect[:4]
    assert [b.get("indices").tolist() for b in e2] == expect[4:]
    assert it2.end_of_epoch()


def test_buffered_and_multi_iterators():
    a, b = synthetic_dataset(100, 50, 3, 10, 100, seed=1), synthetic_dataset(60, 50, 3, 10, 100, seed=2)
    it = DataIterator(a, buffer_size=4).next_epoch_itr()
    assert sum(1 for _ in it) == len(a)
    m = MultiDataIterator([a, b], seed=3)
    assert sum(1 for _ in m.next_epoch_itr()) == len(a) + len(b)


def test_multi_iterator_equal_probability_interleave():
    a, b = synthetic_dataset(100, 50, 3, 10, 100, seed=1), synthetic_dataset(60, 50, 3, 10, 100, seed=2)
    m = MultiDataIterator([a, b], seed=3, probabilities=[1, 1])
    n1 = sum(1 for _ in m.next_epoch_itr())
    first = list(m._schedule)
    assert 0 < n1 <= len(a) + len(b) and n1 == len(m)
    assert min(first.count(0), first.count(1)) > 0 and (first.count(0) == len(a) or first.count(1) == len(b))
    m.next_epoch_itr()
    assert m._schedule != first                     # reseeded per epoch


def test_trainer_skips_a_batch_that_runs_out_of_memory():
    from types import SimpleNamespace
    from nmtgminor_b200.train.trainer import Trainer
    calls = {"zero": 0}

    class _Engine:
        device = "cpu"

        def train_step(self, batch, update=True):
            raise torch.cuda.OutOfMemoryError("CUDA out of memory (simulated on the host)")

    tr = Trainer.__new__(Trainer)
    tr.engine, tr.world_size, tr.cuda = _Engine(), 1, False
    tr.optim = SimpleNamespace(zero_grad=lambda: calls.__setitem__("zero", calls["zero"] + 1))
    tr.log = lambda msg: None
    loss = tr._guarded_step(SimpleNamespace(src_size=5, tgt_size=7), True)
    assert float(loss) == 0.0 and calls["zero"] == 1 and tr.oom_skipped == 1
    tr.world_size = 2
    import pytest
    with pytest.raises(torch.cuda.OutOfMemoryError):
        tr._guarded_step(SimpleNamespace(src_size=5, tgt_size=7), True)


def test_mmap_and_legacy_indexed_roundtrip(tmp_path):
    items = [torch.randint(0, 60000, (n,)) for n in (3, 1, 17, 5)]
    prefix = str(tmp_path / "corpus")
    write_dataset(prefix, items, np.uint16)
    ds = MMapIndexedDataset(prefix)
    assert len(ds) == 4 and ds.sizes.tolist() == [3, 1, 17, 5]
    assert all(torch.equal(ds[i], items[i]) for i in range(4))
    raw = open(prefix + ".idx", "rb").read()
    assert raw[:9] == b"MMIDIDX\x00\x00" and int.from_bytes(raw[9:17], "little") == 1 and raw[17] == 8
    b = IndexedDatasetBuilder(str(tmp_path / "old"), np.int32)
    for it in items:
        b.add_item(it)
    b.finalize()
    old = IndexedDataset(str(tmp_path / "old"))
    assert all(torch.equal(old[i], items[i]) for i in range(4))


def test_auxiliary_target_travels_with_the_batch():
    from nmtgminor_b200.data.dataset import Dataset
    src = [torch.arange(4, 4 + n) for n in (3, 5, 2, 4)]
    tgt = [torch.tensor([2] + [7] * n + [3]) for n in (2, 3, 1, 2)]
    aux = [torch.tensor([2] + [10 + i] * (i + 1) + [3]) for i in range(4)]
    ds = Dataset(src, tgt, batch_size_words=10 ** 6, aux_tgt_data=aux, cleaning=False, round_to=1)
    b = ds.get_batch(0)
    order = b.get("indices").tolist() if b.get("indices") is not None else list(range(4))
    inp, out, lens = b.get("aux_target_input"), b.get("aux_target_output"), b.get("aux_tgt_lengths")
    assert inp.shape == out.shape and inp.shape[1] == 4
    for col, i in enumerate(order):
        L = int(lens[col])
        assert L == i + 2 and inp[:L, col].tolist() == [2] + [10 + i] * (i + 1) and out[L - 1, col] == 3


def test_concat_dataset_joins_random_examples_up_to_the_length_limit():
    """``concat=True``: sources are joined along time, targets become one sentence with a single BOS and EOS, no
    example is used twice inside a batch, and no joined source exceeds the limit."""
    import torch
    from nmtgminor_b200.data.dataset import Dataset
    rng = np.random.RandomState(0)
    n = 60
    src = [torch.full((int(rng.randint(5, 30)), 1), float(i)) for i in range(n)]           # audio-like [T, 1], value = id
    tgt = [torch.tensor([2] + [10 + i] * int(rng.randint(1, 4)) + [3]) for i in range(n)]
    data = Dataset(src, tgt, batch_size_frames=400, max_src_len=100, max_tgt_len=200, data_type="audio", concat=True,
                   concat_seed=5, padded=True, packed=True, round_to=1)
    assert all(len(b) <= 4 for b in data.batches) and sum(len(b) for b in data.batches) == n
    joined_any = False
    for bi in range(len(data)):
        batch = data.get_batch(bi)
        source = batch.get("source")                                                       # [T, B, 1 + 1] with a validity column
        tgt_out, tgt_in = batch.get("target_output"), batch.get("target_input")
        used = []
        for b in range(source.shape[1]):
            valid = source[:, b, 0] > 0
            ids = source[valid, b, 1].long().tolist()
            assert len(ids) <= 100
            order = [k for k, _ in __import__("itertools").groupby(ids)]
            used += order
            joined_any |= len(order) > 1
            assert sum(len(src[k]) for k in order) == len(ids)
            full = [int(tgt_in[0, b])] + [int(t) for t in tgt_out[:, b] if int(t) != 0]
            expect = [2] + [t for k in order for t in tgt[k][1:-1].tolist()] + [3]
            assert full == expect
        assert len(used) == len(set(used))
    assert joined_any

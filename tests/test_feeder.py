"""The packed dataset and the batch feeder deliver exactly the batches of ``RawDataset.iterate``
(khan/data/dataset.py:144-183 of the reference), in the same order, for the same numpy seed --
in order, shuffled and with fuzz -- while running ahead of the consumer on a thread."""
import numpy as np
import pytest

from khan_b200 import RawDataset
from khan_b200.data import synthetic as syn
from khan_b200.data.feeder import BatchFeeder, PackedDataset


def _dataset(n_mols=37, with_grads=True):
    b = syn.config1(n_mols=n_mols)
    mols = b.molecules()
    rng = np.random.default_rng(2)
    ys = list(rng.normal(size=len(mols)))
    grads = [rng.normal(size=(len(m), 3)) for m in mols] if with_grads else None
    return RawDataset(mols, ys, grads)


@pytest.mark.parametrize("shuffle,fuzz", [(False, None), (True, None), (True, 0.05), (False, 0.1)])
@pytest.mark.parametrize("dtype", [np.float32, np.float64])
def test_same_batches_as_raw_dataset(shuffle, fuzz, dtype):
    ds = _dataset()
    np.random.seed(7)
    want = list(ds.iterate(batch_size=8, shuffle=shuffle, fuzz=fuzz))
    np.random.seed(7)
    feeder = BatchFeeder(PackedDataset.from_raw(ds, dtype), 8, shuffle, fuzz, devices=None, depth=2)
    got = 0
    for fed, (mol_Xs, mol_ids, mol_yts, mol_grads) in zip(feeder, want):
        assert fed.index == got and fed.n_atoms == len(mol_Xs) and fed.n_mols == len(mol_yts)
        assert np.array_equal(fed.types.numpy(), mol_Xs[:, 0].astype(np.int32))
        for k, c in enumerate((fed.x, fed.y, fed.z)):
            assert np.array_equal(c.numpy(), mol_Xs[:, 1 + k].astype(dtype))
        assert np.array_equal(fed.mol_ids.numpy(), mol_ids)
        assert np.array_equal(fed.ys.numpy(), np.asarray(mol_yts, dtype))
        assert np.array_equal(fed.grads.numpy().T, mol_grads.astype(dtype))
        counts = np.bincount(mol_ids, minlength=fed.n_mols)
        assert np.array_equal(fed.counts_host, counts)
        assert np.array_equal(fed.offsets_host, np.cumsum(counts) - counts)
        assert np.array_equal(fed.acs, np.bincount(mol_Xs[:, 0].astype(np.int64), minlength=4))
        got += 1
    assert got == len(want) == ds.num_batches(8)
    with pytest.raises(StopIteration):
        next(feeder)


def test_round_robin_hold_and_slot_reuse():
    """Two 'towers' on the host: batches alternate between the rings, a held batch is not
    overwritten while the submitter runs ahead, and many more batches than slots pass through."""
    ds = _dataset(n_mols=64, with_grads=False)
    want = list(ds.iterate(batch_size=4, shuffle=False))
    feeder = BatchFeeder(PackedDataset.from_raw(ds), 4, False, devices=[None, None], depth=1, hold=2)
    previous = None
    for k, fed in enumerate(feeder):
        assert np.array_equal(fed.x.numpy(), want[k][0][:, 1].astype(np.float32))
        if previous is not None:   # still intact although the submitter is ahead by now
            assert np.array_equal(previous.x.numpy(), want[k - 1][0][:, 1].astype(np.float32))
        assert fed.grads is None
        previous = fed
    assert k == len(want) - 1


def test_empty_dataset_and_packing_cache():
    ds = RawDataset([], [])
    assert list(BatchFeeder(PackedDataset.from_raw(ds), 8, False)) == []
    ds = _dataset(5)
    assert PackedDataset.from_raw(ds) is PackedDataset.from_raw(ds)
    assert PackedDataset.from_raw(ds, np.float64) is not PackedDataset.from_raw(ds)
    assert PackedDataset.from_raw(ds).capacity(2)[0] == sum(sorted(len(m) for m in ds.all_Xs)[-2:])


def test_submitter_errors_reach_the_consumer():
    ds = _dataset(9, with_grads=False)
    packed = PackedDataset.from_raw(ds)
    feeder = BatchFeeder(packed, 4, False)
    packed.types = packed.types[:3]          # corrupt the packed data: gather will fail
    with pytest.raises((ValueError, IndexError)):
        list(feeder)

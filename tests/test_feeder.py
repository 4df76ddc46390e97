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


def test_native_submitter_holds_reuses_and_survives_an_early_close():
    """One device and no fuzz: the submitter is the library's thread (ani_feeder_*).  A held batch stays intact
    while it runs ahead, a pass that is abandoned half way leaves the ring usable, and the next feeder on the
    same data set and shape takes the ring AND the native submitter over."""
    ds = _dataset(n_mols=64, with_grads=False)
    want = list(ds.iterate(batch_size=4, shuffle=False))
    packed = PackedDataset.from_raw(ds)
    feeder = BatchFeeder(packed, 4, False, depth=1, hold=2)
    assert feeder._native is not None
    handle = feeder._native["handle"].value
    previous = None
    for k, fed in enumerate(feeder):
        assert fed.index == k and np.array_equal(fed.x.numpy(), want[k][0][:, 1].astype(np.float32))
        if previous is not None:
            assert np.array_equal(previous.x.numpy(), want[k - 1][0][:, 1].astype(np.float32))
        previous = fed
        if k == 5:
            break
    feeder.close()                               # abandoned after six of sixteen batches
    feeder.close()
    for _ in range(3):                           # whole passes on the submitter that was kept with the ring
        feeder = BatchFeeder(packed, 4, False, depth=1, hold=2)
        assert feeder._native["handle"].value == handle
        got = [fed.x.numpy().copy() for fed in feeder]
        assert len(got) == len(want)
        assert all(np.array_equal(g, w[0][:, 1].astype(np.float32)) for g, w in zip(got, want))
    np.random.seed(11)
    shuffled = list(ds.iterate(batch_size=4, shuffle=True))
    np.random.seed(11)
    got = [fed.x.numpy().copy() for fed in BatchFeeder(packed, 4, True, depth=1, hold=2)]
    assert all(np.array_equal(g, w[0][:, 1].astype(np.float32)) for g, w in zip(got, shuffled))
    # another data set of the same shape on the same ring: a new submitter, the old one is retired
    other = PackedDataset(ds.all_Xs, ds.all_ys, None)
    feeder = BatchFeeder(other, 4, False, depth=1, hold=2)
    assert feeder._native["packed"] is other
    assert len(list(feeder)) == len(want)


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
    packed.ptr[-1] += 1000                   # corrupt the molecule table in place: the last batch cannot fit
    with pytest.raises((ValueError, IndexError)):
        list(feeder)
    feeder = BatchFeeder(packed, 4, False, fuzz=0.1)   # the same through the Python submitter
    with pytest.raises((ValueError, IndexError)):
        list(feeder)


@pytest.mark.parametrize("dtype", [np.float32, np.float64])
@pytest.mark.parametrize("source", [np.float32, np.float64])
def test_native_packer_matches_numpy_indexing(dtype, source):
    """ani_host_pack_batch against the numpy assembly of the same batch: every section of the
    arena bit for bit -- shuffled picks with repeats, with and without fuzz, empty molecules."""
    from khan_b200.data.feeder import HostSlot
    rng = np.random.default_rng(5)
    mols = [np.concatenate([rng.integers(0, 4, (n, 1)).astype(source), rng.normal(size=(n, 3)).astype(source)], axis=1)
            for n in rng.integers(0, 30, 50)]
    grads = [rng.normal(size=(len(m), 3)) for m in mols]
    packed = PackedDataset(mols, rng.normal(size=len(mols)), grads, dtype)
    assert packed.xyz.dtype == source
    cap = packed.capacity(16)
    a, b = HostSlot(cap[0], cap[1], dtype, pin=False), HostSlot(cap[0], cap[1], dtype, pin=False)
    for picks, fuzz in ((np.arange(16), None), (np.arange(40, 50), None), (rng.permutation(50)[:16], None),
                        (np.array([7, 7, 3, 49, 0]), 0.1), (np.zeros(0, np.int64), None), (rng.permutation(50)[:13], 0.05)):
        np.random.seed(3)
        packed.gather(picks, a, fuzz)
        np.random.seed(3)
        packed.gather_numpy(np.asarray(picks, np.int64), b, fuzz)
        n, m = b.n_atoms, b.n_mols
        assert (a.n_atoms, a.n_mols, a.has_ys, a.has_grads) == (n, m, True, True)
        assert np.array_equal(a.acs, b.acs)
        for name, used in (("xyz", n), ("grads", n)):
            assert np.array_equal(getattr(a, name)[:, :used], getattr(b, name)[:, :used]), name
        for name, used in (("types", n), ("mol_ids", n), ("mol_offsets", m), ("mol_counts", m), ("ys", m)):
            assert np.array_equal(getattr(a, name)[:used], getattr(b, name)[:used]), name


def test_native_packer_rejects_what_does_not_fit():
    from khan_b200.data.feeder import HostSlot
    ds = _dataset(9, with_grads=False)
    packed = PackedDataset.from_raw(ds)
    small = HostSlot(5, 9, np.float32, pin=False)
    with pytest.raises(ValueError):
        packed.gather(np.arange(9), small)
    slot = HostSlot(*packed.capacity(9), np.float32, pin=False)
    with pytest.raises(Exception) as info:
        packed.gather(np.array([0, 99]), slot)
    assert "ani_host_pack_batch" in str(info.value)
    with pytest.raises(ValueError):
        packed.gather(np.arange(3), HostSlot(*packed.capacity(9), np.float64, pin=False))


def test_fuzz_consumes_numpys_stream_like_the_reference():
    """The reference perturbs x of every atom of the batch, then y, then z, with three draws
    (khan/data/dataset.py:166-169); the same seed must give the same batch here, from RawDataset.iterate
    and from both assemblies of the packed data set."""
    from khan_b200 import RawDataset
    from khan_b200.data.feeder import HostSlot, PackedDataset
    b = syn.gdb_like_batch(9, 3)
    mols = b.molecules()
    raw = RawDataset(mols)
    flat = np.concatenate(mols, axis=0)
    np.random.seed(5)
    want = flat.copy()
    for col in (1, 2, 3):                       # the reference's three draws, in its order
        want[:, col] += np.random.uniform(-0.1, 0.1, want[:, col].shape)
    np.random.seed(5)
    got, _, _, _ = next(raw.iterate(len(mols), shuffle=False, fuzz=0.1))
    np.testing.assert_array_equal(got, want)
    packed = PackedDataset.from_raw(raw, np.float64)
    cap_a, cap_m = packed.capacity(len(mols))
    for assemble in (packed.gather, packed.gather_numpy):
        slot = HostSlot(cap_a, cap_m, np.float64, pin=False)
        np.random.seed(5)
        assemble(np.arange(len(mols)), slot, fuzz=0.1)
        np.testing.assert_array_equal(slot.xyz[:, :slot.n_atoms].T, want[:, 1:4])


def test_packed_copy_follows_replaced_lists_and_invalidate():
    from khan_b200 import RawDataset
    from khan_b200.data.feeder import PackedDataset
    mols = syn.gdb_like_batch(6, 4).molecules()
    raw = RawDataset(mols, [0.0] * len(mols))
    first = PackedDataset.from_raw(raw)
    assert PackedDataset.from_raw(raw) is first
    raw.all_ys = [1.0] * len(mols)              # a new list of targets: the packed copy is rebuilt
    second = PackedDataset.from_raw(raw)
    assert second is not first and float(second.ys[0]) == 1.0
    raw.all_ys[0] = 7.0                         # an edit in place is not seen until invalidate()
    assert PackedDataset.from_raw(raw) is second
    PackedDataset.invalidate(raw)
    assert float(PackedDataset.from_raw(raw).ys[0]) == 7.0

"""Packed datasets and a double-buffered, pinned batch feeder.

The reference assembles every batch in Python from per-molecule arrays
(``khan/data/dataset.py:144-183``) and pushes it through ``feed_dict`` into a TensorFlow queue
from a submitter thread (``khan/training/trainer_multi_tower.py:749-828``); that path, not the
featurizer, bounds its throughput.  Here

* :class:`PackedDataset` concatenates the molecules ONCE into CSR form (``ptr`` + flat element
  ids + ``[3, N]`` coordinates), so a batch is one call of the library's host packer
  (``ani_host_pack_batch``: a per-molecule copy loop in C++) -- no Python work per molecule;
* :class:`BatchFeeder` runs a submitter thread that writes each batch into one pinned host
  arena and moves it to the device with ONE asynchronous copy on a copy stream, ``depth``
  batches ahead of the consumer, handing over with CUDA events.

The batch contents and their order are exactly those of ``RawDataset.iterate`` (same use of
``numpy.random`` for the shuffle and the fuzz), which the tests check.  Without CUDA (device
``None``) the feeder yields the host arrays, which is how the CPU tests run it.
"""
from __future__ import annotations

import ctypes
import queue
import threading

import numpy as np
import torch

from .. import _lib

_ALIGN = 256


class PackedDataset:
    """All molecules of a ``RawDataset`` in CSR form."""

    def __init__(self, all_Xs, all_ys=None, all_grads=None, dtype=np.float32):
        self.dtype = np.dtype(dtype)
        n_mols = len(all_Xs)
        self.counts = np.fromiter((len(m) for m in all_Xs), dtype=np.int64, count=n_mols)
        self.ptr = np.zeros(n_mols + 1, np.int64)
        np.cumsum(self.counts, out=self.ptr[1:])
        self._mol_acs = None
        cat = np.concatenate(all_Xs, axis=0) if n_mols else np.zeros((0, 4))
        self.types = np.ascontiguousarray(cat[:, 0].astype(np.int32))
        # coordinates stay in the precision they were given in; the cast to `dtype` happens per
        # batch, after the fuzz, which is where RawDataset.iterate + the feed would round them
        self.xyz = np.ascontiguousarray(cat[:, 1:4].T)                          # [3, N]
        self.ys = None if all_ys is None else np.asarray(all_ys, dtype=self.dtype).reshape(n_mols)
        if all_grads is None:
            self.grads = None
        else:
            g = np.concatenate(all_grads, axis=0) if n_mols else np.zeros((0, 3))
            self.grads = np.ascontiguousarray(g.T.astype(self.dtype))           # [3, N]

    @classmethod
    def from_raw(cls, raw, dtype=np.float32) -> "PackedDataset":
        """Packs ``raw`` once per precision and keeps the result on the RawDataset object.  The packed copy
        is a SNAPSHOT: it is rebuilt when one of the three lists is replaced or changes its length, but an
        edit of an array inside them (say, subtracting an offset from ``all_ys`` in place) is not seen --
        call ``PackedDataset.invalidate(raw)`` after such an edit."""
        cache = raw.__dict__.setdefault("_packed", {})
        key = np.dtype(dtype).name

        def stamp():
            return tuple((id(lst), None if lst is None else len(lst)) for lst in (raw.all_Xs, raw.all_ys, raw.all_grads))

        if key not in cache or cache[key][0] != stamp():
            cache[key] = (stamp(), cls(raw.all_Xs, raw.all_ys, raw.all_grads, dtype), raw.all_Xs, raw.all_ys,
                          raw.all_grads)        # the lists are kept alive so that their ids stay theirs
        return cache[key][1]

    @staticmethod
    def invalidate(raw) -> None:
        """Forgets the packed copies of ``raw`` (after its arrays were edited in place)."""
        raw.__dict__.pop("_packed", None)

    def num_mols(self) -> int:
        return len(self.counts)

    def num_batches(self, batch_size: int) -> int:
        return -(-self.num_mols() // batch_size)

    def capacity(self, batch_size: int):
        """(atoms, molecules) that any batch of ``batch_size`` molecules fits in."""
        k = min(batch_size, self.num_mols())
        top = np.sort(self.counts)[-k:] if k else np.zeros(0, np.int64)
        return int(top.sum()), k

    def batch_slices(self, batch_size: int):
        """For an UNSHUFFLED pass: per batch, the row range of every molecule within the batch, as ready-made
        ``slice`` objects (cutting a batch result into per-molecule arrays is a third faster with them than
        with freshly built slices; made once per data set and batch size)."""
        cache = self.__dict__.setdefault("_batch_slices", {})
        if batch_size not in cache:
            ptr = self.ptr.tolist()
            n = self.num_mols()
            cache[batch_size] = [[slice(ptr[m] - ptr[b0], ptr[m + 1] - ptr[b0]) for m in range(b0, min(b0 + batch_size, n))]
                                 for b0 in range(0, n, batch_size)]
        return cache[batch_size]

    def mol_acs(self) -> np.ndarray:
        """Atoms per element of every molecule ``[n_mols, 4]``, counted once per data set."""
        if self._mol_acs is None:
            ok = (self.types >= 0) & (self.types < 4)
            mol_of = np.repeat(np.arange(self.num_mols()), self.counts)
            acs = np.zeros((self.num_mols(), 4), np.int32)
            np.add.at(acs, (mol_of[ok], self.types[ok]), 1)
            self._mol_acs = acs
        return self._mol_acs

    def check_shapes(self, slot: "HostSlot") -> None:
        total = int(self.ptr[-1])
        if (self.types.shape[0] != total or self.xyz.shape != (3, total) or slot.np_dtype != self.dtype
                or (self.grads is not None and self.grads.shape != (3, total))
                or (self.ys is not None and self.ys.shape[0] != self.num_mols())):
            raise ValueError("the arrays of the packed dataset do not match its molecule table")

    def fill_pack_args(self, a, slot: "HostSlot") -> None:
        """The fields of an ``ani_host_pack_args`` that depend only on (data set, slot)."""
        a.n_mols_total, a.mol_ptr = self.num_mols(), self.ptr.ctypes.data
        a.src_xyz, a.src_stride = self.xyz.ctypes.data, self.xyz.shape[1]
        a.src_is_f64 = int(self.xyz.dtype == np.float64)
        a.src_types = self.types.ctypes.data
        a.src_ys = None if self.ys is None else self.ys.ctypes.data
        a.src_grads = None if self.grads is None else self.grads.ctypes.data
        a.src_mol_acs = self.mol_acs().ctypes.data
        a.dst_xyz, a.dst_grads, a.dst_ys = slot.xyz.ctypes.data, slot.grads.ctypes.data, slot.ys.ctypes.data
        a.dst_stride, a.dst_is_f64 = slot.cap_atoms, int(slot.np_dtype == np.float64)
        a.dst_types, a.dst_mol_ids = slot.types.ctypes.data, slot.mol_ids.ctypes.data
        a.dst_mol_offsets, a.dst_mol_counts = slot.mol_offsets.ctypes.data, slot.mol_counts.ctypes.data
        a.cap_atoms, a.cap_mols = slot.cap_atoms, slot.cap_mols

    def gather(self, picks: np.ndarray, slot: "HostSlot", fuzz=None) -> None:
        """Writes the batch made of molecules ``picks`` (in that order) into ``slot``: one call of
        the library's host packer (``ani_host_pack_batch``), a per-molecule copy loop in C++."""
        picks = np.ascontiguousarray(picks, dtype=np.int64)
        m = len(picks)
        if m > slot.cap_mols:
            raise ValueError("batch larger than the slot")
        self.check_shapes(slot)
        noise = None
        if fuzz is not None:   # same draws as RawDataset.iterate: x of all atoms, then y, then z
            n = int(self.counts[picks].sum())
            noise = np.ascontiguousarray(np.random.uniform(-fuzz, fuzz, (3, n)).T)
        cached = slot.pack_args
        if cached is None or cached[0] is not self:
            # everything that depends only on (data set, slot) is written once; a batch changes four fields
            a = _lib.HostPackArgs()
            self.fill_pack_args(a, slot)
            n_atoms = ctypes.c_int(0)
            a.n_atoms_out, a.acs_out = ctypes.addressof(n_atoms), slot.acs.ctypes.data
            cached = slot.pack_args = (self, a, n_atoms, (self.xyz, self.types, self.ys, self.grads, self.ptr))
        _, a, n_atoms, _ = cached
        a.picks, a.n_picks = picks.ctypes.data, m
        a.noise = None if noise is None else noise.ctypes.data
        status = _lib.lib().ani_host_pack_batch(ctypes.byref(a))
        if status == -2:
            raise ValueError("batch larger than the slot")
        _lib.check(status, "ani_host_pack_batch")
        slot.n_atoms, slot.n_mols = int(n_atoms.value), m
        slot.has_ys, slot.has_grads = self.ys is not None, self.grads is not None

    def gather_numpy(self, picks: np.ndarray, slot: "HostSlot", fuzz=None) -> None:
        """The same batch assembled with numpy indexing -- what ``gather`` is tested against."""
        counts = self.counts[picks]
        m = len(picks)
        n = int(counts.sum())
        if n > slot.cap_atoms or m > slot.cap_mols:
            raise ValueError("batch larger than the slot")
        offsets = np.cumsum(counts) - counts
        in_order = m > 0 and np.array_equal(picks, np.arange(picks[0], picks[0] + m))
        if in_order:
            src = slice(int(self.ptr[picks[0]]), int(self.ptr[picks[0]]) + n)
        else:
            src = np.repeat(self.ptr[picks] - offsets, counts) + np.arange(n)
        slot.n_atoms, slot.n_mols = n, m
        if fuzz is None:
            slot.xyz[:, :n] = self.xyz[:, src]
        else:   # same draws as RawDataset.iterate: x of all atoms, then y, then z
            slot.xyz[:, :n] = self.xyz[:, src] + np.random.uniform(-fuzz, fuzz, (3, n))
        slot.types[:n] = self.types[src]
        slot.mol_offsets[:m] = offsets
        slot.mol_counts[:m] = counts
        slot.mol_ids[:n] = np.repeat(np.arange(m), counts)
        slot.has_ys = self.ys is not None
        if slot.has_ys:
            slot.ys[:m] = self.ys[picks]
        slot.has_grads = self.grads is not None
        if slot.has_grads:
            slot.grads[:, :n] = self.grads[:, src]
        slot.acs = np.bincount(slot.types[:n], minlength=4).astype(np.int32)


def _layout(cap_atoms: int, cap_mols: int, itemsize: int):
    """Byte offsets of the sections of a slot; every section starts on a 256-byte boundary."""
    sections = [("xyz", 3 * cap_atoms * itemsize), ("grads", 3 * cap_atoms * itemsize),
                ("ys", cap_mols * itemsize), ("mol_ids", cap_atoms * 8), ("types", cap_atoms * 4),
                ("mol_offsets", cap_mols * 4), ("mol_counts", cap_mols * 4)]
    table, off = {}, 0
    for name, size in sections:
        table[name] = (off, size)
        off += -(-size // _ALIGN) * _ALIGN
    return table, max(off, _ALIGN)


class HostSlot:
    """One batch in one (pinned, when CUDA is available) host arena, with numpy views."""

    def __init__(self, cap_atoms: int, cap_mols: int, dtype, pin: bool):
        self.cap_atoms, self.cap_mols = cap_atoms, cap_mols
        self.pack_args = None       # argument block of the host packer for the data set last gathered into this slot
        self.np_dtype = np.dtype(dtype)
        self.table, self.nbytes = _layout(cap_atoms, cap_mols, self.np_dtype.itemsize)
        self.arena = torch.zeros(self.nbytes, dtype=torch.uint8)
        if pin:
            self.arena = self.arena.pin_memory()
        raw = self.arena.numpy()

        def view(name, dt, shape):
            off, size = self.table[name]
            return raw[off:off + size].view(dt).reshape(shape)

        self.xyz = view("xyz", self.np_dtype, (3, cap_atoms))
        self.grads = view("grads", self.np_dtype, (3, cap_atoms))
        self.ys = view("ys", self.np_dtype, (cap_mols,))
        self.mol_ids = view("mol_ids", np.int64, (cap_atoms,))
        self.types = view("types", np.int32, (cap_atoms,))
        self.mol_offsets = view("mol_offsets", np.int32, (cap_mols,))
        self.mol_counts = view("mol_counts", np.int32, (cap_mols,))
        self.n_atoms = self.n_mols = 0
        self.has_ys = self.has_grads = False
        self.acs = np.zeros(4, np.int32)


def arena_views(host: "HostSlot", arena: torch.Tensor) -> dict:
    """Full-capacity typed views of the arrays laid out in ``arena`` (a device or host copy of the slot's
    arena).  Built once per slot: a batch only slices them."""
    tdt = torch.float32 if host.np_dtype == np.float32 else torch.float64

    def view(name, dt, rows):
        off, size = host.table[name]
        t = arena[off:off + size].view(dt)
        return t.view(rows, host.cap_atoms) if rows > 1 else t

    return {"xyz": view("xyz", tdt, 3), "types": view("types", torch.int32, 1),
            "mol_offsets": view("mol_offsets", torch.int32, 1), "mol_counts": view("mol_counts", torch.int32, 1),
            "mol_ids": view("mol_ids", torch.int64, 1), "ys": view("ys", tdt, 1), "grads": view("grads", tdt, 3)}


class FedBatch:
    """What the feeder hands to the consumer: tensors of one batch (device tensors when the
    feeder has a device, host tensors otherwise) plus the host-side sizes the C ABI needs."""

    def __init__(self, index: int, device, host: HostSlot, arena: torch.Tensor, ready, views=None, waiter=None):
        self.index, self.device, self.ready = index, device, ready
        self._waiter = waiter    # native submitter: makes a stream wait for the slot's upload
        n, m = host.n_atoms, host.n_mols
        self.n_atoms, self.n_mols = n, m
        self.acs = host.acs.copy()
        self.offsets_host = host.mol_offsets[:m].copy()
        self.counts_host = host.mol_counts[:m].copy()
        v = views if views is not None else arena_views(host, arena)
        xyz = v["xyz"]
        self.x, self.y, self.z = xyz[0, :n], xyz[1, :n], xyz[2, :n]          # each one contiguous range
        self.types = v["types"][:n]
        self.mol_offsets = v["mol_offsets"][:m]
        self.mol_counts = v["mol_counts"][:m]
        self.mol_ids = v["mol_ids"][:n]
        self.ys = v["ys"][:m] if host.has_ys else None
        self.grads = v["grads"][:, :n] if host.has_grads else None

    def wait(self) -> None:
        """Makes the current stream of the batch's device wait for the upload."""
        if self._waiter is not None:
            self._waiter()
        elif self.ready is not None:
            torch.cuda.current_stream(self.device).wait_event(self.ready)


# Slot rings (pinned host arenas + device arenas) of finished feeders, kept for the next feeder of the same
# shape: allocating pinned memory costs milliseconds, more than a whole pass over a small data set.
_ring_lock = threading.Lock()
_ring_cache: dict = {}
_RING_CACHE_MAX = 4


def _ring_key(dev, cap_atoms, cap_mols, dtype, depth):
    return (None if dev is None else (torch.device(dev).type, torch.device(dev).index), cap_atoms, cap_mols,
            np.dtype(dtype).name, depth)


def _take_ring(dev, cap_atoms, cap_mols, dtype, depth):
    key = _ring_key(dev, cap_atoms, cap_mols, dtype, depth)
    with _ring_lock:
        ring = _ring_cache.pop(key, None)
    if ring is not None:
        return ring
    ring = []
    for _ in range(depth + 1):
        host = HostSlot(cap_atoms, cap_mols, dtype, pin=dev is not None)
        arena = torch.empty(host.nbytes, dtype=torch.uint8, device=dev) if dev is not None else host.arena
        ring.append({"host": host, "arena": arena, "consumed": None, "uploaded": None,
                     "views": arena_views(host, arena)})
    return ring


def _give_ring(dev, cap_atoms, cap_mols, dtype, depth, ring):
    key = _ring_key(dev, cap_atoms, cap_mols, dtype, depth)
    with _ring_lock:
        if key not in _ring_cache and len(_ring_cache) >= _RING_CACHE_MAX:
            _drop_native(_ring_cache.pop(next(iter(_ring_cache))))   # its copies finish before its arenas go
        elif key in _ring_cache and _ring_cache[key] is not ring:
            _drop_native(_ring_cache[key])
        _ring_cache[key] = ring


class _NativeHandle:
    """Owns one ``ani_feeder`` of the library; destroyed (after its copies have finished) with the object."""

    def __init__(self, device_index: int, slots_array, n: int):
        self.ptr = ctypes.c_void_p()
        _lib.check(_lib.lib().ani_feeder_create(device_index, ctypes.addressof(slots_array), n, ctypes.byref(self.ptr)),
                   "ani_feeder_create")

    def __del__(self):
        if self.ptr:
            _lib.lib().ani_feeder_destroy(self.ptr)
            self.ptr = ctypes.c_void_p()


def _drop_native(ring) -> None:
    """Before a ring goes to the Python submitter: the native one is stopped and its copies have finished."""
    nat = ring[0].pop("native", None)
    if nat is not None:
        nat["owner"].__del__()


def _native_submitter(ring, packed: "PackedDataset", dev) -> dict:
    """The native submitter bound to (ring, data set), made once and kept with the ring."""
    nat = ring[0].get("native")
    if nat is not None and nat["packed"] is packed:
        return nat
    _drop_native(ring)
    for slot in ring:       # what a Python submitter left behind on these slots
        for key in ("consumed", "uploaded"):
            if slot[key] is not None:
                slot[key].synchronize()
                slot[key] = None
    n = len(ring)
    arr = (_lib.FeederSlot * n)()
    for k, slot in enumerate(ring):
        host = slot["host"]
        packed.check_shapes(host)
        packed.fill_pack_args(arr[k].pack, host)
        arr[k].host_arena = host.arena.data_ptr()
        arr[k].dev_arena = None if dev is None else slot["arena"].data_ptr()
        arr[k].nbytes = host.nbytes
        host.pack_args = None
    index = -1 if dev is None else (torch.device(dev).index if torch.device(dev).index is not None
                                    else torch.cuda.current_device())
    owner = _NativeHandle(index, arr, n)
    nat = {"owner": owner, "handle": owner.ptr, "packed": packed, "slots": arr, "batch": _lib.FeederBatch(),
           "order": None, "keep": (packed.xyz, packed.types, packed.ys, packed.grads, packed.ptr, packed.mol_acs())}
    ring[0]["native"] = nat
    return nat


class BatchFeeder:
    """Iterates a dataset as ``FedBatch`` objects, ``depth`` batches ahead of the consumer.

    ``devices``: list of CUDA devices; batch b goes to ``devices[b % len(devices)]`` (the
    reference's round-robin over towers, ``trainer_multi_tower.py:753-767``).  ``None`` keeps the
    batches on the host.  The consumer keeps at most ``hold`` batches alive (one per device by
    default): advancing the iterator past that releases the oldest one, whose work must have been
    enqueued on its device's current stream by then; :meth:`release` does it earlier.  Each
    device has ``depth + 1`` slots, so the submitter runs up to ``depth`` batches ahead.
    """

    def __init__(self, packed: PackedDataset, batch_size: int, shuffle: bool, fuzz=None, devices=None,
                 depth: int = 2, hold=None):
        self.packed, self.batch_size, self.shuffle, self.fuzz = packed, batch_size, shuffle, fuzz
        self.devices = list(devices) if devices else [None]
        self.depth = max(1, depth)
        self.hold = max(1, hold if hold is not None else len(self.devices))
        cap_atoms, cap_mols = packed.capacity(batch_size)
        cap_atoms, cap_mols = max(cap_atoms, 1), max(cap_mols, 1)
        self._shape = (cap_atoms, cap_mols, packed.dtype)
        self._slots = [_take_ring(dev, cap_atoms, cap_mols, packed.dtype, self.depth) for dev in self.devices]
        self._copy_streams = [torch.cuda.Stream(device=d) if d is not None else None for d in self.devices]
        self._ready = queue.Queue(maxsize=self.depth * len(self.devices))
        self._free = [queue.Queue() for _ in self.devices]
        for t, ring in enumerate(self._slots):
            for s in range(len(ring)):
                self._free[t].put(s)
        self._error = None
        self._stop = threading.Event()
        self._thread = threading.Thread(target=self._submit, name="khan-b200-feeder", daemon=True)
        self._started = False
        self._finished = False
        self._held = []
        # One device and no fuzz (whose draws come from numpy's global generator, batch by batch): the
        # submitter is the library's native thread, and the interpreter lock stays with the consumer.
        self._native = None
        if fuzz is None and len(self.devices) == 1:
            self._native = _native_submitter(self._slots[0], packed, self.devices[0])
        else:
            for ring in self._slots:
                _drop_native(ring)

    # ---- submitter thread ---------------------------------------------------------------
    def _take_free(self, tower: int):
        while not self._stop.is_set():
            try:
                return self._free[tower].get(timeout=0.1)
            except queue.Empty:
                continue
        return None

    def _submit(self) -> None:
        try:
            p = self.packed
            perm = np.arange(p.num_mols())
            if self.shuffle:
                np.random.shuffle(perm)
            for b in range(p.num_batches(self.batch_size)):
                tower = b % len(self.devices)
                s = self._take_free(tower)
                if s is None:
                    return
                slot = self._slots[tower][s]
                if slot["consumed"] is not None:
                    slot["consumed"].synchronize()     # the consumer's kernels on this slot are done
                    slot["consumed"] = None
                if slot["uploaded"] is not None:
                    slot["uploaded"].synchronize()     # the pinned arena may be rewritten only after its last copy
                    slot["uploaded"] = None
                picks = perm[b * self.batch_size: min((b + 1) * self.batch_size, p.num_mols())]
                p.gather(picks, slot["host"], self.fuzz)
                dev, ready = self.devices[tower], None
                if dev is not None:
                    with torch.cuda.stream(self._copy_streams[tower]):
                        slot["arena"].copy_(slot["host"].arena, non_blocking=True)
                        ready = torch.cuda.Event()
                        ready.record()
                fed = FedBatch(b, dev, slot["host"], slot["arena"], ready, slot["views"])
                slot["uploaded"] = ready
                self._put((tower, s, fed))
            self._put(None)
        except BaseException as exc:   # handed to the consumer, which re-raises it
            self._error = exc
            self._put(None)

    def _put(self, item) -> None:
        while not self._stop.is_set():
            try:
                self._ready.put(item, timeout=0.1)
                return
            except queue.Full:
                continue

    # ---- consumer side ------------------------------------------------------------------
    def __iter__(self):
        return self

    def _stream_ptr(self):
        dev = self.devices[0]
        return None if dev is None else ctypes.c_void_p(torch.cuda.current_stream(dev).cuda_stream)

    def _next_native(self) -> FedBatch:
        nat, p, L = self._native, self.packed, _lib.lib()
        if not self._started:
            self._started = True
            perm = np.arange(p.num_mols(), dtype=np.int64)
            if self.shuffle:
                np.random.shuffle(perm)
            nat["order"] = perm     # read by the native thread until the pass ends
            _lib.check(L.ani_feeder_begin(nat["handle"], perm.ctypes.data, len(perm), self.batch_size),
                       "ani_feeder_begin")
        while len(self._held) >= self.hold:
            self.release(self._held[0][2])
        fb = nat["batch"]
        rc = L.ani_feeder_next(nat["handle"], ctypes.byref(fb))
        if rc <= 0:
            self._finished = True
            self.close()
            if rc == -2:
                raise ValueError("batch larger than the slot")
            _lib.check(rc, "ani_feeder_next")
            raise StopIteration
        s = fb.slot
        slot = self._slots[0][s]
        host = slot["host"]
        host.n_atoms, host.n_mols = fb.n_atoms, fb.n_mols
        host.acs[:] = fb.acs
        host.has_ys, host.has_grads = p.ys is not None, p.grads is not None
        dev = self.devices[0]
        waiter = None
        if dev is not None:
            handle = nat["handle"]

            def waiter(s=s):
                _lib.check(L.ani_feeder_wait(handle, s, self._stream_ptr()), "ani_feeder_wait")
        fed = FedBatch(int(fb.batch_index), dev, host, slot["arena"], None, slot["views"], waiter)
        self._held.append((0, s, fed))
        return fed

    def __next__(self) -> FedBatch:
        if self._finished:
            raise StopIteration
        if self._native is not None:
            return self._next_native()
        if not self._started:
            self._started = True
            self._thread.start()
        while len(self._held) >= self.hold:
            self.release(self._held[0][2])
        item = self._ready.get()
        if item is None:
            self._finished = True
            self.close()
            if self._error is not None:
                raise self._error
            raise StopIteration
        self._held.append(item)
        return item[2]

    def release(self, fed: FedBatch) -> None:
        """Gives the batch's buffers back to the submitter (after the work enqueued so far)."""
        for k, (tower, s, f) in enumerate(self._held):
            if f is fed:
                del self._held[k]
                if self._native is not None:
                    _lib.check(_lib.lib().ani_feeder_release(self._native["handle"], s, self._stream_ptr()),
                               "ani_feeder_release")
                    return
                if fed.device is not None:
                    evt = torch.cuda.Event()
                    evt.record(torch.cuda.current_stream(fed.device))
                    self._slots[tower][s]["consumed"] = evt
                self._free[tower].put(s)
                return

    def close(self) -> None:
        """Stops the submitter and hands the slot rings to the next feeder of the same shape.  Call it after
        the work on the last batches has been enqueued (the iterator does so when it is exhausted)."""
        if self._native is not None:
            if self._slots is None:
                return
            _lib.lib().ani_feeder_end(self._native["handle"])
            for _, _, fed in list(self._held):
                self.release(fed)
            self._native["order"] = None
            _give_ring(self.devices[0], *self._shape, self.depth, self._slots[0])
            self._slots = None
            return
        self._stop.set()
        if self._started and self._thread.is_alive() and threading.current_thread() is not self._thread:
            self._thread.join(timeout=5)
        if self._slots is None or (self._started and self._thread.is_alive()):
            return
        for _, _, fed in list(self._held):      # what is still held counts as consumed from here on
            self.release(fed)
        while True:                             # batches the submitter had prepared but nobody took
            try:
                self._ready.get_nowait()
            except queue.Empty:
                break
        for dev, ring in zip(self.devices, self._slots):
            _give_ring(dev, *self._shape, self.depth, ring)
        self._slots = None

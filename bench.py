"""Benchmark of the ANI-1 AEV hot path: ani_sort -> featurize -> featurize_grad, float32, on
1024-molecule GDB8-like batches (synthetic, seeded), in atoms per second.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

One "step" is one pass of the hot path over one 1024-molecule batch.  The run keeps NB distinct
batches resident in HBM (NB x ~43 MB of inputs and outputs, far more than the 126 MB L2) and
cycles through them, so consecutive steps never find their data in L2.

Printed keys (one JSON line, rank 0):
  value        whole-job atoms/s with every input already in HBM, steps replayed as CUDA graphs,
               timed with CUDA events, max over ranks
  e2e          the same metric through the C ABI with HOST buffers: every step copies its
               inputs (coordinates, element ids, molecule table, upstream dL/dAEV) from pinned
               host memory and copies features and coordinate gradients back
  roofline     HBM roofline of the dominant kernel (algorithmic bytes per launch / its average
               duration, timed live with CUDA events; peak = measured copy bandwidth)
  roofline_fp32  the same kernel's algorithmic flop/s against the FP32 FMA peak
  kernels      average launch duration of each kernel of the step
  cpu_baseline the reference's CPU kernels (oracle/_ref) or the CPU port, all host threads, on a
               bounded sample of the same workload (N=1 only)
  clocks       SM clock / throttle reasons sampled through NVML while the GPU was under load

With --impl reference the script times only the reference's CPU implementation of the path
(all host threads) and prints the same line with "impl": "reference".
"""
from __future__ import annotations

import argparse
import ctypes
import json
import os
import statistics
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import numpy as np  # noqa: E402

METRIC = "AEV fwd+grad atoms/sec (fp32, 1024-mol batch)"
UNIT = "atoms/s"
N_MOLS = 1024
FEATURE_SIZE = 384
# algorithmic work per unit: radial pair / angular triplet, forward and gradient
FLOPS_FWD = (125, 156)
FLOPS_GRAD = (201, 417)
FP32_PEAK_TFLOPS = 148 * 128 * 2 * 1.965e9 / 1e12  # SMs x lanes x FMA x max SM clock
# DRAM bytes per atom that ncu saw (dram__bytes_read.sum + dram__bytes_write.sum) for the kernels
# named in NCU_TRAFFIC_SOURCE, on an 8192-molecule batch whose 170 MB of features exceed the L2;
# traffic grows in proportion to the atoms, so a launch is scaled by its atom count.  The numbers
# belong to those kernels: when a kernel changes, the capture has to be repeated.
NCU_DRAM_BYTES_PER_ATOM = {"featurize": 1063.3, "featurize_grad": 1563.9, "ani_sort": None}
NCU_TRAFFIC_SOURCE = ("one ncu capture of featurize_mol_kernel / featurize_grad_mol_kernel (a molecule per warp / per "
                      "CTA), 8192-molecule batch, scaled by atoms")


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            return json.load(f), "measured"
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}, "fallback"


_probe_lib = None


def probe_lib():
    """libbench_probe.so (built from bench_probe.cu by __graft_entry__.build())."""
    global _probe_lib
    if _probe_lib is None:
        path = os.path.join(ROOT, "libbench_probe.so")
        if not os.path.exists(path):
            import __graft_entry__
            __graft_entry__.build_bench_probe()
        _probe_lib = ctypes.CDLL(path)
        _probe_lib.bench_fma_probe.restype = ctypes.c_int
        _probe_lib.bench_fma_probe.argtypes = [ctypes.c_int, ctypes.c_int, ctypes.c_void_p,
                                               ctypes.POINTER(ctypes.c_longlong), ctypes.c_void_p]
    return _probe_lib


_fma_peak_cache = {}


def measure_fma_peak(bits: int, device) -> float:
    """TFLOP/s of the FMA-only probe kernel (bench_probe.cu), best of 5 launches (CUDA events)."""
    import torch
    if bits in _fma_peak_cache:
        return _fma_peak_cache[bits]
    lib = probe_lib()
    sink = torch.zeros(2, dtype=torch.float64, device=device)
    flops = ctypes.c_longlong(0)
    st = torch.cuda.current_stream()
    iters = 16384 if bits == 32 else 8192
    best = 0.0
    for rep in range(6):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        rc = lib.bench_fma_probe(bits, iters, sink.data_ptr(), ctypes.byref(flops), st.cuda_stream)
        if rc != 0:
            raise RuntimeError(f"bench_fma_probe failed ({rc})")
        e1.record()
        torch.cuda.synchronize()
        if rep:
            best = max(best, flops.value / (e0.elapsed_time(e1) * 1e-3) / 1e12)
    _fma_peak_cache[bits] = best
    return best


def _parse_cpulist(text):
    cpus = set()
    for part in text.strip().split(","):
        if "-" in part:
            lo, hi = part.split("-")
            cpus.update(range(int(lo), int(hi) + 1))
        elif part:
            cpus.add(int(part))
    return cpus


def bind_near_gpu(local_rank, n_local):
    """Restrict this process to host cores on the GPU's own NUMA node, before any pinned buffer is
    allocated (pages are placed where they are first touched) and share those cores evenly with the
    other ranks whose GPUs hang off the same node.  Reads sysfs only; returns a short record for the
    result line, or None where the topology cannot be read (then nothing is changed)."""
    import torch
    try:
        allowed = os.sched_getaffinity(0)
        local = []
        for i in range(n_local):
            p = torch.cuda.get_device_properties(i)
            bus = "%04x:%02x:%02x.0" % (p.pci_domain_id, p.pci_bus_id, p.pci_device_id)
            with open("/sys/bus/pci/devices/%s/local_cpulist" % bus) as f:
                local.append(frozenset(_parse_cpulist(f.read()) & allowed))
        mine = local[local_rank]
        sharers = [i for i in range(n_local) if local[i] == mine]
        cpus = sorted(mine)[sharers.index(local_rank)::len(sharers)]
        if not cpus:
            return None
        os.sched_setaffinity(0, cpus)
        return {"cores": len(cpus), "node_cores": len(mine), "ranks_on_node": len(sharers)}
    except (OSError, AttributeError, ValueError, IndexError, RuntimeError):
        return None


class Ctx:
    """Rank, device and process group of this process (one rank per GPU under torchrun)."""

    def __init__(self):
        import torch
        import torch.distributed as dist
        self.rank = int(os.environ.get("RANK", "0"))
        self.world = int(os.environ.get("WORLD_SIZE", "1"))
        self.local_rank = int(os.environ.get("LOCAL_RANK", "0"))
        assert torch.cuda.is_available(), "bench.py needs a CUDA device (there is no CPU fallback)"
        self.host_binding = bind_near_gpu(self.local_rank, self.world) if self.world > 1 else None
        torch.cuda.set_device(self.local_rank)
        self.dev = torch.device("cuda", self.local_rank)
        if self.world > 1 and not dist.is_initialized():
            dist.init_process_group("nccl", device_id=self.dev)

    def barrier(self):
        import torch.distributed as dist
        if self.world > 1:
            dist.barrier()

    def max_sum(self, ms: float, units: float):
        """(max over ranks of a time, sum over ranks of a count)."""
        import torch
        import torch.distributed as dist
        if self.world == 1:
            return float(ms), float(units)
        t = torch.tensor([ms, units], dtype=torch.float64, device=self.dev)
        tmax = t.clone()
        dist.all_reduce(tmax, op=dist.ReduceOp.MAX)
        dist.all_reduce(t, op=dist.ReduceOp.SUM)
        return float(tmax[0]), float(t[1])

    def close(self):
        import torch.distributed as dist
        if self.world > 1 and dist.is_initialized():
            dist.destroy_process_group()


# ------------------------------------------------------------------------------------------
# clocks
# ------------------------------------------------------------------------------------------
class ClockSampler:
    """Samples SM clock and throttle reasons of one GPU through NVML (read-only) in a thread."""

    REASONS = {
        0x8: "hw_slowdown", 0x40: "hw_thermal_slowdown", 0x20: "sw_thermal_slowdown",
        0x4: "sw_power_cap", 0x80: "hw_power_brake", 0x2: "applications_clocks_setting",
    }

    def __init__(self, torch_index: int, period: float = 0.02):
        self.samples = []
        self.period = period
        self._stop = threading.Event()
        self._thread = None
        self.sm_max = None
        try:
            import pynvml
            import torch
            pynvml.nvmlInit()
            uuid = str(torch.cuda.get_device_properties(torch_index).uuid)
            if not uuid.startswith("GPU-"):
                uuid = "GPU-" + uuid
            self.nv = pynvml
            self.handle = pynvml.nvmlDeviceGetHandleByUUID(uuid.encode())
            self.sm_max = int(pynvml.nvmlDeviceGetMaxClockInfo(self.handle, pynvml.NVML_CLOCK_SM))
        except Exception as exc:  # NVML missing: clocks are reported as unavailable
            self.nv = None
            self.error = repr(exc)

    def _run(self):
        nv = self.nv
        while not self._stop.is_set():
            try:
                mhz = int(nv.nvmlDeviceGetClockInfo(self.handle, nv.NVML_CLOCK_SM))
                reasons = int(nv.nvmlDeviceGetCurrentClocksEventReasons(self.handle))
                power = nv.nvmlDeviceGetPowerUsage(self.handle) / 1000.0
                self.samples.append((time.perf_counter(), mhz, reasons, power))
            except Exception:
                pass
            self._stop.wait(self.period)

    def start(self):
        if self.nv is not None:
            self._thread = threading.Thread(target=self._run, daemon=True)
            self._thread.start()

    def stop(self):
        self._stop.set()
        if self._thread is not None:
            self._thread.join()

    def summary(self, t0: float, t1: float):
        if self.nv is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "note": "NVML unavailable"}
        window = [s for s in self.samples if t0 <= s[0] <= t1] or self.samples
        if not window:
            return {"sm_mhz": None, "sm_max_mhz": self.sm_max, "reasons": [], "samples": 0}
        bits = 0
        for s in window:
            bits |= s[2]
        reasons = [name for bit, name in self.REASONS.items() if bits & bit]
        return {"sm_mhz": int(statistics.median(s[1] for s in window)), "sm_max_mhz": self.sm_max,
                "reasons": reasons, "samples": len(window),
                "power_w_max": round(max(s[3] for s in window), 1)}


# ------------------------------------------------------------------------------------------
# CPU arms
# ------------------------------------------------------------------------------------------
def cpu_fwd_grad(oracle, impl, batch, up, threads):
    """One pass of the reference CPU path on one batch (float32): sort, forward, gradient."""
    x, y, z = batch.coords(np.float32)
    si, gi, ac = oracle.ani_sort(batch.atomic_numbers)
    args = (batch.atomic_numbers, batch.mol_offsets, batch.mol_atom_counts, si, ac)
    oracle.featurize(x, y, z, *args, impl=impl, threads=threads)
    oracle.featurize_grad(x, y, z, *args, *up, impl=impl, threads=threads)


def cpu_baseline(batch, budget_s: float = 12.0):
    import oracle
    from khan_b200.data import synthetic as syn
    impl = "ref_fast" if oracle.available("ref_fast") else "port"
    threads = os.cpu_count() or 1
    ac = np.bincount(batch.atomic_numbers, minlength=4)
    up = syn.upstream_grads(batch, ac, dtype=np.float32)
    cpu_fwd_grad(oracle, impl, batch.slice_mols(0, 64), syn.upstream_grads(
        batch.slice_mols(0, 64), np.bincount(batch.slice_mols(0, 64).atomic_numbers, minlength=4)), threads)
    reps, t0 = 0, time.perf_counter()
    while True:
        cpu_fwd_grad(oracle, impl, batch, up, threads)
        reps += 1
        el = time.perf_counter() - t0
        if el >= budget_s or reps >= 2000:
            break
    return {"value": batch.n_atoms * reps / el, "unit": UNIT, "cores": threads,
            "kind": "reference" if impl == "ref_fast" else "port",
            "sample": f"{reps} passes over one {batch.n_mols}-molecule batch ({batch.n_atoms} atoms), "
                      f"fwd+grad float32, {el:.1f} s",
            "impl": impl}


def run_reference_arm(args):
    """--impl reference: the reference's own CPU kernels, all host threads, same workload."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    import oracle
    from khan_b200.data import synthetic as syn
    impl = "ref_fast" if oracle.available("ref_fast") else "port"
    threads = os.cpu_count() or 1
    batch = syn.config1(seed=1, n_mols=N_MOLS)
    # bound the sample so that warmup + steps stay within ~150 s
    ac = np.bincount(batch.atomic_numbers, minlength=4)
    t0 = time.perf_counter()
    cpu_fwd_grad(oracle, impl, batch, syn.upstream_grads(batch, ac), threads)
    one = time.perf_counter() - t0
    total_steps = args.steps + args.warmup
    n_mols = N_MOLS
    while n_mols > 32 and one * (n_mols / N_MOLS) * total_steps > 150.0:
        n_mols //= 2
    sample = batch.slice_mols(0, n_mols)
    up = syn.upstream_grads(sample, np.bincount(sample.atomic_numbers, minlength=4))
    for _ in range(args.warmup):
        cpu_fwd_grad(oracle, impl, sample, up, threads)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        cpu_fwd_grad(oracle, impl, sample, up, threads)
    el = time.perf_counter() - t0
    value = sample.n_atoms * args.steps / el
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": el / args.steps * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32",
        "data": "synthetic", "gpu_launches": 0,
        "config": {"workload": "config1: 1024 GDB8-like molecules per step per GPU, float32, "
                               "ani_sort + featurize + featurize_grad",
                   "molecules_per_step": sample.n_mols, "atoms_per_step": sample.n_atoms,
                   "host_threads": threads},
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": threads,
                         "kind": "reference" if impl == "ref_fast" else "port",
                         "sample": f"each step = first {sample.n_mols} molecules of the config-1 batch "
                                   f"({sample.n_atoms} atoms), sort+fwd+grad"},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------------------------
# training step (benchmark configuration 3), reported separately from the benchmark metric
# ------------------------------------------------------------------------------------------
def run_forces_workload(args):
    """One step = config-1 batch -> ani_sort -> featurize -> four atomic networks -> molecule
    energies -> network backward to the features -> featurize_grad: energies and forces as
    `predict` + `coordinate_gradients` deliver them, C-ABI calls on pre-allocated buffers; the
    independent batches run side by side on a few streams, one CUDA graph per pass over the pool."""
    import torch
    import torch.distributed as dist

    from khan_b200.data import synthetic as syn
    from khan_b200.inference import EnergyForces
    from khan_b200.model import activations
    from khan_b200.model.nn import MoleculeNN
    from khan_b200.staged import HostBatch, StagedBatch

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    model = MoleculeNN(activation_fn=activations.gaussian, device=dev, seed=1, init="he")
    nb = max(1, min(16, args.steps))
    batches = syn.batch_pool(nb, n_mols=args.mols, seed=1 + 100 * rank)
    cap = max(b.n_atoms for b in batches)
    staged = []
    for b in batches:
        sb = StagedBatch(cap, args.mols, device=dev)
        sb.upload(HostBatch(b, None, pin=False), non_blocking=False, with_upstream=False)
        staged.append(sb)
    # Batches are independent and the weights fixed: a few evaluators (each with its own
    # activation buffers) take the batches round-robin on their own streams, so that the featurizer
    # kernels of one batch run beside the network kernels of another; the weights are packed once
    # per pass over the pool.  The whole pass is one CUDA graph.
    n_ev = max(1, min(args.streams, 4, nb))
    evs = [EnergyForces(model, cap, args.mols, device=dev) for _ in range(n_ev)]
    side = [torch.cuda.Stream(device=dev) for _ in range(n_ev)]
    with torch.cuda.stream(side[0]):
        for k in range(max(3, args.warmup)):
            evs[k % n_ev].run(staged[k % nb])
    torch.cuda.synchronize()

    def issue(batches_to_run):
        cap_stream = torch.cuda.current_stream()
        model.pack_weights(ctypes.c_void_p(cap_stream.cuda_stream))
        for st in side:
            st.wait_stream(cap_stream)
        for b, sb in enumerate(batches_to_run):
            with torch.cuda.stream(side[b % n_ev]):
                evs[b % n_ev].run(sb, pack=False)
        for st in side:
            cap_stream.wait_stream(st)

    def graph_of(batches_to_run):
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            issue(batches_to_run)
        return g

    if args.no_graph:
        whole = tail = None
    else:
        whole = graph_of(staged)
        tail = graph_of(staged[:args.steps % nb]) if args.steps % nb else None

    def run_steps(n_steps):
        done = 0
        while n_steps - done >= nb:
            whole.replay() if whole is not None else issue(staged)
            done += nb
        if n_steps - done:
            tail.replay() if tail is not None else issue(staged[:n_steps - done])

    work = torch.cuda.Stream(device=dev)
    with torch.cuda.stream(work):
        run_steps(nb)
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        run_steps(args.steps)
        e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1)
    atoms = float(sum(batches[k % nb].n_atoms for k in range(args.steps)))
    if world > 1:
        t = torch.tensor([ms, atoms], dtype=torch.float64, device=dev)
        tmax = t.clone()
        dist.all_reduce(tmax, op=dist.ReduceOp.MAX)
        dist.all_reduce(t, op=dist.ReduceOp.SUM)
        ms, atoms = float(tmax[0]), float(t[1])
    if rank == 0:
        print(json.dumps({
            "metric": "energies + forces atoms/sec (fp32, 1024-mol batch per GPU)", "value": atoms / (ms * 1e-3),
            "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": max(3, args.warmup),
            "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "f32 (tf32x3 tensor-core products in the atomic networks)", "data": "synthetic",
            "gpu_launches": args.steps * (EnergyForces.KERNELS_PER_PASS - 1) + -(-args.steps // nb),
            "config": {"workload": "config1 batches: sort + featurize + 4 x MLP 384-128-128-64-1 (gaussian) forward + "
                                   "molecule sums + MLP backward to the features + featurize_grad",
                       "molecules_per_step_per_gpu": args.mols,
                       "launch": ("eager" if args.no_graph else "one cuda_graph per pass over the resident batches"),
                       "streams": n_ev, "resident_batches": nb}}), flush=True)
    if world > 1:
        dist.destroy_process_group()


def measure_fused_train(ctx, mols: int, steps: int, warmup: int, train_path: str = "fused", graphs: bool = True,
                        exposed: bool = True):
    """The training step of benchmark configuration 3 on the C ABI only
    (khan_b200.training.fused_step): no autograd, the gradient all-reduce (NCCL, one flat buffer)
    issued right after the weight gradients.  Returns a dict; with several ranks and ``exposed`` the
    same steps are timed once more without the all-reduce, and the difference per step is the part
    of the collective that nothing hides."""
    import torch

    from khan_b200.data import synthetic as syn
    from khan_b200.model import activations
    from khan_b200.model.nn import MoleculeNN
    from khan_b200.staged import HostBatch, StagedBatch
    from khan_b200.training.fused_step import FusedTrainStep, StepPipeline
    from khan_b200.training.optim import FlatNadam
    from khan_b200.training.trainer_multi_tower import average_gradients

    rank, world, dev = ctx.rank, ctx.world, ctx.dev
    model = MoleculeNN(activation_fn=activations.gaussian, device=dev, seed=1, init="he")
    params = model.get_parameters()
    opt = FlatNadam(params, lr=1e-3, clip_norm=5.0)
    nb = max(1, min(8, steps))
    batches = syn.batch_pool(nb, n_mols=mols, seed=1 + 100 * rank)
    cap = max(b.n_atoms for b in batches)
    staged, labels = [], []
    for k, b in enumerate(batches):
        sb = StagedBatch(cap, mols, device=dev)
        sb.upload(HostBatch(b, None, pin=False), non_blocking=False, with_upstream=False)
        staged.append(sb)
        rng = np.random.default_rng(3000 + 100 * rank + k)
        labels.append(torch.from_numpy(rng.normal(size=b.n_mols).astype(np.float32)).to(dev))
    step = FusedTrainStep(model, opt, cap, mols, device=dev)
    side = torch.cuda.Stream(device=dev)
    with torch.cuda.stream(side):
        for k in range(max(3, warmup)):
            step.step(staged[k % nb], labels[k % nb])
    torch.cuda.synchronize()
    pipelined = train_path == "fused" and nb >= 2
    main = torch.cuda.current_stream()

    def timed(run_one, prime=None):
        if prime is not None:
            prime()
        for k in range(nb):
            run_one(k)
        ctx.barrier()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for k in range(steps):
            run_one(k)
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1)

    ms_local = ms_nccl = peer = peer_err = None
    if pipelined:
        # next batch's sort + featurize and this batch's coordinate gradient beside the network kernels
        if world > 1 and opt.flat_grads.numel() % 4 == 0:
            # the mean over the ranks as one kernel of the library over peer memory, inside the step's graph;
            # checked once against the library all-reduce on a buffer of random numbers
            import torch.distributed as dist
            from khan_b200.training.peer_allreduce import try_peer_allreduce
            peer = try_peer_allreduce(opt.flat_grads.numel(), dev)
            if peer is not None:
                gen = torch.Generator(device=dev)
                gen.manual_seed(77 + rank)
                probe = torch.randn(opt.flat_grads.numel(), device=dev, generator=gen)
                want = probe.clone()
                dist.all_reduce(want, op=dist.ReduceOp.SUM)
                want /= world
                ctx.barrier()
                torch.cuda.synchronize()
                peer_err = float((peer.mean_(probe) - want).abs().max())
                torch.cuda.synchronize()
        pipe = StepPipeline(step, staged, labels, allreduce=world > 1, graphs=graphs, peer=peer)
        ms = timed(pipe.run, pipe.prime)
        if world > 1 and exposed:
            solo = StepPipeline(step, staged, labels, allreduce=False, graphs=graphs)
            ms_local = timed(solo.run, solo.prime)
            if peer is not None:       # the same steps with the library all-reduce between two graphs, for comparison
                lib_pipe = StepPipeline(step, staged, labels, allreduce=True, graphs=graphs)
                ms_nccl = timed(lib_pipe.run, lib_pipe.prime)
    else:
        class _Eager:      # graphs off: the same calls issued directly (what ncu sees kernel by kernel)
            def __init__(self, fn):
                self.replay = fn

        fb_graphs, cg_graphs = [], []
        for sb, y in zip(staged, labels):
            if not graphs:
                fb_graphs.append(_Eager(lambda sb=sb, y=y: step.forward_backward(sb, y)))
                cg_graphs.append(_Eager(lambda sb=sb: step.coordinate_gradient(sb)))
                continue
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                step.forward_backward(sb, y)
            fb_graphs.append(g)
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                step.coordinate_gradient(sb)
            cg_graphs.append(g)
        if not graphs:
            up_graph = _Eager(opt.step)
        else:
            up_graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(up_graph):
                opt.step()

        def serial_step(k, allreduce=True):
            fb_graphs[k % nb].replay()
            if world > 1 and allreduce:      # coordinate gradients on the second stream, under the all-reduce
                side.wait_stream(main)
                with torch.cuda.stream(side):
                    cg_graphs[k % nb].replay()
                average_gradients(params, opt.flat_grads)
                main.wait_stream(side)
            else:
                cg_graphs[k % nb].replay()
            up_graph.replay()

        ms = timed(serial_step)
        if world > 1 and exposed:
            ms_local = timed(lambda k: serial_step(k, allreduce=False))
    atoms = float(sum(batches[k % nb].n_atoms for k in range(steps)))
    loss = float(step.l2s[:batches[(steps - 1) % nb].n_mols].mean())
    ms, atoms = ctx.max_sum(ms, atoms)
    out = {"ms_per_step": ms / steps, "atoms_per_s": atoms / (ms * 1e-3), "steps": steps, "n_gpus": world,
           "final_loss": loss, "gpu_launches_per_step": FusedTrainStep.KERNELS + (1 if peer is not None else 0),
           "resident_batches": nb,
           "pipelined": pipelined,
           "collective": ("none (one rank)" if world == 1 else
                          ("mean of the flat gradient buffer (%d float32 values) by one kernel of the library over peer "
                           "memory (CUDA IPC, plain NVLink loads), inside the step's CUDA graph"
                           if peer is not None else
                           "NCCL all-reduce (mean) of the flat gradient buffer, %d float32 values, between two graphs")
                          % opt.flat_grads.numel())}
    if ms_local is not None:
        ms_local, _ = ctx.max_sum(ms_local, 0.0)
        out["ms_per_step_without_allreduce"] = ms_local / steps
        out["exposed_allreduce_us"] = max(0.0, (ms - ms_local) / steps * 1e3)
    if ms_nccl is not None:
        ms_nccl, _ = ctx.max_sum(ms_nccl, 0.0)
        out["ms_per_step_with_nccl_allreduce"] = ms_nccl / steps
    if peer is not None:
        from khan_b200 import ani_mod
        out["peer_mean_max_abs_err_vs_nccl"] = peer_err
        out["device_status_after"] = int(ani_mod.device_status())   # -8 if a bounded wait for another rank ran out
        ctx.barrier()
        torch.cuda.synchronize()
        peer.close()
    return out


def run_fused_train_workload(args):
    """--workload train: prints the training-step line of benchmark configuration 3."""
    ctx = Ctx()
    r = measure_fused_train(ctx, args.mols, args.steps, args.warmup, args.train_path, graphs=not args.no_graph)
    if ctx.rank == 0:
        print(json.dumps({
            "metric": "training step atoms/sec (fp32, 1024-mol batch per GPU)", "value": r["atoms_per_s"],
            "unit": UNIT, "n_gpus": ctx.world, "steps": args.steps, "warmup": max(3, args.warmup),
            "ms_per_step": r["ms_per_step"], "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "f32 (tf32x3 tensor-core products in the atomic networks)", "data": "synthetic",
            "final_loss": r["final_loss"], "gpu_launches": args.steps * r["gpu_launches_per_step"],
            "exposed_allreduce_us": r.get("exposed_allreduce_us"),
            "collective": r.get("collective"),
            "ms_per_step_without_allreduce": r.get("ms_per_step_without_allreduce"),
            "ms_per_step_with_nccl_allreduce": r.get("ms_per_step_with_nccl_allreduce"),
            "peer_mean_max_abs_err_vs_nccl": r.get("peer_mean_max_abs_err_vs_nccl"),
            "device_status_after": r.get("device_status_after"),
            "config": {"workload": "config3: sort + featurize + 4 x MLP 384-128-128-64-1 (gaussian, He init) + MSE "
                                   "+ backward into weights and coordinates + mean of the weight gradients over the ranks "
                                   "+ Nadam",
                       "molecules_per_step_per_gpu": args.mols, "path": "fused (C ABI only, no autograd)",
                       "resident_batches": r["resident_batches"],
                       "order": ("pipelined: sort + featurize of the next batch and the coordinate gradient of this "
                                 "one run beside the network kernels on two side streams" if r["pipelined"] else
                                 "serial: one kernel after another"),
                       "launch": ("eager" if args.no_graph else
                                  "one cuda_graph per step" if ctx.world == 1 or "peer memory" in (r.get("collective") or "")
                                  else "cuda_graph (all-reduce eager, between the weight gradients and the update)")}}),
              flush=True)
    ctx.close()


def run_frontend_workload(args):
    """--workload frontend: the khan API itself on one GPU -- predict, coordinate_gradients and one training
    epoch through feed_dataset -- over a data set of 32,768 GDB-like molecules held on the host."""
    import torch
    from khan_b200 import RawDataset, TrainerMultiTower
    from khan_b200.data import synthetic as syn
    ctx = Ctx()
    mols = []
    for s in range(16):
        mols += syn.gdb_like_batch(2048, seed=100 + s).molecules()
    ys = list(np.random.default_rng(0).normal(size=len(mols)))
    ds = RawDataset(mols, ys)
    n_atoms = sum(len(m) for m in mols)
    tr = TrainerMultiTower(None, [ctx.dev], layer_sizes=(128, 128, 64, 1), seed=1)
    calls = (("predict", lambda: tr.predict(ds, batch_size=2048)),
             ("coordinate_gradients", lambda: len(list(tr.coordinate_gradients(ds, batch_size=2048)))),
             ("train_epoch_exp_rmse_max_norm", lambda: sum(1 for _ in tr.feed_dataset(
                 ds, True, [tr.train_op], 1024, before_hooks=tr.max_norm_ops))),
             ("train_epoch_mse", lambda: sum(1 for _ in tr.feed_dataset(ds, True, [tr.train_op_mse], 1024))))
    out = {}
    for name, fn in calls:
        fn()
        torch.cuda.synchronize()
        best = None
        for _ in range(3):
            t0 = time.perf_counter()
            fn()
            torch.cuda.synchronize()
            dt = time.perf_counter() - t0
            best = dt if best is None else min(best, dt)
        out[name] = {"atoms_per_s": n_atoms / best, "molecules_per_s": len(mols) / best, "seconds": best}
    if ctx.rank == 0:
        print(json.dumps({"metric": "khan front end atoms/sec (one GPU, wall clock, host data set)", "unit": UNIT,
                          "n_gpus": 1, "data": "synthetic", "dtype": "f32",
                          "config": {"workload": "32,768 GDB-like molecules (%d atoms) in a RawDataset; predict and "
                                                 "coordinate_gradients at batch 2048, training epochs at batch 1024; "
                                                 "fastest of 3 calls after one warm-up call" % n_atoms},
                          "calls": out}), flush=True)
    ctx.close()


def run_train_workload(args):
    """One step = config-1 batch per GPU -> ani_sort -> featurize -> four atomic networks
    (384-128-128-64-1, gaussian, He-normal init seed 1) -> molecule energies -> MSE against
    N(0,1) targets -> backward through the networks and through the featurizer into the
    coordinates -> one NCCL all-reduce of the flat weight-gradient bucket -> Nadam step."""
    import torch
    import torch.distributed as dist

    from khan_b200 import ani_mod
    from khan_b200.data import synthetic as syn
    from khan_b200.model import activations
    from khan_b200.model.nn import MoleculeNN
    from khan_b200.training.trainer_multi_tower import average_gradients

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    model = MoleculeNN(activation_fn=activations.gaussian, device=dev, seed=1, init="he")
    params = model.get_parameters()
    from khan_b200.training.optim import FlatNadam
    opt = FlatNadam(params, lr=1e-3, clip_norm=5.0)    # flat buffers: clip + Nadam + moving average in one call
    model.accumulate_into_grad = True                  # weight gradients are added straight into those buffers
    nb = max(1, min(8, args.steps))
    staged = []
    for k, b in enumerate(syn.batch_pool(nb, n_mols=args.mols, seed=1 + 100 * rank)):
        rng = np.random.default_rng(3000 + 100 * rank + k)
        xyz = torch.from_numpy(np.stack(b.coords(np.float32))).to(dev)
        ids = torch.from_numpy(np.repeat(np.arange(b.n_mols), b.mol_atom_counts)).to(dev)
        staged.append(dict(
            xyz=xyz, a=torch.from_numpy(b.atomic_numbers).to(dev), mo=torch.from_numpy(b.mol_offsets).to(dev),
            mac=torch.from_numpy(b.mol_atom_counts).to(dev), ids=ids, n_mols=b.n_mols, n_atoms=b.n_atoms,
            acs=np.bincount(b.atomic_numbers, minlength=4).astype(np.int32),
            labels=torch.from_numpy(rng.normal(size=b.n_mols).astype(np.float32)).to(dev)))

    def forward_backward(sb):
        x, y, z = (sb["xyz"][k].clone().requires_grad_(True) for k in range(3))
        si, gi, _ = ani_mod.ani_sort(sb["a"])
        feat = ani_mod.featurize_sorted_autograd(x, y, z, sb["a"], sb["mo"], sb["mac"], si, sb["acs"])
        atom_e = model.atom_outputs(feat, sb["acs"], gi)
        pred = torch.zeros(sb["n_mols"], dtype=torch.float32, device=dev).index_add_(0, sb["ids"], atom_e)
        loss = ((pred - sb["labels"]) ** 2).mean()
        opt.zero_grad(set_to_none=False)
        loss.backward()                      # weight gradients and d loss / d coordinates
        return loss

    def update():
        opt.step()

    def step(sb):
        loss = forward_backward(sb)
        average_gradients(params, opt.flat_grads)   # one NCCL all-reduce of the gradient buffer (no-op on one GPU)
        update()
        return loss

    for k in range(max(3, args.warmup)):
        step(staged[k % nb])
    torch.cuda.synchronize()
    # Forward + backward of each staged batch and the optimiser update are captured into CUDA
    # graphs and replayed, so no Python runs between their launches.  The NCCL all-reduce stays
    # outside the graphs (issued eagerly between the two), which keeps every rank's collective
    # order independent of graph capture.
    fb_graphs, up_graph, launch_mode = None, None, "eager (torch autograd drives the step)"
    if not args.no_graph:
        try:
            fb_graphs, losses = [], []
            pool = None
            for sb in staged:
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g, pool=pool):
                    losses.append(forward_backward(sb))
                pool = g.pool()
                fb_graphs.append(g)
            up_graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(up_graph, pool=pool):
                update()
            launch_mode = "cuda_graph (forward+backward per staged batch, update; all-reduce eager)"
        except Exception as exc:
            print(f"[bench] training-step capture failed ({exc!r}); running eagerly", file=sys.stderr)
            fb_graphs = up_graph = None
            torch.cuda.synchronize()
    use_graphs = torch.tensor([1 if fb_graphs is not None else 0], device=dev)
    if world > 1:                            # every rank must take the same path
        dist.all_reduce(use_graphs, op=dist.ReduceOp.MIN)
    if int(use_graphs.item()) == 0:
        fb_graphs = up_graph = None
        launch_mode = "eager (torch autograd drives the step)"
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for k in range(args.steps):
        if fb_graphs is not None:
            fb_graphs[k % nb].replay()
            average_gradients(params, opt.flat_grads)
            up_graph.replay()
            loss = losses[k % nb]
        else:
            loss = step(staged[k % nb])
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1)
    atoms = sum(staged[k % nb]["n_atoms"] for k in range(args.steps))
    if world > 1:
        t = torch.tensor([ms, float(atoms)], dtype=torch.float64, device=dev)
        tmax = t.clone()
        dist.all_reduce(tmax, op=dist.ReduceOp.MAX)
        dist.all_reduce(t, op=dist.ReduceOp.SUM)
        ms, atoms = float(tmax[0]), float(t[1])
    if rank == 0:
        print(json.dumps({
            "metric": "training step atoms/sec (fp32, 1024-mol batch per GPU)", "value": atoms / (ms * 1e-3),
            "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": max(3, args.warmup),
            "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "f32 (tf32x3 tensor-core products in the atomic networks)", "data": "synthetic",
            "final_loss": float(loss),
            "config": {"workload": "config3: sort + featurize + 4 x MLP 384-128-128-64-1 (gaussian, He init) + MSE "
                                   "+ backward into weights and coordinates + NCCL all-reduce + Nadam",
                       "molecules_per_step_per_gpu": args.mols, "launch": launch_mode},
        }), flush=True)
    if world > 1:
        dist.destroy_process_group()


# ------------------------------------------------------------------------------------------
# GPU arm
# ------------------------------------------------------------------------------------------
CASE_WORKLOAD = {
    "config1": "config1: 1024 GDB8-like molecules per step per GPU, float32, "
               "ani_sort + featurize + featurize_grad",
    "config2": "config2: the config1 batches in float64, ani_sort + featurize + featurize_grad",
    "config4": "config4: 256 molecules of 64-256 atoms per step per GPU, float32, "
               "ani_sort + featurize + featurize_grad",
}


CASE_FLOP_PEAK_NOTE = "min(FMA probe kernel measured in this run, 148 SM x 128 lanes x 2 x 1.965 GHz; half of that for float64)"


def capture_overlapped(staged, side, fn_name="run_step"):
    """One CUDA graph that runs ``fn_name`` of the given staged batches on the side streams, round-robin
    (fork from the capture stream, one branch per stream, join)."""
    import torch
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        cap = torch.cuda.current_stream()
        for st in side:
            st.wait_stream(cap)
        for b, sb in enumerate(staged):
            st = side[b % len(side)]
            with torch.cuda.stream(st):
                getattr(sb, fn_name)(ctypes.c_void_p(st.cuda_stream))
        for st in side:
            cap.wait_stream(st)
    return g


def time_kernel_overlapped(staged, side, fn_name, reps):
    """Average time (s) per launch of one kernel kind when its launches over all staged batches are spread over
    the side streams exactly as the steps of the timed region are: the kernel's share of a step there, where
    the tail of one launch runs beside the start of the next (time_kernel_alone has them one after another)."""
    import torch
    g = capture_overlapped(staged, side, fn_name)
    g.replay()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(reps):
        g.replay()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) * 1e-3 / (reps * len(staged))


def time_kernel_alone(staged, fn_name, reps):
    """Average duration (s) of one launch of a kernel kind: a graph of that kernel over all staged batches,
    one after another on one stream, replayed ``reps`` times."""
    import torch

    def stream_ptr():
        return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)

    g = torch.cuda.CUDAGraph()
    try:
        with torch.cuda.graph(g):
            for sb in staged:
                getattr(sb, fn_name)(stream_ptr())
        run = g.replay
    except Exception:
        torch.cuda.synchronize()

        def run():
            for sb in staged:
                getattr(sb, fn_name)(stream_ptr())
    run()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(reps):
        run()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) * 1e-3 / (reps * len(staged))


def work_per_atom(batch, esize):
    """Algorithmic bytes and flops per atom of each kernel for batches like ``batch``."""
    from khan_b200.data import synthetic as syn
    pairs, triplets = syn.count_work(batch)
    p, t = pairs / batch.n_atoms, triplets / batch.n_atoms
    coord = 3 * esize + 4
    nbytes = {"ani_sort": 4 + 8, "featurize": coord + esize * FEATURE_SIZE,
              "featurize_grad": coord + esize * FEATURE_SIZE + 3 * esize}
    flops = {"ani_sort": 0.0, "featurize": FLOPS_FWD[0] * p + FLOPS_FWD[1] * t,
             "featurize_grad": FLOPS_GRAD[0] * p + FLOPS_GRAD[1] * t}
    return nbytes, flops, p, t


def measure_case(ctx, case, n_batches=8, passes=7, n_streams=4):
    """Another benchmark configuration, device-resident: config2 (the config-1 batches in float64) or
    config4 (256 molecules of 64-256 atoms, float32).  One graph = one pass over the pool on a few
    streams; the median of ``passes`` replays is reported, with each kernel timed alone."""
    import torch
    from khan_b200.data import synthetic as syn
    from khan_b200.staged import HostBatch, StagedBatch
    dev, rank = ctx.dev, ctx.rank
    f64 = case == "config2"
    tdtype, esize = (torch.float64, 8) if f64 else (torch.float32, 4)
    if case == "config4":
        mols = 256
        batches = [syn.config4(seed=4 + 10 * k + 1000 * rank, n_mols=mols) for k in range(n_batches)]
    else:
        mols = N_MOLS
        batches = syn.batch_pool(n_batches, n_mols=mols, seed=1 + 100 * rank)
    cap = max(b.n_atoms for b in batches)
    staged = []
    for k, b in enumerate(batches):
        ac = np.bincount(b.atomic_numbers, minlength=4)
        sb = StagedBatch(cap, mols, dtype=tdtype, device=dev)
        sb.upload(HostBatch(b, syn.upstream_grads(b, ac, seed=12 + k), dtype=tdtype, pin=False), non_blocking=False)
        staged.append(sb)
    torch.cuda.synchronize()
    side = [torch.cuda.Stream(device=dev) for _ in range(n_streams)]
    for sb in staged:
        sb.run_step()
    torch.cuda.synchronize()
    g = capture_overlapped(staged, side)
    g.replay()
    torch.cuda.synchronize()
    times = []
    for _ in range(passes):
        ctx.barrier()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        g.replay()
        e1.record()
        torch.cuda.synchronize()
        times.append(e0.elapsed_time(e1))
    atoms = float(sum(b.n_atoms for b in batches))
    ms, atoms = ctx.max_sum(statistics.median(times), atoms)
    kernel_s = {k: time_kernel_alone(staged, fn, 5) for k, fn in
                (("ani_sort", "run_sort"), ("featurize", "run_featurize"), ("featurize_grad", "run_featurize_grad"))}
    nbytes, flops, p, t = work_per_atom(batches[0], esize)
    mean_atoms = sum(b.n_atoms for b in batches) / n_batches
    dominant = max(kernel_s, key=kernel_s.get)
    peak = min(measure_fma_peak(64 if f64 else 32, dev), FP32_PEAK_TFLOPS / (2 if f64 else 1))
    per_gpu = atoms / (ms * 1e-3) / ctx.world
    return {"workload": CASE_WORKLOAD[case], "atoms_per_s": atoms / (ms * 1e-3), "us_per_step": ms * 1e3 / n_batches,
            "atoms_per_step": mean_atoms, "streams": n_streams, "resident_batches": n_batches,
            "kernels_us": {k: v * 1e6 for k, v in kernel_s.items()}, "dominant_kernel": dominant,
            "dominant_frac_of_arith_peak": flops[dominant] * mean_atoms / kernel_s[dominant] / 1e12 / peak,
            "whole_step_frac_of_arith_peak": (flops["featurize"] + flops["featurize_grad"]) * per_gpu / 1e12 / peak,
            "arith_peak_tflops": peak, "arith_peak": ("FP64" if f64 else "FP32") + ": " + CASE_FLOP_PEAK_NOTE,
            "pairs_per_atom": p, "triplets_per_atom": t}


def measure_sharded(ctx, steps=64):
    """Benchmark configuration 1 as ONE 1024-molecule batch cut into contiguous molecule ranges over the
    ranks (khan_b200.data.sharding): every rank sorts, featurizes and differentiates its own shard on its
    GPU, no collective on the data path.  The time of a step is the max over ranks.  Rank 0 also runs the
    whole batch alone and checks the reassembled feature rows (atom order) against it bit for bit."""
    import torch
    import torch.distributed as dist
    from khan_b200.data import sharding, synthetic as syn
    from khan_b200.staged import HostBatch, StagedBatch
    dev, rank, world = ctx.dev, ctx.rank, ctx.world
    batch = syn.config1(seed=1, n_mols=N_MOLS)
    bounds = sharding.shard_bounds(batch.mol_atom_counts, world)
    shard = sharding.shard_batch(batch, rank, world)

    def stage(b):
        ac = np.bincount(b.atomic_numbers, minlength=4)
        sb = StagedBatch(max(1, b.n_atoms), max(1, b.n_mols), device=dev)
        sb.upload(HostBatch(b, syn.upstream_grads(b, ac, seed=12), pin=False), non_blocking=False)
        return sb

    sb = stage(shard)
    for _ in range(3):
        sb.run_step()
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        for _ in range(steps):
            sb.run_step()
    g.replay()
    times = []
    for _ in range(5):
        ctx.barrier()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        g.replay()
        e1.record()
        torch.cuda.synchronize()
        times.append(e0.elapsed_time(e1))
    ms, atoms = ctx.max_sum(statistics.median(times), float(shard.n_atoms) * steps)

    # reassemble the shards' feature rows in atom order on rank 0
    atoms_of = [int(batch.mol_atom_counts[a:b].sum()) for a, b in bounds]
    pad = max(atoms_of)
    mine = torch.zeros((pad, FEATURE_SIZE), dtype=torch.float32, device=dev)
    mine[:shard.n_atoms] = sb.features[:shard.n_atoms][sb.gather[:shard.n_atoms].long()]
    parts = [torch.empty_like(mine) for _ in range(world)]
    dist.all_gather(parts, mine)
    out = {"ms_per_step": ms / steps, "atoms_per_s": atoms / (ms * 1e-3), "n_gpus": world, "steps": steps,
           "atoms_per_shard": atoms_of,
           "note": "one 1024-molecule batch (13.7 k atoms) cut by molecule ranges; every step repeats the same shard, "
                   "which stays in L2; no data-path collective"}
    if rank == 0:
        whole = stage(batch)
        whole.run_step()
        torch.cuda.synchronize()
        ref = whole.features[:batch.n_atoms][whole.gather[:batch.n_atoms].long()]
        got = torch.cat([p[:n] for p, n in zip(parts, atoms_of)])
        out["features_equal_single_gpu_bit_for_bit"] = bool(torch.equal(got, ref))
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=4096)
    ap.add_argument("--warmup", type=int, default=64)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--batches", type=int, default=64, help="distinct batches resident in HBM")
    ap.add_argument("--no-graph", action="store_true", help="launch eagerly instead of CUDA graphs")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--e2e-steps", type=int, default=0, help="0 = min(steps, 256)")
    ap.add_argument("--streams", type=int, default=8,
                    help="independent batches in flight: steps are issued round-robin over this many streams")
    ap.add_argument("--mols", type=int, default=N_MOLS,
                    help="molecules per batch (1024 is the benchmark workload; other sizes are for profiling)")
    ap.add_argument("--workload", default="aev", choices=["aev", "train", "forces", "frontend"],
                    help="aev: the benchmark metric (sort + featurize + featurize_grad); train: the full "
                         "data-parallel training step of benchmark configuration 3; forces: energies + forces of "
                         "config-1 batches through the C ABI only (both reported separately)")
    ap.add_argument("--train-path", default="fused", choices=["fused", "fused-serial", "autograd"],
                    help="train workload: fused = C-ABI calls only (FusedTrainStep) with the next batch's featurize "
                         "and the coordinate gradient beside the network kernels (StepPipeline); fused-serial = the "
                         "same kernels one after another; autograd = torch autograd drives the same kernels (what "
                         "TrainerMultiTower does)")
    ap.add_argument("--e2e-slots", type=int, default=4,
                    help="batches in flight (one stream each) in the end-to-end measurement")
    ap.add_argument("--case", default="config1", choices=["config1", "config2", "config4"],
                    help="config1 is the benchmark workload; config2 (same batches in float64) and config4 "
                         "(256 molecules of 64-256 atoms, float32) are extra measurements")
    ap.add_argument("--profile", action="store_true",
                    help="only W warm-up and K timed steps, launched eagerly on one stream (for ncu)")
    ap.add_argument("--no-extras", action="store_true",
                    help="skip the extra keys of the line (config3 training step, sharded config 1, config2 / config4, "
                         "energies + forces end to end)")
    ap.add_argument("--repeats", type=int, default=5, help="timed regions of exactly K steps each; the median is reported")
    args = ap.parse_args()
    if args.warmup < 3:
        args.warmup = 3

    if args.impl == "reference":
        run_reference_arm(args)
        return
    if args.workload == "train":
        if args.train_path in ("fused", "fused-serial"):
            run_fused_train_workload(args)
        else:
            run_train_workload(args)
        return
    if args.workload == "forces":
        run_forces_workload(args)
        return
    if args.workload == "frontend":
        run_frontend_workload(args)
        return

    import torch
    import torch.distributed as dist

    from khan_b200 import _lib
    from khan_b200.data import synthetic as syn
    from khan_b200.staged import HostBatch, StagedBatch

    ctx = Ctx()
    rank, world, local_rank, dev = ctx.rank, ctx.world, ctx.local_rank, ctx.dev
    _lib.lib()  # fail loudly if the CUDA library is missing

    sampler = ClockSampler(local_rank)
    sampler.start()

    # ---- workload: NB distinct 1024-molecule batches per rank (weak scaling) -------------
    nb = max(1, min(args.batches, args.steps))
    tdtype = torch.float64 if args.case == "config2" else torch.float32
    esize = 8 if args.case == "config2" else 4
    if args.case == "config4":
        nb = min(nb, 16)
        args.mols = 256 if args.mols == N_MOLS else args.mols
        batches = [syn.config4(seed=4 + 10 * k + 1000 * rank, n_mols=args.mols) for k in range(nb)]
    else:
        batches = syn.batch_pool(nb, n_mols=args.mols, seed=1 + 100 * rank)
    max_atoms = max(b.n_atoms for b in batches)
    host = []
    for k, b in enumerate(batches):
        ac = np.bincount(b.atomic_numbers, minlength=4)
        host.append(HostBatch(b, syn.upstream_grads(b, ac, seed=12 + k), dtype=tdtype, pin=(k < 16)))
    staged = []
    for hb in host:
        sb = StagedBatch(max_atoms, args.mols, dtype=tdtype, device=dev)
        sb.upload(hb, non_blocking=False)
        staged.append(sb)
    torch.cuda.synchronize()
    atoms_per_step = [sb.n_atoms for sb in staged]
    launches_per_step = staged[0].kernels_per_step()

    def stream_ptr():
        return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)

    # ---- warm-up: W steps, then keep going until ~1 s of device time has passed ----------
    t_load0 = time.perf_counter()
    for k in range(args.warmup):
        staged[k % nb].run_step(stream_ptr())
    torch.cuda.synchronize()

    if args.profile:
        for k in range(args.steps):
            staged[k % nb].run_step(stream_ptr())
        torch.cuda.synchronize()
        sampler.stop()
        print(json.dumps({"profile_run": True, "steps": args.steps, "warmup": args.warmup}))
        return

    # Steps of different batches are independent, so they are issued round-robin over a few
    # streams: the tail of one batch's kernels overlaps the head of the next batch's.  All
    # NB steps are captured into ONE graph (fork from the capture stream, one branch per
    # stream, join), plus one single-step graph per batch for the remainder K mod NB.
    n_streams = max(1, min(args.streams, nb))
    side = [torch.cuda.Stream(device=dev) for _ in range(n_streams)]
    graphs = mega = tail = None
    launch_mode = "eager"
    if not args.no_graph:
        try:
            graphs = []
            for sb in staged:
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g):
                    sb.run_step(stream_ptr())
                graphs.append(g)
            mega = capture_overlapped(staged, side)
            # the K steps of the timed region are whole passes over the pool plus this remainder
            tail = capture_overlapped(staged[:args.steps % nb], side) if args.steps % nb else None
            launch_mode = "cuda_graph"
        except Exception as exc:
            print(f"[bench] CUDA graph capture failed ({exc!r}); launching eagerly", file=sys.stderr)
            graphs = mega = tail = None
            torch.cuda.synchronize()

    def run_steps(n_steps):
        """Issues exactly n_steps steps (batches 0, 1, 2, ... cyclically)."""
        done = 0
        if mega is not None:
            while n_steps - done >= nb:
                mega.replay()
                done += nb
            rest = n_steps - done
            if rest and tail is not None and rest == args.steps % nb:
                tail.replay()
            else:
                for k in range(rest):
                    graphs[k].replay()
        else:
            main = torch.cuda.current_stream()
            for st in side:
                st.wait_stream(main)
            for k in range(n_steps):
                st = side[k % n_streams]
                staged[k % nb].run_step(ctypes.c_void_p(st.cuda_stream))
            for st in side:
                main.wait_stream(st)

    while time.perf_counter() - t_load0 < 1.0:
        run_steps(nb)
        torch.cuda.synchronize()

    # ---- timed regions: exactly K steps each, between a barrier + synchronize on both sides; the
    # median region gives the headline and every region is listed (at the driver's K the region is
    # a single graph replay of under a millisecond, so one region alone is at the mercy of jitter) ----
    my_atoms = sum(atoms_per_step[k % nb] for k in range(args.steps))
    region_ms = []
    t_timed0 = time.perf_counter()
    for _ in range(max(1, args.repeats)):
        ctx.barrier()
        torch.cuda.synchronize()
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        ev0.record()
        run_steps(args.steps)
        ev1.record()
        torch.cuda.synchronize()
        ctx.barrier()
        ms, total_atoms = ctx.max_sum(ev0.elapsed_time(ev1), float(my_atoms))
        region_ms.append(ms)
    t_timed1 = time.perf_counter()
    elapsed_ms = statistics.median(region_ms)
    value = total_atoms / (elapsed_ms * 1e-3)

    # ---- spread: passes over the resident pool timed one by one (not part of the headline) ----
    pass_ms = []
    if mega is not None:
        evs = [torch.cuda.Event(enable_timing=True) for _ in range(min(32, max(2, args.steps // nb)) + 1)]
        evs[0].record()
        for ev in evs[1:]:
            mega.replay()
            ev.record()
        torch.cuda.synchronize()
        pass_ms = sorted(a.elapsed_time(b) / nb for a, b in zip(evs[:-1], evs[1:]))

    # ---- per-kernel durations (graphs of one kernel kind over all batches) ------------------
    reps = max(3, min(50, args.steps // nb))
    kernel_s = {"ani_sort": time_kernel_alone(staged, "run_sort", reps),
                "featurize": time_kernel_alone(staged, "run_featurize", reps),
                "featurize_grad": time_kernel_alone(staged, "run_featurize_grad", reps)}
    kernel_overlapped_s = None
    if mega is not None:
        kernel_overlapped_s = {k: time_kernel_overlapped(staged, side, fn, reps) for k, fn in
                               (("ani_sort", "run_sort"), ("featurize", "run_featurize"),
                                ("featurize_grad", "run_featurize_grad"))}
    t_load1 = time.perf_counter()

    # ---- end to end through the C ABI with host buffers ---------------------------------------
    e2e_steps = args.e2e_steps or min(args.steps, 256)
    n_slots = max(1, args.e2e_slots)
    n_host = min(len(host), 16)
    slots = [StagedBatch(max_atoms, args.mols, dtype=tdtype, device=dev) for _ in range(n_slots)]
    streams = [torch.cuda.Stream(device=dev) for _ in range(n_slots)]
    out_feat = [torch.empty((max_atoms, FEATURE_SIZE), dtype=tdtype).pin_memory() for _ in range(n_slots)]
    out_grad = [torch.empty((3, max_atoms), dtype=tdtype).pin_memory() for _ in range(n_slots)]

    def e2e_pass(n_steps):
        h2d = d2h = atoms = 0
        for k in range(n_steps):
            s = k % n_slots
            hb = host[k % n_host]
            with torch.cuda.stream(streams[s]):
                h2d += slots[s].upload(hb, non_blocking=True)
                slots[s].run_step(ctypes.c_void_p(streams[s].cuda_stream))
                d2h += slots[s].download(out_feat[s], out_grad[s], non_blocking=True)
                atoms += slots[s].n_atoms
        return h2d, d2h, atoms

    def copy_pass(n_steps, up_too=True, down_too=True):
        """The transfers of e2e_pass with no kernel between them (both directions, or one alone), one queue
        per direction and nothing that orders one against the other: what the host link allows."""
        h2d = d2h = 0
        up, down = streams[0], streams[-1]
        for k in range(n_steps):
            s = k % n_slots
            if up_too:
                with torch.cuda.stream(up):
                    h2d += slots[s].upload(host[k % n_host], non_blocking=True)
            if down_too:
                with torch.cuda.stream(down):
                    d2h += slots[s].download(out_feat[s], out_grad[s], non_blocking=True)
        return h2d, d2h

    main_stream = torch.cuda.current_stream()

    def timed_host_passes(fn, n_passes=3):
        """ms of each of n_passes calls of fn (max over ranks), with the streams fenced on both sides."""
        out, last = [], None
        for _ in range(n_passes):
            ctx.barrier()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(main_stream)
            for st in streams:
                st.wait_event(e0)
            last = fn()
            for st in streams:
                main_stream.wait_stream(st)
            e1.record(main_stream)
            torch.cuda.synchronize()
            out.append(ctx.max_sum(e0.elapsed_time(e1), 0.0)[0])
        return out, last

    e2e_pass(6)
    torch.cuda.synchronize()
    # Three timed passes of e2e_steps steps each; the median is the reported value, the best is listed
    # beside it.  The transfers share the host's PCIe root and memory with whatever else runs on the
    # machine (all ranks of a multi-GPU run included).
    e2e_runs, (h2d, d2h, e2e_atoms) = timed_host_passes(lambda: e2e_pass(e2e_steps))
    e2e_ms = statistics.median(e2e_runs)
    _, e2e_total = ctx.max_sum(0.0, float(e2e_atoms))
    copy_runs, (c_h2d, c_d2h) = timed_host_passes(lambda: copy_pass(e2e_steps))
    copy_ms = statistics.median(copy_runs)
    up_ms = statistics.median(timed_host_passes(lambda: copy_pass(e2e_steps, down_too=False))[0])
    down_ms = statistics.median(timed_host_passes(lambda: copy_pass(e2e_steps, up_too=False))[0])
    e2e_extra = {"copy_only": {"atoms_per_s": e2e_total / (copy_ms * 1e-3),
                               "gbs_per_rank": (c_h2d + c_d2h) / (copy_ms * 1e-3) / 1e9,
                               "h2d_alone_gbs_per_rank": c_h2d / (up_ms * 1e-3) / 1e9,
                               "d2h_alone_gbs_per_rank": c_d2h / (down_ms * 1e-3) / 1e9,
                               "ceiling_atoms_per_s": e2e_total / (max(up_ms, down_ms) * 1e-3),
                               "note": "the same host-to-device and device-to-host copies with no kernel launched, one "
                                       "stream per direction: both directions at once (atoms_per_s, gbs_per_rank), "
                                       "each direction alone, and the ceiling if the slower direction hid the other "
                                       "completely; times are the max over ranks"}}
    del slots, out_feat

    # ---- energies + forces end to end: coordinates in, molecule energies and forces out -----------
    e2e_forces = None
    if not args.no_extras and args.case == "config1":
        from khan_b200.inference import EnergyForces
        from khan_b200.model import activations
        from khan_b200.model.nn import MoleculeNN
        model = MoleculeNN(activation_fn=activations.gaussian, device=dev, seed=1, init="he")
        fslots = [StagedBatch(max_atoms, args.mols, device=dev) for _ in range(n_slots)]
        evs = [EnergyForces(model, max_atoms, args.mols, device=dev) for _ in range(n_slots)]
        out_e = [torch.empty(args.mols, dtype=torch.float32).pin_memory() for _ in range(n_slots)]
        model.pack_weights(ctypes.c_void_p(main_stream.cuda_stream))

        def forces_pass(n_steps):
            h2d = d2h = atoms = 0
            for k in range(n_steps):
                i = k % n_slots
                hb = host[k % n_host]
                with torch.cuda.stream(streams[i]):
                    h2d += fslots[i].upload(hb, non_blocking=True, with_upstream=False)
                    evs[i].run(fslots[i], ctypes.c_void_p(streams[i].cuda_stream), pack=False)
                    n, m = fslots[i].n_atoms, fslots[i].n_mols
                    out_e[i][:m].copy_(evs[i].mol_energy[:m], non_blocking=True)
                    for r in range(3):
                        out_grad[i][r, :n].copy_(fslots[i].grads[r, :n], non_blocking=True)
                    d2h += 4 * (m + 3 * n)
                    atoms += n
            return h2d, d2h, atoms

        forces_pass(6)
        torch.cuda.synchronize()
        f_runs, (f_h2d, f_d2h, f_atoms) = timed_host_passes(lambda: forces_pass(e2e_steps))
        f_ms = statistics.median(f_runs)
        _, f_total = ctx.max_sum(0.0, float(f_atoms))
        e2e_forces = {"value": f_total / (f_ms * 1e-3), "unit": UNIT, "h2d_bytes_per_step": f_h2d / e2e_steps,
                      "d2h_bytes_per_step": f_d2h / e2e_steps, "steps": e2e_steps, "pipeline_slots": n_slots,
                      "passes_atoms_per_s": [f_total / (ms * 1e-3) for ms in f_runs], "reported": "median of 3 passes",
                      "workload": "coordinates, element ids and molecule table in; molecule energies and dE/dx, dE/dy, "
                                  "dE/dz out (sort + featurize + 4 atomic networks forward and backward + featurize_grad, "
                                  "C-ABI calls only): the boundary predict / coordinate_gradients use"}
        del fslots, evs

    # ---- the other benchmark configurations, as extra keys of the same line -----------------------
    extras = {}
    if not args.no_extras and args.case == "config1" and args.mols == N_MOLS:
        del staged, mega, tail, graphs
        torch.cuda.empty_cache()
        extras["config3"] = measure_fused_train(ctx, N_MOLS, steps=max(64, min(args.steps, 512)), warmup=args.warmup)
        extras["config3"]["workload"] = ("config3: config-1 batch per GPU -> sort + featurize + 4 x MLP 384-128-128-64-1 "
                                         "(gaussian, He init) + MSE + backward into weights and coordinates + NCCL "
                                         "all-reduce of the weight gradients + Nadam")
        if world > 1:
            extras["config1_sharded"] = measure_sharded(ctx)
        extras["cases"] = {c: measure_case(ctx, c) for c in ("config2", "config4")}
    sampler.stop()

    if rank != 0:
        ctx.close()
        return

    # ---- roofline of the dominant kernel --------------------------------------------------------
    peaks, peak_kind = measured_peaks()
    mean_atoms = sum(atoms_per_step) / nb
    pairs, triplets = syn.count_work(batches[0])
    p_per_atom, t_per_atom = pairs / batches[0].n_atoms, triplets / batches[0].n_atoms
    coord = 3 * esize + 4
    bytes_per_atom = {"ani_sort": 4 + 8, "featurize": coord + esize * FEATURE_SIZE,
                      "featurize_grad": coord + esize * FEATURE_SIZE + 3 * esize}
    flops_per_atom = {"ani_sort": 0.0,
                      "featurize": FLOPS_FWD[0] * p_per_atom + FLOPS_FWD[1] * t_per_atom,
                      "featurize_grad": FLOPS_GRAD[0] * p_per_atom + FLOPS_GRAD[1] * t_per_atom}
    dominant = max(kernel_s, key=kernel_s.get)
    achieved_gbs = bytes_per_atom[dominant] * mean_atoms / kernel_s[dominant] / 1e9
    achieved_tf = flops_per_atom[dominant] * mean_atoms / kernel_s[dominant] / 1e12
    roofline = {"kernel": dominant, "bound": "hbm", "achieved": achieved_gbs, "peak": peaks["hbm_gbs"],
                "unit": "GB/s", "frac": achieved_gbs / peaks["hbm_gbs"],
                "traffic": (NCU_DRAM_BYTES_PER_ATOM[dominant] * mean_atoms
                            if args.case == "config1" and NCU_DRAM_BYTES_PER_ATOM.get(dominant) else None),
                "traffic_source": NCU_TRAFFIC_SOURCE if args.case == "config1" else None,
                "peak_source": peak_kind,
                "algorithmic_bytes_per_launch": bytes_per_atom[dominant] * mean_atoms}
    formula_peak = FP32_PEAK_TFLOPS / (2 if args.case == "config2" else 1)
    fma_measured = measure_fma_peak(64 if args.case == "config2" else 32, dev)
    arith_peak = min(fma_measured, formula_peak)
    roofline_fp32 = {"kernel": dominant, "achieved": achieved_tf, "peak": arith_peak,
                     "unit": "TFLOP/s", "frac": achieved_tf / arith_peak,
                     "peak_source": "min(FMA probe kernel measured in this run, 148 SM x 128 lanes x 2 x "
                                    "1.965 GHz; half of that for float64)",
                     "peak_measured": fma_measured, "peak_formula": formula_peak,
                     "pairs_per_atom": p_per_atom, "triplets_per_atom": t_per_atom}
    if kernel_overlapped_s:
        # the same kernel with its launches spread over the streams of the timed region (see time_kernel_overlapped)
        t_ov = kernel_overlapped_s[dominant]
        roofline_fp32["frac_on_the_step_streams"] = flops_per_atom[dominant] * mean_atoms / t_ov / 1e12 / arith_peak
        roofline["frac_on_the_step_streams"] = bytes_per_atom[dominant] * mean_atoms / t_ov / 1e9 / roofline["peak"]
    # the bound that binds is the one with the larger fraction: the arithmetic one for these kernels
    roofline["binding_bound"] = ("fp32/fp64 arithmetic (roofline_fp32)" if roofline_fp32["frac"] >= roofline["frac"]
                                 else "hbm")
    step_flops = (flops_per_atom["featurize"] + flops_per_atom["featurize_grad"])
    per_gpu = value / world
    whole_step = {"per_gpu_tflops": step_flops * per_gpu / 1e12,
                  "frac_fp32": step_flops * per_gpu / 1e12 / arith_peak,
                  "per_gpu_gbs": 3116 * per_gpu / 1e9, "frac_hbm": 3116 * per_gpu / 1e9 / peaks["hbm_gbs"]}

    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": elapsed_ms / args.steps, "higher_is_better": True,
        "timed_regions": {"ms_per_step": [ms / args.steps for ms in region_ms], "steps_each": args.steps,
                          "reported": "median region"},
        "ms_per_step_by_pass": ({"median": pass_ms[len(pass_ms) // 2], "best": pass_ms[0], "worst": pass_ms[-1],
                                 "passes": len(pass_ms), "steps_per_pass": nb} if pass_ms else None),
        "scaling": "weak", "vs_baseline": None, "dtype": "f64" if args.case == "config2" else "f32",
        "data": "synthetic",
        "config": {"workload": CASE_WORKLOAD[args.case],
                   "molecules_per_step": args.mols, "atoms_per_step": mean_atoms,
                   "resident_batches": nb, "l2": "inputs larger than L2 (distinct batches cycled)",
                   "launch": launch_mode, "streams": n_streams,
                   "parallelism": f"molecule shards x{world}, no collective"},
        "e2e": {"value": e2e_total / (e2e_ms * 1e-3), "unit": UNIT,
                "h2d_bytes_per_step": h2d / e2e_steps, "d2h_bytes_per_step": d2h / e2e_steps,
                "steps": e2e_steps, "pipeline_slots": n_slots,
                "passes_atoms_per_s": [e2e_total / (ms * 1e-3) for ms in e2e_runs],
                "best_atoms_per_s": e2e_total / (min(e2e_runs) * 1e-3), "reported": "median of 3 passes",
                **e2e_extra},
        "gpu_launches": args.steps * launches_per_step,
        "kernels": {k: {"avg_us": v * 1e6,
                        "avg_us_on_the_step_streams": (kernel_overlapped_s[k] * 1e6 if kernel_overlapped_s else None)}
                    for k, v in kernel_s.items()},
        "roofline": roofline, "roofline_fp32": roofline_fp32, "whole_step": whole_step,
        "host_binding": ctx.host_binding,
        "clocks": sampler.summary(t_load0, t_load1),
        "clocks_timed_region": sampler.summary(t_timed0, t_timed1),
    }
    if e2e_forces is not None:
        line["e2e_forces"] = e2e_forces
    line.update(extras)
    if world == 1 and not args.no_cpu_baseline and args.case == "config1":
        try:
            line["cpu_baseline"] = cpu_baseline(batches[0])
        except Exception as exc:
            line["cpu_baseline"] = {"value": None, "unit": UNIT, "cores": 0, "kind": "port",
                                    "sample": f"failed: {exc!r}"}
    print(json.dumps(line), flush=True)
    ctx.close()


if __name__ == "__main__":
    main()

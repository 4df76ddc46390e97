"""``TrainerMultiTower``: the training / inference front end of khan
(``khan/training/trainer_multi_tower.py`` of the reference) on top of the B200 kernels.

What is kept: the constructor signature, ``feed_dataset`` (a generator with one result per round
of towers), ``predict``, ``featurize``, ``coordinate_gradients``, ``eval_abs_rmse``,
``get_train_op_rmse`` / ``get_train_op_exp``, ``save_numpy`` / ``load_numpy`` with the reference's
variable names, ``initialize``, and the optimiser recipe (Nadam 1e-3, global-norm clip 5, max-norm
3 hook).  What differs by construction: there is no TensorFlow graph or session (``sess`` is
accepted and ignored), a "tower" is a CUDA device of this process, and when
``torch.distributed`` is initialised the weight gradients are averaged over all ranks with one
flat NCCL all-reduce instead of the reference's concat + reduce_mean on the CPU
(``trainer_multi_tower.py:137-179``).  ``train()`` keeps the reference's schedule: epochs at a
fixed batch size until the test error has not improved for ``max_local_epoch_count`` epochs, then
reload the best weights, halve the learning rate and add 128 to the batch size.
"""
from __future__ import annotations

import ctypes
import itertools
import os
import time

import numpy as np
import torch

from .. import _lib, ani_mod
from ..data.feeder import BatchFeeder, PackedDataset
from ..model import activations
from ..model.nn import MoleculeNN
from ..utils.helpers import ed_harder_rmse
from .optim import FlatNadam

HARTREE_TO_KCAL_PER_MOL = 627.509


def initialize_module(so_file=None):
    """The reference loads ``ani.so`` here (``trainer_multi_tower.py:123-127``); this build has
    one library, loaded on first use, so the call only returns the op module."""
    return ani_mod


def flatten_results(res, pos=0):
    flattened = []
    for l in res:
        flattened.append(l[pos])
    return np.concatenate(flattened).reshape((-1,))


def average_gradients(parameters, flat_grads=None, peer=None):
    """Mean of the weight gradients over all ranks: ONE all-reduce of a flat bucket (296,452
    values for four 384-128-128-64-1 networks), the data-parallel replacement of the reference's
    per-variable concat + reduce_mean on the CPU (``trainer_multi_tower.py:137-179``).  A no-op
    without an initialised process group.  ``flat_grads``: the buffer all ``.grad`` tensors are
    slices of (``FlatNadam.flat_grads``); it is reduced in place with no packing.  ``peer``: a
    ``PeerAllReduce`` -- the mean is then one kernel of this library over peer memory instead of the
    library collective (and may be captured in a CUDA graph)."""
    import torch.distributed as dist
    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size() == 1:
        return
    if peer is not None and flat_grads is not None:
        peer.mean_(flat_grads)
        return
    if flat_grads is not None:
        dist.all_reduce(flat_grads, op=dist.ReduceOp.SUM)
        flat_grads /= dist.get_world_size()
        return
    params = [p for p in parameters if p.grad is not None]
    if not params:
        return
    flat = torch.cat([p.grad.reshape(-1) for p in params])
    dist.all_reduce(flat, op=dist.ReduceOp.SUM)
    flat /= dist.get_world_size()
    off = 0
    for p in params:
        n = p.numel()
        p.grad.copy_(flat[off:off + n].view_as(p))
        off += n


def _split_rows(rows, offsets):
    """Per-molecule views of ``rows`` (first row of molecule m is ``offsets[m]``, the last molecule
    ends with the array) -- what ``np.split(rows, offsets[1:])`` returns, five times faster for
    thousands of short pieces."""
    starts = np.asarray(offsets).tolist()
    return [rows[a:b] for a, b in zip(starts, starts[1:] + [len(rows)])]


class _Op:
    """Stand-in for a graph tensor passed in ``target_ops``."""

    def __init__(self, name):
        self.name = name

    def __repr__(self):
        return f"<op {self.name}>"


def _device_of(tower):
    if isinstance(tower, torch.device):
        return tower
    s = str(tower)
    if s.startswith("/gpu:"):
        return torch.device("cuda", int(s.split(":")[1]))
    if s.startswith("/cpu"):
        raise ValueError("khan_b200 has no CPU tower")
    return torch.device(s)


class TrainerMultiTower:

    def __init__(self, sess, towers, precision=torch.float32, layer_sizes=(128, 128, 64, 8, 1),
                 activation_fn=activations.celu, fit_charges=False, seed=None, init="reference",
                 split_precision=True):
        assert fit_charges is False
        precision = {"float32": torch.float32, "float64": torch.float64}.get(str(precision), precision)
        assert precision in (torch.float32, torch.float64)
        assert len(towers) > 0
        self.sess = sess
        self.towers = [_device_of(t) for t in towers]
        if len(self.towers) > 1:
            # The reference builds one graph per tower inside one process (trainer_multi_tower.py:253-259,
            # 290-419).  Here the parameters, the optimiser state and the pre-packed weights live on ONE
            # device, and a kernel launched on another GPU with pointers to them would read memory that
            # device cannot reach.  Several GPUs are one process each (torchrun), the weight gradients
            # meeting in one NCCL all-reduce (average_gradients).
            raise NotImplementedError(
                "TrainerMultiTower takes one tower per process: start one process per GPU "
                "(python -m torch.distributed.run --nproc-per-node N ...) and give each its own device; "
                "the weight gradients are averaged over the ranks with one NCCL all-reduce")
        self.num_towers = len(self.towers)
        self.precision = precision
        self.feat_size = ani_mod.FEATURE_SIZE
        # the parameters live on the (only) tower
        self.model = MoleculeNN(layer_sizes=(self.feat_size,) + tuple(layer_sizes), precision=precision,
                                activation_fn=activation_fn, prefix="near_", device=self.towers[0],
                                seed=seed, init=init, split_precision=split_precision)
        self.all_models = [self.model]
        self.parameters = self.model.get_parameters()
        self.learning_rate = 1e-3
        self.ema_decay = 0.9999
        if precision == torch.float32 and self.towers[0].type == "cuda":
            # flat buffers + one fused clip / Nadam / moving-average call per step
            self.optimizer = FlatNadam(self.parameters, lr=self.learning_rate, clip_norm=5.0,
                                       ema_decay=self.ema_decay)
            self.ema = [self.optimizer.ema_of(k) for k in range(len(self.parameters))]
            self.model.accumulate_into_grad = True    # gradients only ever come from .backward() here
        else:
            self.optimizer = torch.optim.NAdam(self.parameters, lr=self.learning_rate, betas=(0.9, 0.999), eps=1e-8)
            self.ema = [p.detach().clone() for p in self.parameters]
        self.global_step = 0
        self.global_epoch_count = 0
        self.local_epoch_count = 0
        # ops that feed_dataset understands
        self.tower_preds = _Op("tower_preds")
        self.tower_bids = _Op("tower_bids")
        self.tower_l2s = _Op("tower_l2s")
        self.unordered_l2s = _Op("unordered_l2s")
        self.tower_mos = _Op("tower_mos")
        self.tower_coord_grads = _Op("tower_coord_grads")
        self.tower_features = _Op("tower_features")
        self.tower_exp_loss = _Op("tower_exp_loss")
        self.tower_force_rmses = _Op("tower_force_rmses")
        self.train_op = _Op("train_op")                # exp(rmse) of the energies
        self.train_op_rmse = _Op("train_op_rmse")
        self.train_op_mse = _Op("train_op_mse")
        self.train_op_forces = _Op("train_op_forces")  # exp(force rmse)
        self.max_norm_ops = _Op("max_norm_ops")
        self._device_l2s = _Op("_device_l2s")          # squared errors left on the device (no host wait)
        self._fused = None                              # (capacity, StagedBatch, FusedTrainStep) of the fused path

    # ------------------------------------------------------------------ bookkeeping
    def initialize(self):
        """Parameters are initialised at construction; kept for interface compatibility."""

    def _weight_matrices(self):
        return [p for n, p in self.model.named_parameters().items() if "W" in n.split("_")[1]]

    def _biases(self):
        return [p for n, p in self.model.named_parameters().items() if "b" in n.split("_")[1]]

    def get_train_op_rmse(self):
        return self.train_op_rmse

    def get_train_op_exp(self):
        return self.train_op

    def get_loss_op(self):
        return self.tower_exp_loss

    # Names of the optimiser's variables in a reference checkpoint: TensorFlow names a slot after
    # its variable ("near_W_H_384x128_l1:0" -> "near_W_H_384x128_l1/Nadam:0" and ".../Nadam_1:0" for
    # the two moments, ".../ExponentialMovingAverage:0" for the shadow), and the Nadam optimiser keeps
    # beta1_power / beta2_power (trainer_multi_tower.py:261-266, 451-470 saves every global variable).
    _SLOTS = ("/Nadam:0", "/Nadam_1:0", "/ExponentialMovingAverage:0")

    def _optimizer_slots(self):
        """{checkpoint name: tensor} of the two Nadam moments and the moving average of every parameter."""
        out = {}
        names = list(self.model.named_parameters().keys())
        by_id = {id(p): k for k, p in enumerate(self.parameters)}
        for name, p in self.model.named_parameters().items():
            k, base = by_id[id(p)], name[:-2]
            if isinstance(self.optimizer, FlatNadam):
                m, v, ema = self.optimizer.slots_of(k)
            else:
                st = self.optimizer.state.get(p, {})
                m, v, ema = st.get("exp_avg"), st.get("exp_avg_sq"), self.ema[k]
            for suffix, t in zip(self._SLOTS, (m, v, ema)):
                if t is not None:
                    out[base + suffix] = t
        assert len(names) == len(self.parameters)
        return out

    def _optimizer_steps(self) -> int:
        if isinstance(self.optimizer, FlatNadam):
            return self.optimizer.steps_done()
        steps = [int(st["step"]) for st in self.optimizer.state.values() if "step" in st]
        return max(steps) if steps else 0

    def save_numpy(self, npz_file):
        """Saves every variable under the reference's names (``near_W_H_384x128_l1:0`` ...): the weights,
        the two Nadam moments and the moving average of each, the step count behind the optimiser's bias
        corrections, the learning rate and the epoch counters (the reference saves all of
        ``tf.global_variables()``, ``trainer_multi_tower.py:451-470``)."""
        _, ext = os.path.splitext(npz_file)
        assert ext == ".npz"
        objs = {k: v.detach().cpu().numpy() for k, v in self.model.named_parameters().items()}
        objs.update({k: v.detach().cpu().numpy() for k, v in self._optimizer_slots().items()})
        steps = self._optimizer_steps()
        objs["optimizer_step:0"] = np.asarray(steps, dtype=np.int32)
        objs["beta1_power:0"] = np.asarray(0.9 ** (steps + 1), dtype=np.float32)
        objs["beta2_power:0"] = np.asarray(0.999 ** (steps + 1), dtype=np.float32)
        objs["learning_rate:0"] = np.asarray(self.learning_rate)
        objs["global_step:0"] = np.asarray(self.global_step, dtype=np.int32)
        objs["global_epoch_count:0"] = np.asarray(self.global_epoch_count, dtype=np.int32)
        objs["local_epoch_count:0"] = np.asarray(self.local_epoch_count, dtype=np.int32)
        np.savez(npz_file, **objs)

    def load_numpy(self, npz_file, strict=False):
        """Restores a checkpoint written by ``save_numpy`` or by the reference.  Weights, moments, moving
        averages and the optimiser's step count are restored when present; a checkpoint that holds only
        weights leaves the optimiser in the state of a new one around those weights (moments 0, step 0,
        moving average = weights).  A name that matches nothing is reported (the reference raises on an
        unknown name, ``trainer_multi_tower.py:493``; with ``strict`` so does this)."""
        import warnings
        objs = np.load(npz_file, allow_pickle=False)
        named = self.model.named_parameters()
        if not isinstance(self.optimizer, FlatNadam):       # torch creates its slots at the first step
            for p in self.parameters:
                if p not in self.optimizer.state:
                    self.optimizer.state[p] = {"step": torch.as_tensor(0.0), "mu_product": torch.as_tensor(1.0),
                                               "exp_avg": torch.zeros_like(p), "exp_avg_sq": torch.zeros_like(p)}
        slots = self._optimizer_slots()
        ignore = {"beta1_power:0", "beta2_power:0"}          # functions of the step count
        have_slots, steps, unknown = 0, None, []
        for k in objs.keys():
            arr = objs[k]
            if k in named or k in slots:
                p = named[k] if k in named else slots[k]
                have_slots += k in slots
                want = np.float32 if p.dtype == torch.float32 else np.float64
                if arr.dtype != want and strict:
                    raise TypeError(f"Cannot deserialize {arr.dtype} into {want}. You may want to set strict=False.")
                with torch.no_grad():
                    p.copy_(torch.from_numpy(arr.astype(want)).to(p.device).view(p.shape))
            elif k == "learning_rate:0":
                self.set_learning_rate(float(arr))
            elif k == "global_step:0":
                self.global_step = int(arr)
            elif k == "optimizer_step:0":
                steps = int(arr)
            elif k == "global_epoch_count:0":
                self.global_epoch_count = int(arr)
            elif k == "local_epoch_count:0":
                self.local_epoch_count = int(arr)
            elif k not in ignore:
                unknown.append(k)
        if unknown:
            msg = f"load_numpy: {len(unknown)} names of {npz_file} match no variable of this trainer: {unknown[:6]}"
            if strict:
                raise KeyError(msg)
            warnings.warn(msg)
        if isinstance(self.optimizer, FlatNadam):
            if have_slots == 0:
                self.optimizer.reset_state()                 # weights only: a new optimiser around them
            else:
                # a reference checkpoint has no optimizer_step: its global_step counts the same updates
                self.optimizer.set_steps(steps if steps is not None else self.global_step)
            if self.model.fused:
                self.model.pack_weights()
        else:
            n_steps = steps if steps is not None else self.global_step
            mu_product = 1.0      # torch.optim.NAdam keeps the running product of its momentum schedule
            for i in range(1, n_steps + 1):
                mu_product *= 0.9 * (1.0 - 0.5 * 0.96 ** (i * 0.004))
            for k, p in enumerate(self.parameters):
                if have_slots == 0:
                    self.optimizer.state.pop(p, None)
                    self.ema[k].copy_(p.detach())
                elif p in self.optimizer.state:
                    self.optimizer.state[p]["step"] = torch.as_tensor(float(n_steps))
                    self.optimizer.state[p]["mu_product"] = torch.as_tensor(mu_product)

    def set_learning_rate(self, lr: float):
        self.learning_rate = lr
        if isinstance(self.optimizer, FlatNadam):
            self.optimizer.set_lr(lr)
            return
        for g in self.optimizer.param_groups:
            g["lr"] = lr

    # ------------------------------------------------------------------ one tower, one batch
    def _tower_forward(self, device, fed, need_coord_grad):
        """Sort -> featurize -> atomic networks -> per-molecule sum for one fed batch
        (``trainer_multi_tower.py:295-350``).  The inputs are already on the device (one
        asynchronous copy by the feeder); nothing here synchronises with the host."""
        dt = self.precision
        fed.wait()
        x, y, z = fed.x, fed.y, fed.z
        if need_coord_grad:
            x, y, z = (c.detach().requires_grad_(True) for c in (x, y, z))
        acs = fed.acs    # what ani_sort returns, counted on the host while the batch was packed
        with torch.cuda.device(device):
            si, gi, _ = ani_mod.ani_sort(fed.types)
            fn = ani_mod.featurize_sorted_autograd if need_coord_grad else ani_mod.featurize_sorted
            feat_buf = fn(x, y, z, fed.types, fed.mol_offsets, fed.mol_counts, si, acs)   # [n_atoms, 384], H, C, N, O rows
            atom_out = self.model.atom_outputs(feat_buf, acs, gi)
            pred = torch.zeros(fed.n_mols, dtype=dt, device=device).index_add_(0, fed.mol_ids, atom_out)
        return dict(x=x, y=y, z=z, pred=pred, feat_buf=feat_buf, gi=gi, offsets=fed.offsets_host,
                    counts=fed.counts_host)

    # ------------------------------------------------------------------ feeding
    def feed_dataset(self, dataset, shuffle, target_ops, batch_size, fuzz=None, before_hooks=None):
        """Runs ``target_ops`` over the dataset; yields one list of results per round of towers,
        each result a list with one entry per tower that had a batch
        (``trainer_multi_tower.py:710-828``).  Training ops return None."""
        flat_ops = list(target_ops)
        names = [op.name for op in flat_ops]
        training = [n for n in names if n.startswith("train_op")]
        need_grad = bool(training) or "tower_coord_grads" in names or "tower_force_rmses" in names
        need_coord = "tower_coord_grads" in names or "tower_force_rmses" in names or "train_op_forces" in names
        np_dt = np.float32 if self.precision == torch.float32 else np.float64
        packed = PackedDataset.from_raw(dataset, np_dt)
        fused_names = {"train_op", "train_op_rmse", "train_op_mse", "unordered_l2s", "tower_l2s", "tower_exp_loss",
                       "tower_bids", "_device_l2s"}
        fused = (self.num_towers == 1 and isinstance(self.optimizer, FlatNadam) and self.model.fused
                 and len(training) == 1 and training[0] != "train_op_forces" and set(names) <= fused_names
                 and packed.ys is not None and packed.num_mols() > 0)
        # the fused path works on two batches at a time (this one's networks, the next one's featurizer)
        it = BatchFeeder(packed, batch_size, shuffle, fuzz, devices=self.towers, depth=3 if fused else 2,
                         hold=2 if fused else self.num_towers)
        try:
            if fused:
                yield from self._fused_rounds(it, names, training[0], packed.capacity(batch_size), before_hooks)
            else:
                yield from self._feed_rounds(it, names, training, need_grad, need_coord, before_hooks)
        finally:
            it.close()

    def _fused_rounds(self, it, names, kind, capacity, before_hooks):
        """Energy training on one device without autograd (``FusedTrainStep``): per batch sort,
        featurize, networks forward, molecule energies + MSE gradient, networks backward, weight
        gradients; the gradient of the requested loss is the MSE gradient times a scalar --
        1 / (2 rmse) for the rmse loss, exp(rmse) / (2 rmse) for the reference's exp(rmse) loss
        (``trainer_multi_tower.py:390-396``) -- computed on the device, so nothing waits for the GPU
        unless a result is asked for."""
        from ..staged import StagedBatch
        from .fused_step import FusedTrainStep
        cap_atoms, cap_mols = max(capacity[0], 1), max(capacity[1], 1)
        dev = self.towers[0]
        if self._fused is None or self._fused[0][0] < cap_atoms or self._fused[0][1] < cap_mols:
            self._fused = ((cap_atoms, cap_mols),
                           [StagedBatch(cap_atoms, cap_mols, device=dev), StagedBatch(cap_atoms, cap_mols, device=dev)],
                           FusedTrainStep(self.model, self.optimizer, cap_atoms, cap_mols, device=dev),
                           torch.cuda.Stream(device=dev))
        _, sbs, step, side = self._fused
        if getattr(self, "_rmse_buf", None) is None:
            self._rmse_buf = torch.zeros((), dtype=torch.float32, device=dev)
        # Two batches in flight: sort + featurize of the NEXT batch run on a side stream beside the network
        # kernels of this one (they need nothing but the coordinates; the network kernels leave a quarter of
        # the SMs free), as in StepPipeline.  The sequence of weights is that of the serial order.
        feeder = iter(it)

        def start(fed, sb):
            """Sort + featurize of a fed batch on the side stream, behind everything enqueued on the main one
            (the previous use of ``sb`` among it)."""
            side.wait_stream(torch.cuda.current_stream(dev))
            with torch.cuda.stream(side):
                fed.wait()
                sb.adopt(fed)
                step.featurize_pass(sb)

        with torch.cuda.device(dev):
            fed = next(feeder, None)
            if fed is not None:
                start(fed, sbs[0])
        k = 0
        while fed is not None:
            if before_hooks is not None:
                self._run_hooks(before_hooks)
            with torch.cuda.device(dev), torch.no_grad():
                sb = sbs[k & 1]
                main = torch.cuda.current_stream(dev)
                main.wait_stream(side)                      # this batch's features are there
                nxt = next(feeder, None)
                if nxt is not None:
                    start(nxt, sbs[(k + 1) & 1])
                step.forward_backward(sb, fed.ys, feature_grad=False, featurized=True)
                l2 = step.l2s[:fed.n_mols]
                rmse = None
                if kind in ("train_op", "train_op_rmse"):
                    # one launch: rmse on the device, the weight gradients scaled by d loss / d mse
                    rmse = self._rmse_buf
                    g = self.optimizer.flat_grads
                    _lib.check(_lib.lib().ani_scale_by_loss_f32(
                        g.data_ptr(), g.numel(), l2.data_ptr(), fed.n_mols, 2 if kind == "train_op" else 1,
                        rmse.data_ptr(), ctypes.c_void_p(main.cuda_stream)), "ani_scale_by_loss_f32")
                elif "tower_exp_loss" in names:
                    rmse = l2.mean().sqrt().clamp_min(1e-30)
                average_gradients(self.parameters, self.optimizer.flat_grads)
                self.optimizer.step()
                self.global_step += 1
                row = []
                for n in names:
                    if n.startswith("train_op"):
                        row.append(None)
                    elif n in ("unordered_l2s", "tower_l2s"):
                        row.append([l2.cpu().numpy()])
                    elif n == "_device_l2s":
                        row.append([l2.clone()])
                    elif n == "tower_exp_loss":
                        row.append([float(torch.exp(rmse.double()))])
                    elif n == "tower_bids":
                        row.append([np.array(fed.index)])
                fed, k = nxt, k + 1
            yield row

    def _feed_rounds(self, it, names, training, need_grad, need_coord, before_hooks):
        done = False
        while not done:
            round_batches = []
            for _ in range(self.num_towers):
                try:
                    round_batches.append(next(it))
                except StopIteration:
                    done = True
                    break
            if not round_batches:
                break
            if before_hooks is not None:
                self._run_hooks(before_hooks)
            per_tower = []
            losses = []
            ctx = torch.enable_grad() if need_grad else torch.no_grad()
            with ctx:
                for tower, fed in zip(self.towers, round_batches):
                    out = self._tower_forward(tower, fed, need_coord)
                    mol_yts, mol_grads = fed.ys, fed.grads
                    res = {"tower_bids": np.array(fed.index), "tower_mos": out["offsets"]}
                    pred = out["pred"]
                    # only what was asked for is brought to the host: every copy is a wait for the GPU
                    if "tower_preds" in names:
                        res["tower_preds"] = pred.detach().cpu().numpy()
                    if mol_yts is not None:
                        l2 = (pred - mol_yts) ** 2
                        if "tower_l2s" in names or "unordered_l2s" in names:
                            res["tower_l2s"] = l2.detach().cpu().numpy()
                            res["unordered_l2s"] = res["tower_l2s"]
                        if "_device_l2s" in names:
                            res["_device_l2s"] = l2.detach().clone()
                        rmse = torch.sqrt(l2.mean())
                        if "tower_exp_loss" in names:
                            res["tower_exp_loss"] = float(torch.exp(rmse.detach().double()))
                    if "tower_features" in names:
                        res["tower_features"] = out["feat_buf"].detach()[out["gi"].long()].cpu().numpy()
                    if need_coord:
                        gx, gy, gz = torch.autograd.grad(pred.sum(), [out["x"], out["y"], out["z"]],
                                                         create_graph="train_op_forces" in names,
                                                         retain_graph=True)
                        res["tower_coord_grads"] = [g.detach().cpu().numpy() for g in (gx, gy, gz)]
                        if mol_grads is not None:
                            frmse = sum(torch.sqrt(((-g - mol_grads[k]) ** 2).mean()) for k, g in enumerate((gx, gy, gz)))
                            res["tower_force_rmses"] = float(frmse.detach())
                    if training and mol_yts is not None:
                        kind = training[0]
                        if kind == "train_op":
                            losses.append(torch.exp(rmse.double()))
                        elif kind == "train_op_rmse":
                            losses.append(rmse)
                        elif kind == "train_op_mse":
                            losses.append(l2.mean())
                        elif kind == "train_op_forces":
                            losses.append(torch.exp(frmse.double()))
                    per_tower.append(res)
                if training and losses:
                    self._apply_gradients(losses)
            yield [[r.get(n) for r in per_tower] if not n.startswith("train_op") else None for n in names]

    def _run_hooks(self, hooks):
        hooks = hooks if isinstance(hooks, (list, tuple)) else [hooks]
        for h in hooks:
            if isinstance(h, _Op) and h.name == "max_norm_ops":
                # tf.clip_by_norm(w, 3.0, axes=1) over all weight matrices, trainer_multi_tower.py:432-436
                if isinstance(self.optimizer, FlatNadam):
                    if not hasattr(self, "_weight_indices"):
                        weights = {id(w) for w in self._weight_matrices()}
                        self._weight_indices = [k for k, p in enumerate(self.parameters) if id(p) in weights]
                    self.optimizer.clip_rows(self._weight_indices, 3.0)
                    continue
                with torch.no_grad():
                    for w in self._weight_matrices():
                        norms = w.norm(dim=1, keepdim=True).clamp_min(1e-30)
                        w.mul_(torch.clamp(3.0 / norms, max=1.0))
            elif callable(h):
                h()

    def _apply_gradients(self, losses):
        """Average of the tower gradients (and of all ranks when torch.distributed is up),
        global-norm clip 5, Nadam step, EMA (``trainer_multi_tower.py:421-427``)."""
        fused = isinstance(self.optimizer, FlatNadam)
        self.optimizer.zero_grad(set_to_none=not fused)
        total = sum(l.to(self.towers[0]) if l.device != self.towers[0] else l for l in losses) / len(losses)
        total.backward()
        self.global_step += 1
        if fused:      # clip, Nadam and the moving average are inside the fused step
            average_gradients(self.parameters, self.optimizer.flat_grads)
            self.optimizer.step()
            return
        average_gradients(self.parameters)
        torch.nn.utils.clip_grad_norm_(self.parameters, 5.0)
        self.optimizer.step()
        with torch.no_grad():
            decay = min(self.ema_decay, (1.0 + self.global_step) / (10.0 + self.global_step))
            for e, p in zip(self.ema, self.parameters):
                e.mul_(decay).add_(p.detach(), alpha=1.0 - decay)

    # ------------------------------------------------------------------ user-facing helpers
    def _device_predictions(self, dataset, batch_size):
        """Energies (and squared errors, when the data set has targets) of every batch, left on
        the devices: nothing here waits for the GPU, so the host runs ahead of it by as many
        batches as the feeder allows, and the caller synchronises once."""
        np_dt = np.float32 if self.precision == torch.float32 else np.float64
        if self._evaluator_usable(dataset):
            return self._evaluator_predictions(dataset, batch_size)
        it = BatchFeeder(PackedDataset.from_raw(dataset, np_dt), batch_size, False, None,
                         devices=self.towers, depth=2, hold=self.num_towers)
        preds, l2s = [], []
        try:
            with torch.no_grad():
                for k, fed in enumerate(it):
                    out = self._tower_forward(self.towers[k % self.num_towers], fed, False)
                    preds.append(out["pred"])
                    if fed.ys is not None:
                        l2s.append((out["pred"] - fed.ys) ** 2)
        finally:
            it.close()
        return preds, l2s

    def predict(self, dataset, batch_size=2048):
        """Predicted energies in dataset order (``trainer_multi_tower.py:655-678``)."""
        preds, _ = self._device_predictions(dataset, batch_size)
        if not preds:
            return []
        return torch.cat([p.to(self.towers[0]) for p in preds]).cpu().tolist()

    def featurize(self, dataset, batch_size=1024):
        """Per-molecule feature arrays, in dataset order (``trainer_multi_tower.py:617-653``)."""
        ops = [self.tower_features, self.tower_mos, self.tower_bids]
        for feats, mos, ids in self.feed_dataset(dataset, False, ops, batch_size):
            for k in np.argsort(np.array(ids)):
                for f in _split_rows(feats[k], mos[k]):
                    yield f

    def coordinate_gradients(self, dataset, batch_size=1024, use_evaluator=True):
        """Per-molecule ``(n, 3)`` gradients of the predicted energy
        (``trainer_multi_tower.py:580-614``).  On one float32 tower with the fused networks the
        batches go through the allocation-free evaluator (``khan_b200.inference.EnergyForces``: C-ABI
        calls only, no host wait per batch); ``use_evaluator=False`` forces the autograd path."""
        # an iterator, as in the reference; the per-batch lists are chained in C, so a molecule costs no
        # Python frame of its own (two nested generators had cost more than cutting the arrays)
        if use_evaluator and self._evaluator_usable(dataset):
            return itertools.chain.from_iterable(self._evaluator_gradients(dataset, batch_size))
        return itertools.chain.from_iterable(self._autograd_gradients(dataset, batch_size))

    def _autograd_gradients(self, dataset, batch_size):
        """One list of per-molecule ``(n, 3)`` arrays per batch, through ``feed_dataset`` and autograd."""
        ops = [self.tower_coord_grads, self.tower_mos, self.tower_bids]
        for grads, mos, ids in self.feed_dataset(dataset, False, ops, batch_size):
            for k in np.argsort(np.array(ids)):
                # one (n_atoms, 3) array per batch, cut once into per-molecule pieces
                yield _split_rows(np.stack(grads[k], axis=1), mos[k])

    def _evaluator_usable(self, dataset) -> bool:
        """One float32 CUDA tower with the fused networks: batches can go through the
        allocation-free evaluator (``khan_b200.inference.EnergyForces``)."""
        return (self.num_towers == 1 and self.precision == torch.float32 and self.model.fused
                and self.towers[0].type == "cuda" and dataset.num_mols() > 0)

    def _evaluator(self, packed, batch_size):
        from ..inference import EnergyForces
        from ..staged import StagedBatch
        cap_atoms, cap_mols = (max(v, 1) for v in packed.capacity(batch_size))
        dev = self.towers[0]
        cached = getattr(self, "_infer", None)
        if cached is None or cached[0][0] < cap_atoms or cached[0][1] < cap_mols:
            self._infer = cached = ((cap_atoms, cap_mols), StagedBatch(cap_atoms, cap_mols, device=dev),
                                    EnergyForces(self.model, cap_atoms, cap_mols, device=dev))
        return cached[1], cached[2]

    def _evaluator_predictions(self, dataset, batch_size):
        """``_device_predictions`` through the evaluator: sort, featurize, networks forward and the
        molecule sums as four C-ABI calls per batch, the weights packed once."""
        packed = PackedDataset.from_raw(dataset, np.float32)
        sb, ev = self._evaluator(packed, batch_size)
        dev = self.towers[0]
        # two batches at a time: sort + featurize of the next one on a side stream beside the networks of this one
        twin = getattr(self, "_infer_twin", None)
        if twin is None or twin[0].n_atoms_cap < sb.n_atoms_cap or twin[0].n_mols_cap < sb.n_mols_cap:
            from ..staged import StagedBatch
            twin = self._infer_twin = (StagedBatch(sb.n_atoms_cap, sb.n_mols_cap, device=dev), torch.cuda.Stream(device=dev))
        sbs, side = (sb, twin[0]), twin[1]
        it = BatchFeeder(packed, batch_size, False, None, devices=self.towers, depth=3, hold=2)
        preds, l2s = [], []

        def start(fed, target):
            side.wait_stream(torch.cuda.current_stream(dev))      # the previous use of `target` is among it
            with torch.cuda.stream(side):
                fed.wait()
                target.adopt(fed)
                ev.featurize(target)

        try:
            with torch.cuda.device(dev), torch.no_grad():
                feeder = iter(it)
                fed, k = next(feeder, None), 0
                if fed is not None:
                    start(fed, sbs[0])
                while fed is not None:
                    torch.cuda.current_stream(dev).wait_stream(side)
                    nxt = next(feeder, None)
                    if nxt is not None:
                        start(nxt, sbs[(k + 1) & 1])
                    ev.run(sbs[k & 1], pack=(k == 0), forces=False, featurized=True)
                    preds.append(ev.mol_energy[:fed.n_mols].clone())
                    if fed.ys is not None:
                        l2s.append((preds[-1] - fed.ys) ** 2)
                    fed, k = nxt, k + 1
        finally:
            it.close()
        return preds, l2s

    def _evaluator_gradients(self, dataset, batch_size):
        """Gradients of all molecules through the evaluator, one list per batch.  The result of a batch is copied to a pinned
        host buffer behind its kernels, and the host cuts the PREVIOUS batch into per-molecule arrays while
        the GPU works on this one (cutting 32,768 molecules takes as long as computing them)."""
        packed = PackedDataset.from_raw(dataset, np.float32)
        sb, ev = self._evaluator(packed, batch_size)
        cap = sb.n_atoms_cap
        ring = getattr(self, "_grad_ring", None)
        if ring is None or ring[0].shape[0] < cap:
            ring = self._grad_ring = [torch.empty((cap, 3), dtype=torch.float32).pin_memory() for _ in range(3)]
        it = BatchFeeder(packed, batch_size, False, None, devices=self.towers, depth=2, hold=1)
        pending = []      # (host buffer, event, n_atoms, batch index) of batches whose copy is in flight
        slices = packed.batch_slices(batch_size)

        def finished(entry):
            buf, evt, n, k = entry
            evt.synchronize()
            return list(map(buf[:n].numpy().copy().__getitem__, slices[k]))

        try:
            with torch.cuda.device(self.towers[0]), torch.no_grad():
                for k, fed in enumerate(it):
                    fed.wait()
                    sb.adopt(fed)
                    ev.run(sb, pack=(k == 0))
                    n = fed.n_atoms
                    buf = ring[k % len(ring)]
                    buf[:n].copy_(sb.grads[:, :n].t(), non_blocking=True)      # (n_atoms, 3), strided read on the device
                    evt = torch.cuda.Event()
                    evt.record()
                    pending.append((buf, evt, n, fed.index))
                    if len(pending) == len(ring):       # the buffer of batch k + 1 must be free again
                        yield finished(pending.pop(0))
        finally:
            it.close()
        for entry in pending:
            yield finished(entry)

    def eval_abs_rmse(self, dataset, batch_size=1024):
        """Absolute RMSE of the energies in kcal/mol (``trainer_multi_tower.py:560-578``)."""
        _, l2s = self._device_predictions(dataset, batch_size)
        total = torch.cat([v.to(self.towers[0]).double() for v in l2s])
        return float(torch.sqrt(total.mean())) * HARTREE_TO_KCAL_PER_MOL


    def eval_rel_rmse(self, dataset, group_ys, batch_size=1024):
        """Conformer-group RMSE in kcal/mol; the dataset's own targets are ignored
        (``trainer_multi_tower.py:680-702``)."""
        return ed_harder_rmse(group_ys, self.predict(dataset, batch_size)) * HARTREE_TO_KCAL_PER_MOL

    def eval_eh_rmse(self, dataset, group_ys, batch_size=1024):
        """Old name of :meth:`eval_rel_rmse` (``trainer_multi_tower.py:704-708``)."""
        return self.eval_rel_rmse(dataset, group_ys, batch_size)

    def train(self, save_dir, rd_train, rd_test, rd_gdb11=None, eval_names=(), eval_datasets=(),
              eval_groups=(), batch_size=1024, max_local_epoch_count=25, max_batch_size=1e4,
              min_learning_rate=1e-7, max_global_epoch_count=1000, log=print):
        """The reference's training schedule (``trainer_multi_tower.py:832-891``): train with the
        exp-RMSE loss, the max-norm hook and a fuzz that shrinks with the epoch; keep the weights
        with the best test error in ``save_dir/best.npz``; after ``max_local_epoch_count`` epochs
        without improvement reload them, halve the learning rate and add 128 to the batch size.
        Returns the best test error (kcal/mol)."""
        train_ops = [self._device_l2s, self.train_op]
        best = self.eval_abs_rmse(rd_test)
        os.makedirs(save_dir, exist_ok=True)
        best_file = os.path.join(save_dir, "best.npz")
        self.save_numpy(best_file)
        start = time.time()
        while (batch_size < max_batch_size and self.learning_rate > min_learning_rate
               and self.global_epoch_count <= max_global_epoch_count):
            while (self.local_epoch_count < max_local_epoch_count
                   and self.global_epoch_count <= max_global_epoch_count):
                fuzz = max(1e-3 / (self.global_epoch_count + 1), 1e-5)
                results = list(self.feed_dataset(rd_train, shuffle=True, target_ops=train_ops,
                                                 batch_size=batch_size, before_hooks=self.max_norm_ops,
                                                 fuzz=fuzz))
                l2s = torch.cat([v.reshape(-1).double() for r in results for v in r[0]])   # one wait per epoch
                train_rmse = float(torch.sqrt(l2s.mean())) * HARTREE_TO_KCAL_PER_MOL
                test_rmse = self.eval_abs_rmse(rd_test)
                line = (f"{save_dir} tpe: {time.time() - start:.2f}s, g-epoch {self.global_epoch_count} "
                        f"l-epoch {self.local_epoch_count} lr {self.learning_rate:.0e} batch_size {batch_size} "
                        f"| train/test abs rmse: {train_rmse:.2f} kcal/mol, {test_rmse:.2f} kcal/mol")
                start = time.time()
                if test_rmse < best:
                    self.save_numpy(best_file)
                    best = test_rmse
                    self.local_epoch_count = 0
                else:
                    self.local_epoch_count += 1
                self.global_epoch_count += 1
                if rd_gdb11 is not None:
                    line += f" | gdb11 abs rmse {self.eval_abs_rmse(rd_gdb11):.2f} kcal/mol"
                for name, data, groups in zip(eval_names, eval_datasets, eval_groups):
                    line += (f" | {name} abs/rel rmses {self.eval_abs_rmse(data):.2f} kcal/mol, "
                             f"{self.eval_rel_rmse(data, groups):.2f} kcal/mol")
                if log is not None:
                    log(line)
            if log is not None:
                log("========== Decreasing learning rate, increasing batch size ==========")
            self.load_numpy(best_file)
            self.set_learning_rate(self.learning_rate * 0.5)
            self.local_epoch_count = 0
            self.global_epoch_count += 1
            batch_size += 128
        return best


class TrainerMultiGPU(TrainerMultiTower):
    """The spelling used in the reference README (``README.md:138-151``): ``TrainerMultiGPU(sess,
    n_gpus=...)``."""

    def __init__(self, sess=None, n_gpus=1, precision=torch.float32, layer_sizes=(128, 128, 64, 1), **kw):
        if n_gpus != 1:
            raise NotImplementedError(
                f"TrainerMultiGPU(n_gpus={n_gpus}): one process drives one GPU here; start {n_gpus} processes with "
                "torchrun (one rank per GPU) and construct TrainerMultiGPU(n_gpus=1) in each -- its device is the "
                "rank's current CUDA device and the weight gradients are averaged with one NCCL all-reduce")
        super().__init__(sess, [torch.device("cuda", torch.cuda.current_device() if torch.cuda.is_available() else 0)],
                         precision, layer_sizes=layer_sizes, **kw)

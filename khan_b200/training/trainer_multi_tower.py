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
(``trainer_multi_tower.py:137-179``).  The learning-rate schedule of ``train()`` is host-side
policy and is not reproduced.
"""
from __future__ import annotations

import os

import numpy as np
import torch

from .. import ani_mod
from ..model import activations
from ..model.nn import MoleculeNN

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


def average_gradients(parameters):
    """Mean of the weight gradients over all ranks: ONE all-reduce of a flat bucket (296,452
    values for four 384-128-128-64-1 networks), the data-parallel replacement of the reference's
    per-variable concat + reduce_mean on the CPU (``trainer_multi_tower.py:137-179``).  A no-op
    without an initialised process group."""
    import torch.distributed as dist
    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size() == 1:
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
        self.num_towers = len(self.towers)
        self.precision = precision
        self.feat_size = ani_mod.FEATURE_SIZE
        # parameters live on the first tower; other towers get a broadcast copy per step
        self.model = MoleculeNN(layer_sizes=(self.feat_size,) + tuple(layer_sizes), precision=precision,
                                activation_fn=activation_fn, prefix="near_", device=self.towers[0],
                                seed=seed, init=init, split_precision=split_precision)
        self.all_models = [self.model]
        self.parameters = self.model.get_parameters()
        self.learning_rate = 1e-3
        self.optimizer = torch.optim.NAdam(self.parameters, lr=self.learning_rate, betas=(0.9, 0.999), eps=1e-8)
        self.global_step = 0
        self.global_epoch_count = 0
        self.local_epoch_count = 0
        self.ema_decay = 0.9999
        self.ema = [p.detach().clone() for p in self.parameters]
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

    def save_numpy(self, npz_file):
        """Saves every variable under the reference's names (``near_W_H_384x128_l1:0`` ...)."""
        _, ext = os.path.splitext(npz_file)
        assert ext == ".npz"
        objs = {k: v.detach().cpu().numpy() for k, v in self.model.named_parameters().items()}
        objs["learning_rate:0"] = np.asarray(self.learning_rate)
        objs["global_step:0"] = np.asarray(self.global_step, dtype=np.int32)
        objs["global_epoch_count:0"] = np.asarray(self.global_epoch_count, dtype=np.int32)
        objs["local_epoch_count:0"] = np.asarray(self.local_epoch_count, dtype=np.int32)
        np.savez(npz_file, **objs)

    def load_numpy(self, npz_file, strict=False):
        objs = np.load(npz_file, allow_pickle=False)
        named = self.model.named_parameters()
        for k in objs.keys():
            arr = objs[k]
            if k in named:
                p = named[k]
                want = np.float32 if p.dtype == torch.float32 else np.float64
                if arr.dtype != want and strict:
                    raise TypeError(f"Cannot deserialize {arr.dtype} into {want}. You may want to set strict=False.")
                with torch.no_grad():
                    p.copy_(torch.from_numpy(arr.astype(want)).to(p.device))
            elif k == "learning_rate:0":
                self.set_learning_rate(float(arr))
            elif k == "global_step:0":
                self.global_step = int(arr)
            elif k == "global_epoch_count:0":
                self.global_epoch_count = int(arr)
            elif k == "local_epoch_count:0":
                self.local_epoch_count = int(arr)

    def set_learning_rate(self, lr: float):
        self.learning_rate = lr
        for g in self.optimizer.param_groups:
            g["lr"] = lr

    # ------------------------------------------------------------------ one tower, one batch
    def _tower_forward(self, device, mol_Xs, mol_ids, need_coord_grad):
        dt = self.precision
        xyz = torch.from_numpy(np.ascontiguousarray(mol_Xs[:, 1:4].T)).to(device=device, dtype=dt)
        x, y, z = xyz[0].contiguous(), xyz[1].contiguous(), xyz[2].contiguous()
        if need_coord_grad:
            x.requires_grad_(True); y.requires_grad_(True); z.requires_grad_(True)
        types_host = mol_Xs[:, 0].astype(np.int32)
        a = torch.from_numpy(types_host).to(device)
        ids_host = np.asarray(mol_ids, dtype=np.int64)
        n_mols = int(ids_host[-1]) + 1 if len(ids_host) else 0
        counts = np.bincount(ids_host, minlength=n_mols).astype(np.int32)
        offsets = (np.cumsum(counts) - counts).astype(np.int32)   # tf.cumsum(exclusive=True)
        mo = torch.from_numpy(offsets).to(device)
        mac = torch.from_numpy(counts).to(device)
        acs = np.bincount(types_host, minlength=4).astype(np.int32)   # what ani_sort returns, on the host
        with torch.cuda.device(device):
            si, gi, _ = ani_mod.ani_sort(a)
            fn = ani_mod.featurize_sorted_autograd if need_coord_grad else ani_mod.featurize_sorted
            feat_buf = fn(x, y, z, a, mo, mac, si, acs)   # [n_atoms, 384], H rows, C rows, N rows, O rows
            model = self.model
            atom_out = model.atom_outputs(feat_buf, acs, gi)
            ids = torch.from_numpy(ids_host).to(device)
            pred = torch.zeros(n_mols, dtype=dt, device=device).index_add_(0, ids, atom_out)
        return dict(x=x, y=y, z=z, pred=pred, feat_buf=feat_buf, gi=gi, offsets=offsets, counts=counts)

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
        it = dataset.iterate(batch_size=batch_size, shuffle=shuffle, fuzz=fuzz)
        b_idx = 0
        done = False
        while not done:
            round_batches = []
            for _ in range(self.num_towers):
                try:
                    round_batches.append((b_idx, next(it)))
                    b_idx += 1
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
                for tower, (bid, (mol_Xs, mol_ids, mol_yts, mol_grads)) in zip(self.towers, round_batches):
                    out = self._tower_forward(tower, mol_Xs, mol_ids, need_coord)
                    res = {"tower_bids": np.array(bid), "tower_mos": out["offsets"]}
                    pred = out["pred"]
                    res["tower_preds"] = pred.detach().cpu().numpy()
                    if mol_yts is not None:
                        labels = torch.as_tensor(np.asarray(mol_yts), dtype=self.precision, device=tower)
                        l2 = (pred - labels) ** 2
                        res["tower_l2s"] = l2.detach().cpu().numpy()
                        res["unordered_l2s"] = res["tower_l2s"]
                        rmse = torch.sqrt(l2.mean())
                        res["tower_exp_loss"] = float(torch.exp(rmse.detach().double()))
                    if "tower_features" in names:
                        res["tower_features"] = out["feat_buf"].detach()[out["gi"].long()].cpu().numpy()
                    if need_coord:
                        gx, gy, gz = torch.autograd.grad(pred.sum(), [out["x"], out["y"], out["z"]],
                                                         create_graph="train_op_forces" in names,
                                                         retain_graph=True)
                        res["tower_coord_grads"] = [g.detach().cpu().numpy() for g in (gx, gy, gz)]
                        if mol_grads is not None:
                            f = torch.as_tensor(np.asarray(mol_grads), dtype=self.precision, device=tower)
                            frmse = sum(torch.sqrt(((-g - f[:, k]) ** 2).mean()) for k, g in enumerate((gx, gy, gz)))
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
                with torch.no_grad():   # tf.clip_by_norm(w, 3.0, axes=1), trainer_multi_tower.py:432-436
                    for w in self._weight_matrices():
                        norms = w.norm(dim=1, keepdim=True).clamp_min(1e-30)
                        w.mul_(torch.clamp(3.0 / norms, max=1.0))
            elif callable(h):
                h()

    def _apply_gradients(self, losses):
        """Average of the tower gradients (and of all ranks when torch.distributed is up),
        global-norm clip 5, Nadam step, EMA (``trainer_multi_tower.py:421-427``)."""
        self.optimizer.zero_grad(set_to_none=True)
        total = sum(l.to(self.towers[0]) if l.device != self.towers[0] else l for l in losses) / len(losses)
        total.backward()
        average_gradients(self.parameters)
        torch.nn.utils.clip_grad_norm_(self.parameters, 5.0)
        self.optimizer.step()
        self.global_step += 1
        with torch.no_grad():
            for e, p in zip(self.ema, self.parameters):
                e.mul_(self.ema_decay).add_(p.detach(), alpha=1.0 - self.ema_decay)

    # ------------------------------------------------------------------ user-facing helpers
    def predict(self, dataset, batch_size=2048):
        """Predicted energies in dataset order (``trainer_multi_tower.py:655-678``)."""
        ordered = []
        for ys, ids in self.feed_dataset(dataset, False, [self.tower_preds, self.tower_bids], batch_size):
            order = np.argsort(np.array(ids))
            for k in order:
                ordered.extend(ys[k].tolist())
        return ordered

    def featurize(self, dataset, batch_size=1024):
        """Per-molecule feature arrays, in dataset order (``trainer_multi_tower.py:617-653``)."""
        ops = [self.tower_features, self.tower_mos, self.tower_bids]
        for feats, mos, ids in self.feed_dataset(dataset, False, ops, batch_size):
            for k in np.argsort(np.array(ids)):
                for f in np.split(feats[k], mos[k][1:]):
                    yield f

    def coordinate_gradients(self, dataset, batch_size=1024):
        """Per-molecule ``(n, 3)`` gradients of the predicted energy
        (``trainer_multi_tower.py:580-614``)."""
        ops = [self.tower_coord_grads, self.tower_mos, self.tower_bids]
        for grads, mos, ids in self.feed_dataset(dataset, False, ops, batch_size):
            for k in np.argsort(np.array(ids)):
                gx, gy, gz = grads[k]
                cut = mos[k][1:]
                for x, y, z in zip(np.split(gx, cut), np.split(gy, cut), np.split(gz, cut)):
                    yield np.vstack([x, y, z]).transpose()

    def eval_abs_rmse(self, dataset, batch_size=1024):
        res = list(self.feed_dataset(dataset, False, [self.unordered_l2s], batch_size))
        l2s = np.concatenate([np.concatenate(r[0]).reshape(-1) for r in res])
        return float(np.sqrt(np.mean(l2s)) * HARTREE_TO_KCAL_PER_MOL)


class TrainerMultiGPU(TrainerMultiTower):
    """The spelling used in the reference README (``README.md:138-151``): ``TrainerMultiGPU(sess,
    n_gpus=...)``."""

    def __init__(self, sess=None, n_gpus=1, precision=torch.float32, layer_sizes=(128, 128, 64, 1), **kw):
        super().__init__(sess, [torch.device("cuda", i) for i in range(n_gpus)], precision,
                         layer_sizes=layer_sizes, **kw)

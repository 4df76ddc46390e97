"""The khan front end (RawDataset + TrainerMultiTower) on the GPU: predictions, features and
coordinate gradients agree with the CPU oracle / a dense float64 evaluation of the same weights,
training lowers the loss, checkpoints round-trip."""
import numpy as np
import pytest

from conftest import normwise
from khan_b200.data import synthetic as syn

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def small_dataset():
    from khan_b200 import RawDataset
    b = syn.config1(n_mols=70)
    rng = np.random.default_rng(0)
    ys = rng.normal(size=b.n_mols)
    return RawDataset(b.molecules(), ys), b


def _dense_energy(trainer, feats_by_mol, mols):
    """Molecule energies from per-molecule feature arrays with float64 dense algebra."""
    import torch
    out = []
    for f, mol in zip(feats_by_mol, mols):
        e = 0.0
        for row, t in zip(f, mol[:, 0].astype(int)):
            a = torch.from_numpy(row.astype(np.float64))
            ann = trainer.model.anns[t]
            last = len(ann.Ws) - 1
            for k, (w, b) in enumerate(zip(ann.Ws, ann.bs)):
                a = a @ w.detach().double().cpu() + b.detach().double().cpu()
                if k != last:
                    a = trainer.model.activation_fn(a)
            e += float(a)
        out.append(e)
    return np.array(out)


def test_featurize_and_predict(small_dataset, oracle_mod):
    import torch
    from khan_b200 import TrainerMultiTower
    from khan_b200.model import activations
    ds, b = small_dataset
    tr = TrainerMultiTower(None, ["cuda:0"], torch.float32, layer_sizes=(128, 128, 64, 1),
                           activation_fn=activations.celu, seed=5)
    feats = list(tr.featurize(ds, batch_size=32))           # 3 batches, last one ragged
    assert len(feats) == b.n_mols
    si, gi, ac = oracle_mod.ani_sort(b.atomic_numbers)
    x, y, z = b.coords(np.float32)
    ref = oracle_mod.featurize(x, y, z, b.atomic_numbers, b.mol_offsets, b.mol_atom_counts, si, ac)
    ref_rows = np.concatenate([r.reshape(-1, 384) for r in ref])[gi]
    got_rows = np.concatenate(feats)
    assert normwise(got_rows, ref_rows) < 1e-5
    preds = np.array(tr.predict(ds, batch_size=32))
    dense = _dense_energy(tr, feats, ds.all_Xs)
    assert normwise(preds, dense) < 1e-4


def test_coordinate_gradients_match_finite_differences(oracle_mod):
    import torch
    from khan_b200 import RawDataset, TrainerMultiTower
    from khan_b200.model import activations
    b = syn.kat_fixture()
    ds = RawDataset(b.molecules())
    tr = TrainerMultiTower(None, ["cuda:0"], torch.float64, layer_sizes=(128, 128, 64, 1),
                           activation_fn=activations.gaussian, seed=2, init="he")
    grads = list(tr.coordinate_gradients(ds, batch_size=8))
    assert [g.shape for g in grads] == [(8, 3), (3, 3)]
    base = ds.all_Xs
    for mol_idx, atom, axis in [(0, 0, 0), (0, 3, 2), (1, 1, 1)]:
        e = []
        for sign in (+1, -1):
            mols = [m.copy() for m in base]
            mols[mol_idx][atom, 1 + axis] += sign * 1e-5
            e.append(tr.predict(RawDataset(mols), batch_size=8)[mol_idx])
        fd = (e[0] - e[1]) / 2e-5
        assert abs(fd - grads[mol_idx][atom, axis]) < 1e-6 * max(1.0, abs(fd))


def test_training_lowers_the_loss_and_checkpoint_round_trips(small_dataset, tmp_path):
    import torch
    from khan_b200 import TrainerMultiTower
    from khan_b200.model import activations
    ds, b = small_dataset
    tr = TrainerMultiTower(None, ["cuda:0"], torch.float32, layer_sizes=(128, 128, 64, 1),
                           activation_fn=activations.gaussian, seed=1, init="he")
    first = tr.eval_abs_rmse(ds, batch_size=35)
    for _ in range(30):
        list(tr.feed_dataset(ds, shuffle=True, target_ops=[tr.train_op_mse], batch_size=35,
                             before_hooks=tr.max_norm_ops))
    after = tr.eval_abs_rmse(ds, batch_size=35)
    assert after < first
    assert tr.global_step == 60
    path = str(tmp_path / "ckpt.npz")
    tr.save_numpy(path)
    keys = set(np.load(path).keys())
    assert "near_W_H_384x128_l1:0" in keys and "near_b_O_64x1_l4:0" in keys
    other = TrainerMultiTower(None, ["cuda:0"], torch.float32, layer_sizes=(128, 128, 64, 1),
                              activation_fn=activations.gaussian, seed=9)
    other.load_numpy(path)
    np.testing.assert_allclose(other.predict(ds, 64), tr.predict(ds, 64), rtol=0, atol=1e-6)
    # the optimiser state travels too, under the reference's slot names: the resumed trainer takes the
    # SAME next steps as the one that kept running (moments, moving average and step count restored)
    assert {"near_W_H_384x128_l1/Nadam:0", "near_W_H_384x128_l1/Nadam_1:0",
            "near_W_H_384x128_l1/ExponentialMovingAverage:0", "beta1_power:0", "optimizer_step:0"} <= keys
    assert other.optimizer.steps_done() == tr.optimizer.steps_done() == 60
    assert torch.equal(other.optimizer.m, tr.optimizer.m) and torch.equal(other.optimizer.ema, tr.optimizer.ema)
    for t in (tr, other):
        list(t.feed_dataset(ds, shuffle=False, target_ops=[t.train_op_mse], batch_size=35))
    assert (other.optimizer.flat_params - tr.optimizer.flat_params).abs().max().item() < 1e-6
    # a checkpoint with weights only: the optimiser starts afresh around them, and says nothing is unknown
    weights_only = {k: v for k, v in np.load(path).items() if k.endswith("_l1:0") or k.endswith("_l2:0")
                    or k.endswith("_l3:0") or k.endswith("_l4:0")}
    np.savez(str(tmp_path / "w.npz"), **weights_only)
    other.load_numpy(str(tmp_path / "w.npz"))
    assert other.optimizer.steps_done() == 0 and float(other.optimizer.m.abs().max()) == 0.0
    assert torch.equal(other.optimizer.ema, other.optimizer.flat_params)
    np.savez(str(tmp_path / "odd.npz"), **weights_only, some_other_variable=np.zeros(3))
    with pytest.warns(UserWarning, match="match no variable"):
        other.load_numpy(str(tmp_path / "odd.npz"))


def test_feeder_uploads_match_the_host_batches():
    """The pinned arena arrives intact on the device, batch after batch, with slots reused."""
    import torch
    from khan_b200 import RawDataset
    from khan_b200.data.feeder import BatchFeeder, PackedDataset
    b = syn.config1(n_mols=50)
    mols = b.molecules()
    ds = RawDataset(mols, list(np.arange(len(mols), dtype=np.float64)))
    want = list(ds.iterate(batch_size=6, shuffle=False))
    feeder = BatchFeeder(PackedDataset.from_raw(ds, np.float32), 6, False, devices=[torch.device("cuda", 0)], depth=2)
    n = 0
    for fed, (mol_Xs, mol_ids, mol_yts, _) in zip(feeder, want):
        fed.wait()
        assert fed.x.is_cuda and fed.types.dtype == torch.int32
        assert np.array_equal(fed.y.cpu().numpy(), mol_Xs[:, 2].astype(np.float32))
        assert np.array_equal(fed.types.cpu().numpy(), mol_Xs[:, 0].astype(np.int32))
        assert np.array_equal(fed.mol_ids.cpu().numpy(), mol_ids)
        assert np.array_equal(fed.ys.cpu().numpy(), np.asarray(mol_yts, np.float32))
        assert np.array_equal(fed.mol_offsets.cpu().numpy(), fed.offsets_host)
        n += 1
    assert n == len(want)


def test_train_schedule_halves_the_rate_and_keeps_the_best_weights(tmp_path):
    """The reference's schedule (trainer_multi_tower.py:832-891) on a toy problem: the learning
    rate is halved and the batch size grows once an epoch budget without improvement is used
    up, best.npz holds the weights of the best test error, and the error does not get worse."""
    import torch
    from khan_b200 import RawDataset, TrainerMultiTower
    b = syn.config1(n_mols=48)
    mols = b.molecules()
    ys = [0.01 * len(m) for m in mols]
    train, test = RawDataset(mols[:36], ys[:36]), RawDataset(mols[36:], ys[36:])
    tr = TrainerMultiTower(None, [torch.device("cuda", 0)], layer_sizes=(128, 128, 64, 1), seed=3)
    before = tr.eval_abs_rmse(test)
    lines = []
    best = tr.train(str(tmp_path), train, test, batch_size=16, max_local_epoch_count=2,
                    max_batch_size=16 + 128 + 1, max_global_epoch_count=6, log=lines.append)
    assert best <= before
    assert (tmp_path / "best.npz").exists()
    assert tr.global_epoch_count >= 2 and any("Decreasing learning rate" in l for l in lines)
    assert tr.learning_rate < 1e-3
    # the weights in best.npz reproduce the best score
    tr2 = TrainerMultiTower(None, [torch.device("cuda", 0)], layer_sizes=(128, 128, 64, 1), seed=9)
    tr2.load_numpy(str(tmp_path / "best.npz"))
    assert abs(tr2.eval_abs_rmse(test) - best) < 1e-3 * max(1.0, best)
    groups = [ys[36:42], ys[42:48]]
    assert tr2.eval_rel_rmse(test, groups) >= 0


def test_energy_forces_evaluator_matches_the_trainer():
    """The allocation-free evaluator (C ABI only) against predict + coordinate_gradients of the
    trainer (autograd path) on the same weights."""
    import ctypes
    import torch
    from khan_b200 import RawDataset, TrainerMultiTower
    from khan_b200.inference import EnergyForces
    from khan_b200.staged import HostBatch, StagedBatch
    b = syn.config1(n_mols=40)
    mols = b.molecules()
    ds = RawDataset(mols)
    tr = TrainerMultiTower(None, [torch.device("cuda", 0)], layer_sizes=(128, 128, 64, 1), seed=5)
    want_e = np.array(tr.predict(ds, batch_size=64))
    want_g = np.concatenate(list(tr.coordinate_gradients(ds, batch_size=64, use_evaluator=False)), axis=0)   # autograd path, (n_atoms, 3)
    fast_g = np.concatenate(list(tr.coordinate_gradients(ds, batch_size=16)), axis=0)                         # evaluator path, several batches
    assert np.abs(fast_g - want_g).max() < 1e-4 * np.abs(want_g).max()
    sb = StagedBatch(b.n_atoms, b.n_mols)
    sb.upload(HostBatch(b, None, pin=False), non_blocking=False, with_upstream=False)
    ev = EnergyForces(tr.model, b.n_atoms, b.n_mols)
    for _ in range(2):                      # twice: the buffers are reused
        ev.run(sb)
    torch.cuda.synchronize()
    got_e = ev.mol_energy[:b.n_mols].cpu().numpy()
    got_g = sb.grads[:, :b.n_atoms].cpu().numpy().T
    assert np.abs(got_e - want_e).max() < 1e-5 * np.abs(want_e).max()
    assert np.abs(got_g - want_g).max() < 1e-4 * np.abs(want_g).max()
    # a second evaluator on another stream, reusing the weights packed above
    other, st = EnergyForces(tr.model, b.n_atoms, b.n_mols), torch.cuda.Stream()
    sb.grads.zero_()
    st.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(st):
        other.run(sb, pack=False)
    torch.cuda.synchronize()
    assert np.array_equal(other.mol_energy[:b.n_mols].cpu().numpy(), got_e)
    assert np.abs(sb.grads[:, :b.n_atoms].cpu().numpy().T - want_g).max() < 1e-4 * np.abs(want_g).max()
    # the pass in two halves -- sort + featurize on one stream, the rest on another -- gives the same bits
    keep_g = sb.grads[:, :b.n_atoms].clone()
    sb.features.fill_(float("nan"))
    sb.grads.zero_()
    main = torch.cuda.current_stream()
    st.wait_stream(main)
    with torch.cuda.stream(st):
        ev.featurize(sb)
    main.wait_stream(st)
    ev.run(sb, pack=False, featurized=True)
    torch.cuda.synchronize()
    assert np.array_equal(ev.mol_energy[:b.n_mols].cpu().numpy(), got_e)
    assert torch.equal(sb.grads[:, :b.n_atoms], keep_g)


def test_fused_train_step_matches_the_autograd_step():
    """FusedTrainStep (C ABI only) against the same step driven by torch autograd: same loss,
    same weight gradients, same coordinate gradients, same weights after the update."""
    import torch
    from khan_b200 import ani_mod
    from khan_b200.model import activations
    from khan_b200.model.nn import MoleculeNN
    from khan_b200.staged import HostBatch, StagedBatch
    from khan_b200.training.fused_step import FusedTrainStep
    from khan_b200.training.optim import FlatNadam
    b = syn.config1(n_mols=60)
    dev = torch.device("cuda", 0)
    y = torch.from_numpy(np.random.default_rng(1).normal(size=b.n_mols).astype(np.float32)).to(dev)
    results = []
    for path in ("fused", "autograd"):
        model = MoleculeNN(activation_fn=activations.gaussian, device=dev, seed=11, init="he")
        params = model.get_parameters()
        opt = FlatNadam(params, lr=1e-3)
        model.accumulate_into_grad = path == "autograd"
        if path == "fused":
            sb = StagedBatch(b.n_atoms, b.n_mols)
            sb.upload(HostBatch(b, None, pin=False), non_blocking=False, with_upstream=False)
            step = FusedTrainStep(model, opt, b.n_atoms, b.n_mols)
            step.forward_backward(sb, y)
            step.coordinate_gradient(sb)
            torch.cuda.synchronize()
            loss = float(step.l2s[:b.n_mols].mean())
            coord = sb.grads[:, :b.n_atoms].clone()
        else:
            xyz = torch.from_numpy(np.stack(b.coords(np.float32))).to(dev)
            x, yy, z = (xyz[k].clone().requires_grad_(True) for k in range(3))
            a = torch.from_numpy(b.atomic_numbers).to(dev)
            mo, mac = torch.from_numpy(b.mol_offsets).to(dev), torch.from_numpy(b.mol_atom_counts).to(dev)
            acs = np.bincount(b.atomic_numbers, minlength=4).astype(np.int32)
            si, gi, _ = ani_mod.ani_sort(a)
            feat = ani_mod.featurize_sorted_autograd(x, yy, z, a, mo, mac, si, acs)
            ids = torch.from_numpy(np.repeat(np.arange(b.n_mols), b.mol_atom_counts)).to(dev)
            pred = torch.zeros(b.n_mols, device=dev).index_add_(0, ids, model.atom_outputs(feat, acs, gi))
            l = ((pred - y) ** 2).mean()
            opt.zero_grad()
            l.backward()
            loss = float(l)
            coord = torch.stack([x.grad, yy.grad, z.grad])
        grads = opt.flat_grads.clone()
        opt.step()
        torch.cuda.synchronize()
        results.append((loss, grads, coord, opt.flat_params.clone()))
    (l0, g0, c0, w0), (l1, g1, c1, w1) = results
    assert abs(l0 - l1) < 1e-5 * abs(l1)
    assert (g0 - g1).abs().max().item() < 1e-4 * g1.abs().max().item()
    assert (c0 - c1).abs().max().item() < 1e-4 * c1.abs().max().item()
    assert (w0 - w1).abs().max().item() < 1e-5


@pytest.mark.parametrize("graphs,allreduce", [(True, False), (False, False), (True, True), (False, True)])
def test_step_pipeline_gives_the_weights_of_the_serial_steps(graphs, allreduce):
    """StepPipeline (next batch's featurize and this batch's coordinate gradient on side streams,
    optionally as CUDA graphs) against FusedTrainStep.step one kernel after another: the same
    weights after seven steps over three batches, the same losses and coordinate gradients.
    ``allreduce`` selects the multi-rank arrangement (the collective is a no-op in one process)."""
    import torch
    from khan_b200.model import activations
    from khan_b200.model.nn import MoleculeNN
    from khan_b200.staged import HostBatch, StagedBatch
    from khan_b200.training.fused_step import FusedTrainStep, StepPipeline
    from khan_b200.training.optim import FlatNadam
    dev = torch.device("cuda", 0)
    pool = syn.batch_pool(3, n_mols=48, seed=21)
    cap = max(b.n_atoms for b in pool)
    ys = [torch.from_numpy(np.random.default_rng(30 + k).normal(size=b.n_mols).astype(np.float32)).to(dev)
          for k, b in enumerate(pool)]
    n_steps = 7
    results = []
    for pipelined in (False, True):
        model = MoleculeNN(activation_fn=activations.gaussian, device=dev, seed=13, init="he")
        opt = FlatNadam(model.get_parameters(), lr=1e-3, clip_norm=5.0)
        staged = []
        for b in pool:
            sb = StagedBatch(cap, 48)
            sb.upload(HostBatch(b, None, pin=False), non_blocking=False, with_upstream=False)
            staged.append(sb)
        step = FusedTrainStep(model, opt, cap, 48)
        losses, coords = [], []
        if pipelined:
            side = torch.cuda.Stream()       # graphs are captured and replayed off the default stream
            with torch.cuda.stream(side):
                pipe = StepPipeline(step, staged, ys, allreduce=allreduce, graphs=graphs)
                pipe.prime()
                for k in range(n_steps):
                    pipe.run(k)
                    losses.append(step.l2s[:48].mean().clone())
                    coords.append(staged[k % 3].grads[:, :pool[k % 3].n_atoms].clone())
            torch.cuda.synchronize()
        else:
            for k in range(n_steps):
                step.step(staged[k % 3], ys[k % 3])
                losses.append(step.l2s[:48].mean().clone())
                coords.append(staged[k % 3].grads[:, :pool[k % 3].n_atoms].clone())
            torch.cuda.synchronize()
        assert opt.steps_done() == n_steps
        results.append((torch.stack(losses).cpu(), coords, opt.flat_params.clone()))
    (l0, c0, w0), (l1, c1, w1) = results
    assert (l0 - l1).abs().max().item() < 1e-4 * l0.abs().max().item()
    for a, b in zip(c0, c1):
        assert (a - b).abs().max().item() < 1e-3 * a.abs().max().item()
    assert (w0 - w1).abs().max().item() < 1e-5


def test_step_pipeline_needs_two_batches():
    import torch
    from khan_b200.model import activations
    from khan_b200.model.nn import MoleculeNN
    from khan_b200.staged import StagedBatch
    from khan_b200.training.fused_step import FusedTrainStep, StepPipeline
    from khan_b200.training.optim import FlatNadam
    dev = torch.device("cuda", 0)
    model = MoleculeNN(activation_fn=activations.gaussian, device=dev, seed=13, init="he")
    opt = FlatNadam(model.get_parameters(), lr=1e-3)
    step = FusedTrainStep(model, opt, 64, 4)
    with pytest.raises(ValueError):
        StepPipeline(step, [StagedBatch(64, 4)], [torch.zeros(4, device=dev)])


def test_molecule_energy_kernel_on_a_ragged_table():
    """ani_molecule_energy_f32 directly: sums through gather_idxs, squared errors, the MSE gradient
    scattered back to the sorted order; empty molecules give 0; a bad gather index is reported."""
    import ctypes
    import torch
    from khan_b200 import _lib, ani_mod
    rng = np.random.default_rng(4)
    counts = np.array([3, 0, 5, 1, 40, 2], np.int32)
    offs = (np.cumsum(counts) - counts).astype(np.int32)
    n = int(counts.sum())
    e_sorted = rng.normal(size=n).astype(np.float32)
    gather = rng.permutation(n).astype(np.int32)
    labels = rng.normal(size=len(counts)).astype(np.float32)
    dev = "cuda:0"
    t = {k: torch.from_numpy(v).to(dev) for k, v in dict(e=e_sorted, g=gather, o=offs, c=counts, y=labels).items()}
    mol = torch.full((len(counts),), 7.0, device=dev)
    l2s = torch.zeros(len(counts), device=dev)
    grad = torch.zeros(n, device=dev)
    st = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    p = lambda x: ctypes.c_void_p(x.data_ptr())
    rc = _lib.lib().ani_molecule_energy_f32(p(t["e"]), p(t["g"]), p(t["o"]), p(t["c"]), len(counts), n, p(t["y"]),
                                            1.0 / len(counts), p(mol), p(l2s), p(grad), st)
    assert rc == 0 and ani_mod.device_status() == 0
    atom_e = e_sorted[gather]
    want = np.array([atom_e[o:o + c].sum(dtype=np.float64) for o, c in zip(offs, counts)])
    assert np.allclose(mol.cpu().numpy(), want, rtol=1e-5, atol=1e-6) and mol[1].item() == 0.0
    assert np.allclose(l2s.cpu().numpy(), (want - labels) ** 2, rtol=1e-4, atol=1e-6)
    want_g = np.zeros(n)
    want_g[gather] = np.repeat(2 * (want - labels) / len(counts), counts)
    assert np.allclose(grad.cpu().numpy(), want_g, rtol=1e-4, atol=1e-6)
    bad = t["g"].clone()
    bad[4] = n + 3
    assert _lib.lib().ani_molecule_energy_f32(p(t["e"]), p(bad), p(t["o"]), p(t["c"]), len(counts), n, None, 0.0,
                                              p(mol), None, None, st) == 0
    assert ani_mod.device_status() == -6


@pytest.mark.parametrize("op_name", ["train_op", "train_op_rmse", "train_op_mse"])
def test_fused_training_path_of_the_trainer_matches_autograd(op_name, monkeypatch):
    """feed_dataset with an energy-training op takes the autograd-free path on one float32 tower;
    forcing the autograd path (by asking for a result the fused path does not produce) must give
    the same weights after a few steps."""
    import torch
    from khan_b200 import RawDataset, TrainerMultiTower
    b = syn.config1(n_mols=70)
    mols = b.molecules()
    ys = list(np.random.default_rng(2).normal(scale=0.1, size=len(mols)))
    ds = RawDataset(mols, ys)
    weights = []
    for extra in (False, True):
        tr = TrainerMultiTower(None, [torch.device("cuda", 0)], layer_sizes=(128, 128, 64, 1), seed=21)
        ops = [getattr(tr, op_name)] + ([tr.tower_preds] if extra else [tr.unordered_l2s])
        out = list(tr.feed_dataset(ds, False, ops, batch_size=32))
        assert len(out) == 3 and all(r[0] is None for r in out)
        if not extra:
            assert tr._fused is not None and out[0][1][0].shape == (32,)
        else:
            assert tr._fused is None
        assert tr.global_step == 3
        weights.append(tr.optimizer.flat_params.clone())
    assert (weights[0] - weights[1]).abs().max().item() < 2e-5


def test_energy_server_answers_with_the_trainers_numbers():
    """The server's evaluator is a trainer: its answer is predict + self energies and the coordinate gradient
    in Hartree/Bohr, checked by finite differences of the served energy."""
    import torch
    from khan_b200 import TrainerMultiTower, energy_server as es
    b = syn.kat_fixture()
    mol = b.molecules()[0]
    tr = TrainerMultiTower(None, ["cuda:0"], torch.float64, layer_sizes=(128, 128, 64, 1), seed=4)
    ans = es.evaluate(tr, mol.tolist())
    assert len(ans["gradient"]) == 3 * len(mol)
    g = np.array(ans["gradient"]).reshape(-1, 3) / es.BOHR          # back to Hartree/Angstrom
    for atom, axis in ((0, 0), (2, 1), (len(mol) - 1, 2)):
        plus, minus = mol.copy(), mol.copy()
        plus[atom, 1 + axis] += 1e-5
        minus[atom, 1 + axis] -= 1e-5
        fd = (es.evaluate(tr, plus.tolist())["energy"] - es.evaluate(tr, minus.tolist())["energy"]) / 2e-5
        assert abs(fd - g[atom, axis]) < 1e-6 * max(1.0, abs(fd))

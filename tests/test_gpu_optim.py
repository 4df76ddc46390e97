"""The fused optimiser step against the formulas of the reference's update written out in
float64 numpy: tf.clip_by_global_norm(5) -> Adam with Nesterov momentum (NadamOptimizer, lr 1e-3,
0.9, 0.999, 1e-8) -> ExponentialMovingAverage(0.9999, global_step)
(khan/training/trainer_multi_tower.py:261-266,421-427)."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _reference_step(w, g, m, v, ema, t, lr=1e-3, b1=0.9, b2=0.999, eps=1e-8, clip=5.0, ema_decay=0.9999):
    norm = np.sqrt(np.sum(g * g))
    g = g * (clip / max(norm, clip))
    m = b1 * m + (1 - b1) * g
    v = b2 * v + (1 - b2) * g * g
    lr_t = lr * np.sqrt(1 - b2 ** t) / (1 - b1 ** t)
    w = w - lr_t * (b1 * m + (1 - b1) * g) / (np.sqrt(v) + eps)
    d = min(ema_decay, (1 + t) / (10 + t))
    ema = ema - (1 - d) * (ema - w)
    return w, m, v, ema


def test_flat_nadam_follows_the_reference_update():
    import torch
    from khan_b200.training.optim import FlatNadam
    rng = np.random.default_rng(0)
    shapes = [(384, 128), (128,), (128, 64), (64, 1), (1,), (7, 3)]     # odd sizes exercise the padding
    params = [torch.tensor(rng.normal(size=s), dtype=torch.float32, device="cuda", requires_grad=True) for s in shapes]
    w = np.concatenate([p.detach().cpu().numpy().reshape(-1).astype(np.float64) for p in params])
    m, v, ema = np.zeros_like(w), np.zeros_like(w), w.copy()
    opt = FlatNadam(params, lr=1e-3)
    for t in range(1, 8):
        scale = 10.0 if t % 2 else 1e-3                      # clipping active on odd steps only
        grads = [rng.normal(size=s) * scale for s in shapes]
        opt.zero_grad()
        for p, g in zip(params, grads):
            p.grad.add_(torch.tensor(g, dtype=torch.float32, device="cuda"))
        if t == 4:
            opt.set_lr(5e-4)
        opt.step()
        g64 = np.concatenate([g.astype(np.float32).astype(np.float64).reshape(-1) for g in grads])
        w, m, v, ema = _reference_step(w, g64, m, v, ema, t, lr=5e-4 if t >= 4 else 1e-3)
        got = np.concatenate([p.detach().cpu().numpy().reshape(-1) for p in params])
        assert np.abs(got - w).max() < 2e-6 * np.abs(w).max(), t
        got_ema = np.concatenate([opt.ema_of(k).cpu().numpy().reshape(-1) for k in range(len(params))])
        assert np.abs(got_ema - ema).max() < 2e-6 * np.abs(ema).max(), t
    assert opt.steps_done() == 7
    # the parameters are still slices of the flat buffer and gradients still land in the flat one
    assert all(p.data_ptr() == opt.flat_params.data_ptr() + 4 * o for p, o in zip(params, opt.offsets))
    (params[0].sum() * 2.0).backward()
    assert float(opt.flat_grads[:5].sum()) != 0.0


def test_step_inside_a_cuda_graph_sees_later_learning_rates():
    import torch
    from khan_b200.training.optim import FlatNadam
    p = torch.ones(1000, device="cuda", requires_grad=True)
    opt = FlatNadam([p], lr=1e-2, clip_norm=0.0)
    opt.flat_grads.fill_(1.0)
    opt.step()                     # warm-up outside the graph
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        opt.step()
    before = p.detach().clone()
    g.replay()
    d1 = float((before - p.detach()).mean())
    opt.set_lr(1e-3)
    before = p.detach().clone()
    g.replay()
    d2 = float((before - p.detach()).mean())
    assert 0.08 < d2 / d1 < 0.12       # ten times smaller step after the rate change
    assert opt.steps_done() == 3       # the warm-up and two replays; the capture itself runs nothing


def test_clip_rows_is_clip_by_norm_over_axis_one():
    """FlatNadam.clip_rows against tf.clip_by_norm(w, 3.0, axes=1) written out in torch
    (khan/training/trainer_multi_tower.py:432-436); biases and vectors in the buffer are left alone."""
    import torch
    from khan_b200.training.optim import FlatNadam
    gen = torch.Generator(device="cuda").manual_seed(3)
    shapes = [(384, 128), (128,), (128, 64), (64,), (64, 1), (1,)]
    params = [(torch.randn(s, device="cuda", generator=gen) * (0.5 if k % 2 == 0 else 5.0)).requires_grad_(True)
              for k, s in enumerate(shapes)]
    want = [p.detach().clone() for p in params]
    for k in (0, 2, 4):
        norms = want[k].norm(dim=1, keepdim=True).clamp_min(1e-30)
        want[k] = want[k] * torch.clamp(3.0 / norms, max=1.0)
    opt = FlatNadam(params)
    opt.clip_rows([0, 2, 4], 3.0)
    opt.clip_rows([0, 2, 4], 3.0)      # idempotent, and the row table is reused
    for p, w in zip(params, want):
        assert (p.detach() - w).abs().max().item() <= 1e-6 * max(1.0, w.abs().max().item())
    assert float(params[0].detach().norm(dim=1).max()) <= 3.0 + 1e-5
    assert float(params[0].detach().norm(dim=1).max()) > 2.9          # the constraint was active


@pytest.mark.parametrize("kind", [1, 2])
def test_scale_by_loss_turns_the_mse_gradient_into_the_rmse_and_exp_rmse_gradients(kind):
    """d rmse = d mse / (2 rmse), d exp(rmse) = exp(rmse) d mse / (2 rmse) with rmse = sqrt(mean(l2)):
    the loss khan minimises (khan/training/trainer_multi_tower.py:390-396), against float64 numpy."""
    import ctypes
    import torch
    from khan_b200 import _lib
    rng = np.random.default_rng(kind)
    for n, n_mols in ((296_464, 1024), (1000, 1), (37, 2049)):
        g = rng.normal(size=n).astype(np.float32)
        l2 = (rng.normal(size=n_mols) ** 2).astype(np.float32) * 0.01
        rmse = np.sqrt(l2.astype(np.float64).mean())
        factor = (np.exp(rmse) if kind == 2 else 1.0) / (2.0 * rmse)
        dg, dl2 = torch.tensor(g, device="cuda"), torch.tensor(l2, device="cuda")
        out_rmse = torch.zeros((), device="cuda")
        stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
        assert _lib.lib().ani_scale_by_loss_f32(dg.data_ptr(), n, dl2.data_ptr(), n_mols, kind, out_rmse.data_ptr(),
                                                stream) == 0
        np.testing.assert_allclose(float(out_rmse), rmse, rtol=2e-6)
        np.testing.assert_allclose(dg.cpu().numpy(), g.astype(np.float64) * factor, rtol=5e-6, atol=0)
    assert _lib.lib().ani_scale_by_loss_f32(dg.data_ptr(), n, dl2.data_ptr(), n_mols, 3, None, stream) == -2
    assert _lib.lib().ani_scale_by_loss_f32(dg.data_ptr(), n, dl2.data_ptr(), 0, 1, None, stream) == -2

"""The fused tensor-core atomic-network kernel against a plain float64 torch evaluation of the
same four 384-128-128-64-1 stacks.  Tolerances (relative to the largest energy): 2e-5 with the
split-precision products (float32-grade), 5e-3 with plain tf32."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _reference(model, feats64, acs):
    import torch
    starts = np.concatenate([[0], np.cumsum(acs)])
    out = []
    for t, ann in enumerate(model.anns):
        a = feats64[int(starts[t]):int(starts[t + 1])]
        last = len(ann.Ws) - 1
        for k, (w, b) in enumerate(zip(ann.Ws, ann.bs)):
            a = a @ w.detach().double() + b.detach().double()
            if k != last:
                a = model.activation_fn(a)
        out.append(a.reshape(-1))
    return torch.cat(out)


@pytest.mark.parametrize("act", ["celu", "gaussian", "normal", "softplus"])
@pytest.mark.parametrize("split,tol", [(True, 2e-5), (False, 5e-3)])
def test_fused_forward_matches_dense_float64(act, split, tol):
    import torch
    from khan_b200.model import activations, nn
    torch.manual_seed(0)
    acs = np.array([300, 129, 0, 7])          # a full tile + remainder, an exact edge, empty, tiny
    n = int(acs.sum())
    model = nn.MoleculeNN(activation_fn=activations.get_fn_by_name(act), seed=1, split_precision=split)
    for ann in model.anns:                     # non-zero biases so that they are exercised
        for b in ann.bs:
            b.data.normal_(0.0, 0.1)
    feats = (torch.rand((n, 384), device="cuda") * 2.0).float()
    got = model.atom_energies_sorted(feats, acs)
    from khan_b200 import ani_mod
    ani_mod.check_device_status("mlp")
    ref = _reference(model, feats.double(), acs)
    scale = ref.abs().max().item()
    assert (got.double() - ref).abs().max().item() < tol * scale


def _interleaved(model):
    out = []
    for ann in model.anns:
        for w, b in zip(ann.Ws, ann.bs):
            out.extend([w, b])
    return out


def _dense64(model, feats64, acs, params64):
    import torch
    starts = np.concatenate([[0], np.cumsum(acs)])
    out = []
    for t in range(4):
        a = feats64[int(starts[t]):int(starts[t + 1])]
        w1, b1, w2, b2, w3, b3, w4, b4 = params64[8 * t: 8 * t + 8]
        for w, b in ((w1, b1), (w2, b2), (w3, b3)):
            a = model.activation_fn(a @ w + b)
        out.append((a @ w4 + b4).reshape(-1))
    return torch.cat(out)


@pytest.mark.parametrize("act", ["celu", "gaussian", "normal", "softplus"])
def test_backward_kernel_matches_dense_float64(act):
    """Feature gradient (from the backward kernel) and all weight gradients against float64
    autograd of the same networks; tolerance 5e-5 of the largest entry of each gradient."""
    import torch
    from khan_b200.model import activations, nn
    acs = np.array([300, 129, 0, 7])
    n = int(acs.sum())
    model = nn.MoleculeNN(activation_fn=activations.get_fn_by_name(act), seed=3, init="he")
    for ann in model.anns:
        for b in ann.bs:
            b.data.normal_(0.0, 0.1)
    gen = torch.Generator(device="cuda").manual_seed(5)
    feats = torch.rand((n, 384), device="cuda", generator=gen).requires_grad_(True)
    w = torch.randn(n, device="cuda", generator=gen)
    (model.atom_energies_sorted(feats, acs) * w).sum().backward()
    fused = [feats.grad.clone()] + [None if p.grad is None else p.grad.clone() for p in _interleaved(model)]
    feats64 = feats.detach().double().requires_grad_(True)
    params64 = [p.detach().double().requires_grad_(True) for p in _interleaved(model)]
    (_dense64(model, feats64, acs, params64) * w.double()).sum().backward()
    plain = [feats64.grad] + [p.grad for p in params64]
    from khan_b200 import ani_mod
    ani_mod.check_device_status("mlp backward")
    for k, (a, b) in enumerate(zip(fused, plain)):
        if b is None or b.abs().max().item() == 0.0:      # the empty element
            assert a is None or a.abs().max().item() == 0.0
            continue
        assert (a.double() - b).abs().max().item() < 5e-5 * b.abs().max().item(), k


def test_double_backward_keeps_the_second_derivative():
    """Force-training path: the gradient of a function of dE/dfeatures with respect to the
    weights (create_graph=True) against float64 autograd."""
    import torch
    from khan_b200.model import activations, nn
    acs = np.array([70, 20, 9, 5])
    n = int(acs.sum())
    model = nn.MoleculeNN(activation_fn=activations.celu, seed=4, init="he")
    gen = torch.Generator(device="cuda").manual_seed(6)
    feats = torch.rand((n, 384), device="cuda", generator=gen).requires_grad_(True)
    e = model.atom_energies_sorted(feats, acs)
    (gf,) = torch.autograd.grad(e.sum(), feats, create_graph=True)
    (gf ** 2).sum().backward()
    fused = [None if p.grad is None else p.grad.clone() for p in _interleaved(model)]
    feats64 = feats.detach().double().requires_grad_(True)
    params64 = [p.detach().double().requires_grad_(True) for p in _interleaved(model)]
    (gf64,) = torch.autograd.grad(_dense64(model, feats64, acs, params64).sum(), feats64, create_graph=True)
    (gf64 ** 2).sum().backward()
    for a, p in zip(fused, params64):
        b = p.grad
        if b is None or b.abs().max().item() == 0.0:     # the output bias does not reach dE/dfeatures
            assert a is None or a.abs().max().item() == 0.0
            continue
        assert (a.double() - b).abs().max().item() < 1e-3 * b.abs().max().item()


def test_weight_gradients_accumulate_into_existing_buffers():
    """Second backward pass: the parameters already have gradient buffers, so the kernel adds
    into them directly; the result must be exactly twice the first pass up to rounding."""
    import torch
    from khan_b200.model import activations, nn
    acs = np.array([140, 0, 33, 600])
    n = int(acs.sum())
    model = nn.MoleculeNN(activation_fn=activations.celu, seed=8, init="he")
    model.accumulate_into_grad = True
    gen = torch.Generator(device="cuda").manual_seed(9)
    feats = torch.rand((n, 384), device="cuda", generator=gen)
    w = torch.randn(n, device="cuda", generator=gen)
    (model.atom_energies_sorted(feats, acs) * w).sum().backward()
    params = [p for p in _interleaved(model) if p.grad is not None]
    first = [p.grad.clone() for p in params]
    ptrs = [p.grad.data_ptr() for p in params]
    (model.atom_energies_sorted(feats, acs) * w).sum().backward()
    for p, f, ptr in zip(params, first, ptrs):
        assert p.grad.data_ptr() == ptr
        assert (p.grad - 2 * f).abs().max().item() <= 1e-5 * f.abs().max().item()
    # without the flag torch.autograd.grad still gets its gradients returned
    model.accumulate_into_grad = False
    got = torch.autograd.grad((model.atom_energies_sorted(feats, acs) * w).sum(), params)
    for g, f in zip(got, first):
        assert (g - f).abs().max().item() <= 1e-5 * f.abs().max().item()


def test_packed_and_unpacked_weight_paths_agree(monkeypatch):
    """The kernels fetch pre-packed weight chunks with bulk copies by default; without a packed
    copy they stage the weights themselves.  Same operands, same MMAs: identical energies, and
    gradients equal up to the order of the floating-point reductions."""
    import torch
    from khan_b200.model import activations, nn
    acs = np.array([300, 129, 0, 7])
    n = int(acs.sum())
    gen = torch.Generator(device="cuda").manual_seed(12)
    base = torch.rand((n, 384), device="cuda", generator=gen)
    w = torch.randn(n, device="cuda", generator=gen)
    results = []
    for packed in (True, False):
        model = nn.MoleculeNN(activation_fn=activations.gaussian, seed=13, init="he")
        if not packed:
            monkeypatch.setattr(nn.MoleculeNN, "pack_weights", lambda self, stream=None: None)
        feats = base.clone().requires_grad_(True)
        e = model.atom_energies_sorted(feats, acs)
        (e * w).sum().backward()
        results.append((e.detach().clone(), feats.grad.clone(),
                        [p.grad.clone() for p in _interleaved(model) if p.grad is not None]))
    (e0, f0, g0), (e1, f1, g1) = results
    assert torch.equal(e0, e1)
    assert torch.equal(f0, f1)
    for a, b in zip(g0, g1):
        assert (a - b).abs().max().item() <= 1e-5 * b.abs().max().item()

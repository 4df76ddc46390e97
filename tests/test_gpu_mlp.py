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


def test_backward_matches_dense_autograd():
    import torch
    from khan_b200.model import activations, nn
    acs = np.array([200, 90, 40, 33])
    n = int(acs.sum())
    model = nn.MoleculeNN(activation_fn=activations.gaussian, seed=3, init="he")
    feats = torch.rand((n, 384), device="cuda").requires_grad_(True)
    w = torch.randn(n, device="cuda")
    (model.atom_energies_sorted(feats, acs) * w).sum().backward()
    fused = [feats.grad.clone()] + [p.grad.clone() for p in model.get_parameters()]
    feats.grad = None
    for p in model.get_parameters():
        p.grad = None
    starts = np.concatenate([[0], np.cumsum(acs)])
    dense = torch.cat([ann.atom_energies(feats[int(starts[t]):int(starts[t + 1])])
                       for t, ann in enumerate(model.anns)])
    (dense * w).sum().backward()
    plain = [feats.grad] + [p.grad for p in model.get_parameters()]
    for a, b in zip(fused, plain):
        scale = b.abs().max().item() + 1e-30
        assert (a - b).abs().max().item() < 2e-4 * scale

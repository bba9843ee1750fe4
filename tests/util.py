"""Test helpers: wrap torch tensors as framework tensors and compare against torch autograd."""
import torch

import dummygrad_b200 as dg


def T(t: torch.Tensor, device, requires_grad=True, dtype=torch.float32):
    """Framework tensor holding a copy of ``t`` on ``device``."""
    d = t.detach().to(device=device, dtype=torch.float32).clone()
    if dtype != torch.float32:
        d = dg.ops.kernels.cast(d.contiguous(), dtype)
    return dg.Tensor.from_torch(d, requires_grad)


def close(a, b, tol=1e-5, what=""):
    a = a.detach().float().cpu()
    b = b.detach().float().cpu()
    assert a.shape == b.shape, f"{what}: shape {tuple(a.shape)} vs {tuple(b.shape)}"
    err = (a - b).abs().max().item() if a.numel() else 0.0
    scale = max(1.0, b.abs().max().item() if b.numel() else 1.0)
    assert err <= tol * scale, f"{what}: max abs err {err:.3e} (scale {scale:.3e}, tol {tol})"


def check(fn_dg, fn_torch, inputs, device, tol=1e-5, grad_mask=None, dtype=torch.float32):
    """Run ``fn_dg`` on framework tensors and ``fn_torch`` on fp32 torch tensors built from the same
    values; compare outputs and the gradients of sum(out * w) for a fixed random w."""
    torch.manual_seed(1234)
    tin = [x.detach().clone().float().requires_grad_(True) for x in inputs]
    din = [T(x, device, True, dtype) for x in inputs]
    if dtype != torch.float32:
        # compare against the reference evaluated on the rounded inputs
        tin = [d.data.float().cpu().clone().requires_grad_(True) for d in din]
    out_t = fn_torch(*tin)
    out_d = fn_dg(*din)
    close(out_d.data, out_t, tol, "forward")
    w = torch.randn_like(out_t)
    (out_t * w).sum().backward()
    wd = T(w, device, False, dtype)
    loss = dg.simple_sum(dg.mul(out_d, wd)) if out_d.shape == wd.shape else None
    loss.backward()
    for i, (a, b) in enumerate(zip(din, tin)):
        if grad_mask is not None and not grad_mask[i]:
            continue
        assert a.grad is not None, f"input {i}: no gradient"
        close(a.grad.data, b.grad, tol * 4, f"grad of input {i}")

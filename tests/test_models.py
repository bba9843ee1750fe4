"""T3: modules and models. Fused modules against the reference-style op chains, and both against
plain PyTorch; the toy decoder must actually train."""
import math

import pytest
import torch

import dummygrad_b200 as dg
from dummygrad_b200.models import layers
from util import T, close


def _copy_params(dst, src):
    for a, b in zip(dst.parameters(), src.parameters()):
        dg.ops.kernels.strided_copy(a.data, b.data)


def _grads_close(m1, m2, tol):
    for i, (a, b) in enumerate(zip(m1.parameters(), m2.parameters())):
        assert (a.grad is None) == (b.grad is None), f"param {i}"
        if a.grad is not None:
            close(a.grad.data, b.grad.data, tol, f"grad of param {i}")


@pytest.mark.parametrize("cls,args,xshape", [
    (dg.Linear, (12, 20), (3, 5, 12)),
    (dg.LayerNorm, (16,), (4, 6, 16)),
    (dg.FeedForward, (16,), (2, 5, 16)),
    (dg.SelfAttention, (16, True), (2, 6, 16)),
    (dg.MultiHeadAttention, (16, 4, True), (2, 6, 16)),
    (dg.MultiHeadAttention, (16, 2, False), (7, 16)),
    (dg.TransformerBlock, (16, 4), (2, 6, 16)),
])
def test_fused_matches_op_chain(device, cls, args, xshape):
    dg.manual_seed(0)
    torch.manual_seed(0)
    fused = cls(*args, device=device, fused=True)
    chain = cls(*args, device=device, fused=False)
    _copy_params(chain, fused)
    x = torch.randn(*xshape)
    xa, xb = T(x, device), T(x, device)
    ya, yb = fused.forward(xa), chain.forward(xb)
    close(ya.data, yb.data, 5e-5, "forward")
    w = T(torch.randn(*ya.shape), device, False)
    dg.simple_sum(dg.mul(ya, w)).backward()
    dg.simple_sum(dg.mul(yb, w)).backward()
    close(xa.grad.data, xb.grad.data, 2e-4, "input grad")
    _grads_close(fused, chain, 2e-4)


def test_layernorm_matches_torch(device):
    torch.manual_seed(1)
    ln = dg.LayerNorm(24, device=device, fused=False)
    x = torch.randn(3, 5, 24, requires_grad=True)
    y = ln.forward(T(x, device))
    close(y.data, torch.nn.functional.layer_norm(x, (24,)), 5e-5)


def test_embedding_matches_one_hot_matmul(device):
    dg.manual_seed(2)
    e1 = dg.Embedding(11, 8, device=device, fused=True)
    e2 = dg.Embedding(11, 8, device=device, fused=False)
    _copy_params(e2, e1)
    idx = T(torch.tensor([1.0, 5.0, 5.0, 10.0, 0.0]), device, False)
    a, b = e1.forward(idx), e2.forward(idx)
    assert a.shape == [5, 8]
    close(a.data, b.data)
    dg.simple_sum(a).backward()
    dg.simple_sum(b).backward()
    close(e1.weight.grad.data, e2.weight.grad.data)


def test_gpt_reference_program_converges(device):
    """The reference's integration test (src/test_transformer.cpp:5-83): GPT(V=10, seq=4, d=16, H=2,
    L=2), one fixed sequence, softmax -> cross_entropy on one-hot targets, Adam 1e-3, 50 steps."""
    dg.manual_seed(3)
    model = dg.GPT(10, 4, 16, 2, 2, device=device)
    opt = dg.Adam(0.001)
    params = model.parameters()
    assert len(params) == 2 + 2 * 16 + 2
    ids = T(torch.tensor([1.0, 3.0, 5.0, 7.0]), device, False)
    pos = T(torch.tensor([0.0, 1.0, 2.0, 3.0]), device, False)
    targets = dg.Tensor([4, 10], False, device=device)
    oh = torch.zeros(4, 10)
    oh[0, 1] = oh[1, 3] = oh[2, 5] = oh[3, 7] = 1
    targets.fill(oh.flatten().tolist())
    first = last = None
    for step in range(50):
        for p in params:
            p.zero_grad()
        logits = model.forward(ids, pos)
        loss = dg.cross_entropy(dg.softmax(logits), targets)
        last = loss.data_at(0)
        first = last if first is None else first
        loss.backward()
        for p in params:
            opt.step(p)
    assert math.isfinite(last) and last < first


def test_toy_decoder_trains_and_matches_unfused(device):
    """Config-2 shape (V256 d64 L2 H4 FFN256 S32 B8, Adam 3e-4): fused and op-chain models stay
    together for several steps and the loss goes down."""
    dg.manual_seed(4)
    torch.manual_seed(4)
    mf = dg.models.build_preset("toy", device=device, fused=True)
    mc = dg.models.build_preset("toy", device=device, fused=False)
    _copy_params(mc, mf)
    of, oc = dg.Adam(3e-4), dg.Adam(3e-4)
    ids = torch.randint(0, 256, (8, 32)).to(device)
    tgt = torch.randint(0, 256, (8 * 32,)).to(device)
    lf, lc = [], []
    for step in range(4):
        for m, o, rec in ((mf, of, lf), (mc, oc, lc)):
            m.zero_grad()
            loss = m.loss(ids, tgt)
            loss.backward()
            for p in m.parameters():
                o.step(p)
            rec.append(loss.item())
    assert lf[-1] < lf[0]
    for a, b in zip(lf, lc):
        assert abs(a - b) < 2e-3 * max(1.0, abs(b)), (lf, lc)
    assert abs(lf[0] - math.log(256)) < 1.0


def test_mlp_config_trains(device):
    """Config 1: 784 -> 128 ReLU -> 10, batch 64, SGD 1e-2, reference loss normalisation."""
    dg.manual_seed(0)
    torch.manual_seed(0)
    m = dg.MLP(device=device)
    x = T(torch.randn(64, 784), device, False)
    y = torch.randint(0, 10, (64,)).to(device)
    losses = []
    for _ in range(20):
        m.zero_grad()
        loss = m.loss(x, y)
        loss.backward()
        for p in m.parameters():
            dg.SGD(p, 1e-2)
        losses.append(loss.item())
    assert losses[-1] < losses[0]


def test_mars_model_step(device):
    dg.manual_seed(5)
    torch.manual_seed(5)
    m = dg.Mars(d_in=12, d_model=16, n_heads=4, max_seq=8, device=device)
    opt = dg.Adam(1e-3)
    x = T(torch.randn(3, 8, 12), device, False)
    y = T(torch.randn(3, 12), device, False)
    losses = []
    for _ in range(5):
        m.zero_grad()
        loss = dg.mse(m.forward(x), y)
        loss.backward()
        dg.optim.clip_grad_value_(m.parameters(), -1.0, 1.0)
        for p in m.parameters():
            opt.step(p)
        losses.append(loss.item())
    assert losses[-1] < losses[0]


def test_bf16_model_step(device):
    """bf16 parameters with fp32 master weights in AdamW."""
    dg.manual_seed(6)
    torch.manual_seed(6)
    m = dg.GPT(64, 16, 32, 2, 2, dtype=torch.bfloat16, device=device)
    opt = dg.AdamW(m.parameters(), lr=1e-3)
    ids = torch.randint(0, 64, (4, 16)).to(device)
    tgt = torch.randint(0, 64, (64,)).to(device)
    losses = []
    for _ in range(6):
        opt.zero_grad()
        loss = m.loss(ids, tgt)
        loss.backward()
        opt.step()
        losses.append(loss.item())
    assert all(math.isfinite(v) for v in losses) and losses[-1] < losses[0], losses


def test_residual_gradient_joins_inside_layernorm_backward(device):
    """x feeds a LayerNorm branch and a residual connection: the engine hands the residual path's
    gradient to LayerNormBackward, which returns the sum (no separate add); values match autograd."""
    import torch.nn.functional as TF
    from dummygrad_b200.ops import functional as F
    torch.manual_seed(0)
    xv, wv = torch.randn(6, 16), torch.randn(16, 16) * 0.3
    gam, bet = 1 + 0.1 * torch.randn(1, 16), 0.1 * torch.randn(1, 16)
    x, W = T(xv, device), T(wv, device)
    g_, b_ = T(gam, device), T(bet, device)
    calls = []
    orig = F.LayerNormBackward.apply

    def spy(self, grads):
        calls.append(self._input_grad_addend is not None)
        return orig(self, grads)

    F.LayerNormBackward.apply = spy
    try:
        y = F.linear(F.layer_norm(x, g_, b_), W, None, residual=x)
        dg.simple_sum(dg.mul(y, y)).backward()
    finally:
        F.LayerNormBackward.apply = orig
    assert calls == [True], "the waiting residual gradient must be offered to the LayerNorm backward node"
    xt, wt = xv.clone().requires_grad_(True), wv.clone().requires_grad_(True)
    gt, bt = gam.clone().requires_grad_(True), bet.clone().requires_grad_(True)
    yt = TF.layer_norm(xt, (16,), gt.reshape(-1), bt.reshape(-1), 1e-5) @ wt + xt
    (yt * yt).sum().backward()
    close(x.grad.data, xt.grad, 1e-4, "dx")
    close(W.grad.data, wt.grad, 1e-4, "dW")
    close(g_.grad.data, gt.grad, 1e-4, "dgamma")

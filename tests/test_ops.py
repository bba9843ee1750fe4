"""T0: every op of the reference API, forward and backward, against a plain PyTorch fp32
statement of the same mathematics (torch autograd supplies the reference gradients)."""
import math

import pytest
import torch

import dummygrad_b200 as dg
from util import T, check, close

R = lambda *s: torch.randn(*s)  # noqa: E731
P = lambda *s: torch.rand(*s) + 0.5  # noqa: E731


def gelu_t(x):
    return 0.5 * x * (1 + torch.tanh(0.7978845608 * (x + 0.044715 * x ** 3)))


BINARY = [
    ("add", dg.add, lambda a, b: a + b, R), ("sub", dg.sub, lambda a, b: a - b, R),
    ("mul", dg.mul, lambda a, b: a * b, R), ("div", dg.div, lambda a, b: a / b, P),
]


@pytest.mark.parametrize("name,fd,ft,gen", BINARY, ids=[b[0] for b in BINARY])
@pytest.mark.parametrize("shape", [(3, 5), (2, 3, 4), (2, 2, 3, 8)])
def test_binary(device, name, fd, ft, gen, shape):
    torch.manual_seed(0)
    check(fd, ft, [gen(*shape), gen(*shape)], device)


def test_binary_shape_mismatch(device):
    with pytest.raises(RuntimeError):
        dg.add(T(R(2, 3), device), T(R(3, 2), device))


UNARY = [
    ("pow3", lambda a: dg.pow(a, 3), lambda a: a ** 3, R), ("pow-2", lambda a: dg.pow(a, -2), lambda a: a ** -2, P),
    ("sqrt", dg.sqrt, torch.sqrt, P), ("log", dg.log, lambda a: torch.log(a + 1e-8), P), ("exp", dg.exp, torch.exp, R),
    ("relu", dg.relu, torch.relu, R), ("tanh", dg.tanh, torch.tanh, R), ("gelu", dg.gelu, gelu_t, R),
    ("add_scalar", lambda a: dg.add_scalar(a, 1.5), lambda a: a + 1.5, R),
    ("sub_scalar", lambda a: dg.sub_scalar(a, 1.5), lambda a: a - 1.5, R),
    ("mul_scalar", lambda a: dg.mul_scalar(a, -2.5), lambda a: a * -2.5, R),
    ("div_scalar", lambda a: dg.div_scalar(a, 4.0), lambda a: a / 4.0, R),
    ("neg", dg.neg, lambda a: -a, R),
    ("rsub_scalar", lambda a: dg.rsub_scalar(2.0, a), lambda a: 2.0 - a, R),
    ("rdiv_scalar", lambda a: dg.rdiv_scalar(2.0, a), lambda a: 2.0 / a, P),
    ("causal_mask", dg.causal_mask, lambda a: a.masked_fill(torch.triu(torch.ones(a.shape[-2:], dtype=torch.bool), 1), -1e9), R),
    ("softmax", dg.softmax, lambda a: torch.softmax(a, -1), R),
]


@pytest.mark.parametrize("name,fd,ft,gen", UNARY, ids=[u[0] for u in UNARY])
@pytest.mark.parametrize("shape", [(4, 7), (2, 3, 5, 6)])
def test_unary(device, name, fd, ft, gen, shape):
    torch.manual_seed(1)
    check(fd, ft, [gen(*shape)], device, tol=2e-5)


def test_simple_sum(device):
    x = R(3, 4, 5)
    check(lambda a: dg.mul_scalar(dg.simple_sum(a), 2.0), lambda a: (a.sum() * 2.0).reshape(1, 1), [x], device)
    assert dg.simple_sum(T(x, device)).shape == [1, 1]


@pytest.mark.parametrize("axis", [0, 1])
def test_broadcast(device, axis):
    x = R(2, 1, 5) if axis == 0 else R(2, 4, 1)
    ft = (lambda a: a.expand(2, 3, 5)) if axis == 0 else (lambda a: a.expand(2, 4, 6))
    check(lambda a: dg.broadcast(a, axis, 3 if axis == 0 else 6), ft, [x], device)
    with pytest.raises(RuntimeError):
        dg.broadcast(T(R(2, 3, 5), device), 0, 2)


CAST = [("add", dg.cast_n_add, lambda x, y: x + y, R), ("sub", dg.cast_n_sub, lambda x, y: x - y, R),
        ("mul", dg.cast_n_mul, lambda x, y: x * y, R), ("div", dg.cast_n_div, lambda x, y: x / y, P)]


@pytest.mark.parametrize("name,fd,ft,gen", CAST, ids=[c[0] for c in CAST])
@pytest.mark.parametrize("yshape", [(1, 6), (4, 1), (4, 6), (1, 1)])
@pytest.mark.parametrize("xshape", [(4, 6), (3, 2, 4, 6)])
def test_cast_n(device, name, fd, ft, gen, yshape, xshape):
    torch.manual_seed(2)
    check(fd, ft, [gen(*xshape), gen(*yshape)], device, tol=3e-5)


def test_cast_n_keepdim_statistic(device):
    """y = keepdim reduction of a batched x broadcasts per batch entry."""
    x = R(3, 4, 6)
    check(lambda a: dg.cast_n_sub(a, dg.mean(a, 1)), lambda a: a - a.mean(-1, keepdim=True), [x], device)
    check(lambda a: dg.cast_n_div(a, dg.add_scalar(dg.var(a, 0), 1.0)), lambda a: a / (a.var(-2, unbiased=False, keepdim=True) + 1.0),
          [x], device, tol=3e-5)


MM = [((5, 7), (7, 3)), ((2, 5, 7), (7, 3)), ((2, 3, 5, 7), (2, 3, 7, 4)), ((2, 1, 2, 2), (1, 2, 2, 2)),
      ((5, 7), (3, 7, 2)), ((4, 1, 3, 5), (2, 5, 6))]


@pytest.mark.parametrize("sa,sb", MM)
def test_matmul(device, sa, sb):
    torch.manual_seed(3)
    check(dg.matmul, torch.matmul, [R(*sa), R(*sb)], device, tol=2e-5)


def test_matmul_reference_case(device):
    """The reference's own check (src/test.cpp:8-70): ones [2,1,2,2] x ones [1,2,2,2]."""
    a = dg.Tensor([2, 1, 2, 2], device=device)
    b = dg.Tensor([1, 2, 2, 2], device=device)
    a.fill(1.0)
    b.fill(1.0)
    out = dg.matmul(a, b)
    assert out.shape == [2, 2, 2, 2]
    dg.simple_sum(out).backward()
    assert all(abs(v - 2.0) < 1e-5 for v in out.data.flatten().tolist())
    assert all(abs(v - 4.0) < 1e-5 for v in a.grad.data.flatten().tolist())
    assert all(abs(v - 4.0) < 1e-5 for v in b.grad.data.flatten().tolist())


def test_matmul_transposed_weight(device):
    """matmul(x, transpose(W)) with non-square W: the tied-head case."""
    torch.manual_seed(4)
    check(lambda x, w: dg.matmul(x, dg.transpose(w, 0, 1)), lambda x, w: x @ w.t(), [R(6, 5), R(9, 5)], device, tol=2e-5)
    check(lambda x, w: dg.matmul(x, dg.transpose(w, 0, 1)), lambda x, w: x @ w.t(), [R(2, 6, 5), R(9, 5)], device, tol=2e-5)


def test_views(device):
    torch.manual_seed(5)
    x = R(2, 3, 4)
    check(lambda a: dg.reshape(dg.transpose(a, 1, 2), [2, 12]), lambda a: a.transpose(1, 2).reshape(2, 12), [x], device)
    check(lambda a: dg.view(a, [6, 4]), lambda a: a.view(6, 4), [x], device)
    check(lambda a: dg.transpose(a, 0, 2), lambda a: a.transpose(0, 2), [x], device)
    with pytest.raises(RuntimeError):
        dg.view(dg.transpose(T(x, device), 0, 1), [24])


def test_strided_inputs_are_right(device):
    """Ops must honour strides (a transposed view is not its untransposed storage)."""
    torch.manual_seed(6)
    a, b = R(4, 6), R(6, 4)
    check(lambda x, y: dg.add(dg.transpose(x), y), lambda x, y: x.t() + y, [a, b], device)
    check(lambda x: dg.softmax(dg.transpose(x)), lambda x: torch.softmax(x.t(), -1), [a], device)
    check(lambda x: dg.var(dg.transpose(x), 1), lambda x: x.t().var(-1, unbiased=False, keepdim=True), [a], device, tol=2e-5)
    check(lambda x, y: dg.concat(dg.transpose(x), y, 0), lambda x, y: torch.cat([x.t(), y], 0), [a, b], device)


@pytest.mark.parametrize("axis", [0, 1])
def test_concat(device, axis):
    a, b = (R(2, 3, 5), R(2, 4, 5)) if axis == 0 else (R(2, 3, 5), R(2, 3, 2))
    check(lambda x, y: dg.concat(x, y, axis), lambda x, y: torch.cat([x, y], -2 if axis == 0 else -1), [a, b], device)


def test_scale_n_shift(device):
    torch.manual_seed(7)
    check(dg.scale_n_shift, lambda x, g, b: x * g + b, [R(3, 5, 8), R(1, 8), R(1, 8)], device, tol=2e-5)


def test_bool_mask(device):
    x = R(2, 4, 4)
    m = (torch.rand(2, 4, 4) > 0.4).float()
    check(lambda a: dg.bool_mask(a, T(m, a.device, False)), lambda a: torch.where(m == 0, torch.full_like(a, -1e9), a),
          [x], device)


def test_masked_softmax_matches_chain(device):
    torch.manual_seed(8)
    x = R(2, 3, 6, 6)
    fused = lambda a: dg.masked_softmax(a, scale=0.3, causal=True)  # noqa: E731
    chain = lambda a: dg.softmax(dg.causal_mask(dg.mul_scalar(a, 0.3)))  # noqa: E731
    ft = lambda a: torch.softmax((a * 0.3).masked_fill(torch.triu(torch.ones(6, 6, dtype=torch.bool), 1), -1e9), -1)  # noqa: E731
    check(fused, ft, [x], device, tol=2e-5)
    check(chain, ft, [x], device, tol=2e-5)


@pytest.mark.parametrize("axis", [-1, -2, 1, 2])
def test_sum(device, axis):
    x = R(2, 3, 5)
    check(lambda a: dg.sum(a, axis), lambda a: a.sum(axis, keepdim=True), [x], device)
    with pytest.raises(RuntimeError):
        dg.sum(T(x, device), 0)


@pytest.mark.parametrize("axis", [0, 1])
@pytest.mark.parametrize("shape", [(5, 7), (2, 3, 5, 7), (1, 300, 70)])
def test_mean_var_std(device, axis, shape):
    torch.manual_seed(9)
    x = R(*shape)
    d = -2 if axis == 0 else -1
    check(lambda a: dg.mean(a, axis), lambda a: a.mean(d, keepdim=True), [x], device)
    check(lambda a: dg.var(a, axis), lambda a: a.var(d, unbiased=False, keepdim=True), [x], device, tol=2e-5)
    n = x.shape[d]

    def std_ref(a):
        return StdRef.apply(a, d, n)
    check(lambda a: dg.std_dev(a, axis), std_ref, [x], device, tol=2e-5)


class StdRef(torch.autograd.Function):
    """sqrt(biased var) with the reference's gradient (a - mu) / (N (sigma + 1e-8))."""

    @staticmethod
    def forward(ctx, a, d, n):
        mu = a.mean(d, keepdim=True)
        sd = a.var(d, unbiased=False, keepdim=True).sqrt()
        ctx.save_for_backward(a, mu, sd)
        ctx.n = n
        return sd

    @staticmethod
    def backward(ctx, g):
        a, mu, sd = ctx.saved_tensors
        return (a - mu) / (ctx.n * (sd + 1e-8)) * g, None, None


def test_losses(device):
    torch.manual_seed(10)
    p = torch.softmax(R(6, 5), -1)
    t = torch.nn.functional.one_hot(torch.randint(0, 5, (6,)), 5).float()
    check(lambda a: dg.cross_entropy(a, T(t, a.device, False)), lambda a: (-(t * torch.log(a + 1e-8)).sum() / a.numel()).reshape(1, 1),
          [p], device, tol=1e-4)
    y = R(6, 5)
    check(lambda a, b: dg.mse(a, b), lambda a, b: (((a - b) ** 2).sum() / a.numel()).reshape(1, 1), [R(6, 5), y], device)


def test_slice_last_user_node(device):
    x = R(3, 4, 5)
    check(dg.slice_last, lambda a: a[:, -1, :], [x], device)


def test_one_hot_and_embedding(device):
    idx = torch.tensor([1.0, 3.0, 0.0, 3.0])
    oh = dg.one_hot(T(idx, device, False), 5)
    close(oh.data, torch.nn.functional.one_hot(idx.long(), 5).float())
    with pytest.raises(IndexError):
        dg.one_hot(T(torch.tensor([7.0]), device, False), 5)
    w = R(5, 8)
    check(lambda W: dg.embedding(W, T(idx, W.device, False)), lambda W: W[idx.long()], [w], device)
    pw = R(4, 8)
    pidx = torch.tensor([0.0, 1.0, 2.0, 3.0])
    check(lambda W, Pw: dg.embedding(W, T(idx, W.device, False), Pw, T(pidx, W.device, False)),
          lambda W, Pw: W[idx.long()] + Pw[pidx.long()], [w, pw], device)


def test_fused_linear(device):
    torch.manual_seed(11)
    x, W, b, r = R(2, 5, 12), R(12, 20) * 0.3, R(1, 20), R(2, 5, 20)
    check(lambda x, W, b: dg.linear(x, W, b), lambda x, W, b: x @ W + b, [x, W, b], device, tol=3e-5)
    check(lambda x, W, b, r: dg.linear(x, W, b, act="gelu", residual=r), lambda x, W, b, r: gelu_t(x @ W + b) + r,
          [x, W, b, r], device, tol=3e-5)
    check(lambda x, W, b: dg.linear(x, W, b, act="relu"), lambda x, W, b: torch.relu(x @ W + b), [x, W, b], device, tol=3e-5)


def test_fused_mlp(device):
    torch.manual_seed(12)
    x, W1, b1, W2, b2 = R(3, 4, 8), R(8, 32) * 0.3, R(1, 32) * 0.1, R(32, 8) * 0.2, R(1, 8) * 0.1
    check(lambda x, W1, b1, W2, b2: dg.mlp(x, W1, b1, W2, b2, residual=x),
          lambda x, W1, b1, W2, b2: gelu_t(x @ W1 + b1) @ W2 + b2 + x, [x, W1, b1, W2, b2], device, tol=5e-5)


def test_fused_layer_norm(device):
    torch.manual_seed(13)
    for d in (8, 64, 100):
        x, g, b = R(3, 5, d), R(1, d), R(1, d)
        check(lambda x, g, b: dg.layer_norm(x, g, b, 1e-5),
              lambda x, g, b: torch.nn.functional.layer_norm(x, (d,), g.reshape(d), b.reshape(d), 1e-5), [x, g, b], device, tol=5e-5)


def attn_ref(q, k, v, causal):
    s = q @ k.transpose(-1, -2) / math.sqrt(q.shape[-1])
    if causal:
        S = q.shape[-2]
        s = s.masked_fill(torch.triu(torch.ones(S, S, dtype=torch.bool), 1), -1e9)
    return torch.softmax(s, -1) @ v


@pytest.mark.parametrize("causal", [False, True])
def test_fused_attention(device, causal):
    torch.manual_seed(14)
    q, k, v = R(2, 3, 10, 8), R(2, 3, 10, 8), R(2, 3, 10, 8)
    check(lambda q, k, v: dg.attention(q, k, v, causal=causal), lambda q, k, v: attn_ref(q, k, v, causal), [q, k, v], device, tol=5e-5)


def test_softmax_cross_entropy(device):
    torch.manual_seed(15)
    logits = R(7, 11)
    tgt = torch.randint(0, 11, (7,))
    check(lambda a: dg.softmax_cross_entropy(a, tgt.to(a.device)),
          lambda a: torch.nn.functional.cross_entropy(a, tgt).reshape(1, 1), [logits], device, tol=2e-5)
    check(lambda a: dg.softmax_cross_entropy(a, tgt.to(a.device), reduction="reference"),
          lambda a: (torch.nn.functional.cross_entropy(a, tgt) / 11).reshape(1, 1), [logits], device, tol=2e-5)

"""The tensor-core dense maps (forward and both gradients) against float64 matrix products, on the
shapes of the GCN configurations: 128 -> 256 -> 64 at N = 235 868 (third configuration) and
100 -> 256 -> 256 -> 47 on a slice of the fifth, plus ragged sizes.  Tolerance: the reference's
atol = rtol = 1e-4 relative to the magnitude of the result (sums of `in` or N products)."""
import pytest
import torch

from cbm4gnn_b200 import dense

pytestmark = pytest.mark.gpu


def _check(got, want):
    scale = want.abs().max().item()
    err = (got.double() - want).abs().max().item()
    assert err <= 1e-4 * scale + 1e-6, (err, scale)
    # an fp32-accurate product is far better than that: a single bf16 / tf32 pass would show ~1e-3
    assert err <= 2e-6 * scale * max(1.0, want.size(-1) ** 0.5 / 8), (err, scale)


@pytest.mark.parametrize("n,n_in,n_out", [(235_868, 128, 256), (235_868, 256, 64), (50_000, 100, 256), (50_000, 256, 47),
                                          (1000, 12, 20), (129, 4, 4), (17, 33, 5)])
def test_forward_and_gradients(n, n_in, n_out):
    g = torch.Generator(device="cuda").manual_seed(n_in * 1000 + n_out)
    x = torch.randn((n, n_in), device="cuda", generator=g)
    w = torch.randn((n_out, n_in), device="cuda", generator=g) * 0.1
    gy = torch.randn((n, n_out), device="cuda", generator=g)
    _check(dense.dense_forward(x, w), x.double() @ w.double().t())
    _check(dense.dense_grad_input(gy, w), gy.double() @ w.double())
    _check(dense.dense_grad_weight(gy, x), gy.double().t() @ x.double())


def test_autograd_and_strided_operands():
    g = torch.Generator(device="cuda").manual_seed(3)
    big = torch.randn((4096, 200), device="cuda", generator=g)
    x = big[:, 8:136].detach().requires_grad_(True)           # a column window: row stride 200
    w = (torch.randn((64, 128), device="cuda", generator=g) * 0.1).requires_grad_(True)
    y = dense.linear(x, w)
    y.backward(torch.ones_like(y))
    xr, wr = x.detach().double().requires_grad_(True), w.detach().double().requires_grad_(True)
    yr = xr @ wr.t()
    yr.backward(torch.ones_like(yr))
    _check(y.detach(), yr.detach())
    _check(x.grad, xr.grad)
    _check(w.grad, wr.grad)
    out = torch.full((4096, 72), -1.0, device="cuda")
    dense.dense_forward(x.detach(), w.detach(), out=out[:, 4:68])
    _check(out[:, 4:68], yr.detach())
    assert (out[:, :4] == -1).all() and (out[:, 68:] == -1).all()


def test_relu_in_the_epilogue():
    g = torch.Generator(device="cuda").manual_seed(9)
    x = torch.randn((30_000, 128), device="cuda", generator=g).requires_grad_(True)
    w = (torch.randn((256, 128), device="cuda", generator=g) * 0.1).requires_grad_(True)
    h = dense.linear_relu(x, w)
    gy = torch.randn(h.shape, device="cuda", generator=g)
    h.backward(gy)
    xr, wr = x.detach().double().requires_grad_(True), w.detach().double().requires_grad_(True)
    pre = xr @ wr.t()
    # same mask as the fp32 result: pre-activations within rounding of zero may differ in sign
    mask = (h.detach() > 0)
    assert ((mask != (pre.detach() > 0)) & (pre.detach().abs() > 1e-5)).sum().item() == 0
    hr = pre * mask
    hr.backward(gy.double())
    _check(h.detach(), hr.detach())
    _check(x.grad, xr.grad)
    _check(w.grad, wr.grad)
    out = torch.empty((30_000, 47), device="cuda")
    dense.dense_forward(x.detach(), w.detach()[:47], out=out, relu=True)     # ragged width, narrow tiles
    _check(out, (x.detach().double() @ w.detach()[:47].double().t()).clamp_min(0))

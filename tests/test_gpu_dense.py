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


@pytest.mark.parametrize("n,n_in,n_out", [(235_868, 256, 64), (50_000, 256, 256), (1000, 20, 12), (129, 100, 47), (17, 33, 5)])
def test_input_gradient_masked_in_the_epilogue(n, n_in, n_out):
    """`dense_grad_input(gy, w, relu_output=h)` = (gy w) where h is non-zero, 0 elsewhere; the mask
    is exact (whole elements are kept or dropped), the kept values those of the unmasked map."""
    g = torch.Generator(device="cuda").manual_seed(n_in + n_out)
    gy = torch.randn((n, n_out), device="cuda", generator=g)
    w = torch.randn((n_out, n_in), device="cuda", generator=g) * 0.1
    h = torch.randn((n, n_in), device="cuda", generator=g).relu()
    got = dense.dense_grad_input(gy, w, relu_output=h)
    plain = dense.dense_grad_input(gy, w)
    assert torch.equal(got, torch.where(h > 0, plain, torch.zeros_like(plain)))
    _check(got, (gy.double() @ w.double()) * (h > 0))
    # a window of a wider buffer as the mask operand (row stride larger than the width)
    wide = torch.zeros((n, n_in + 8), device="cuda")
    wide[:, 4:4 + n_in] = h
    assert torch.equal(dense.dense_grad_input(gy, w, relu_output=wide[:, 4:4 + n_in]), got)


def test_two_maps_around_a_relu_as_one_step():
    """`relu_linear_linear` against float64 autograd of the same expression: value and all three
    gradients, also when the first operand needs no gradient."""
    g = torch.Generator(device="cuda").manual_seed(11)
    p = torch.randn((30_000, 128), device="cuda", generator=g)
    w1 = torch.randn((256, 128), device="cuda", generator=g) * 0.1
    w2 = torch.randn((64, 256), device="cuda", generator=g) * 0.1
    gu = torch.randn((30_000, 64), device="cuda", generator=g)
    for p_needs_grad in (True, False):
        pa = p.clone().requires_grad_(p_needs_grad)
        a1, a2 = w1.clone().requires_grad_(True), w2.clone().requires_grad_(True)
        u = dense.relu_linear_linear(pa, a1, a2)
        u.backward(gu)
        pr = p.double().requires_grad_(True)
        r1, r2 = w1.double().requires_grad_(True), w2.double().requires_grad_(True)
        h64 = pr @ r1.t()
        # the reference uses the mask the fp32 path saw: elements within rounding of 0 may differ
        h32 = dense.dense_forward(p, w1)
        mask = h32 > 0
        assert ((h64 > 0) != mask).logical_and(h64.abs() > 1e-4).sum().item() == 0
        ur = (h64 * mask) @ r2.t()
        ur.backward(gu.double())
        _check(u.detach(), ur.detach())
        _check(a1.grad, r1.grad)
        _check(a2.grad, r2.grad)
        if p_needs_grad:
            _check(pa.grad, pr.grad)
        else:
            assert pa.grad is None
    # CPU operands take the torch path
    pc, c1, c2 = p[:100].cpu(), w1.cpu(), w2.cpu()
    assert torch.allclose(dense.relu_linear_linear(pc, c1, c2), (pc @ c1.t()).relu() @ c2.t())

"""Block-scaled FP8 training path of the linear layers (ops/fp8_linear.py) on the CPU reference kernels:
forward, input gradient and weight gradient against the fp32 layer, the routing rules of ``linear`` and a small
training run."""
import torch

from jax_gpt_b200.ops.fp8_linear import fp8_eligible, fp8_linear, fp8_training
from jax_gpt_b200.ops.gemm import linear


def _rel(a, b):
    return ((a.float() - b.float()).norm() / (b.float().norm() + 1e-12)).item()


def test_fp8_linear_forward_and_gradients_close_to_fp32():
    torch.manual_seed(0)
    x = torch.randn(2, 128, 256, requires_grad=True)
    w = (torch.randn(256, 384) * 0.05).requires_grad_()
    b = torch.randn(384, requires_grad=True)
    dy = torch.randn(2, 128, 384)
    y0 = linear(x, w, b)
    y0.backward(dy)
    ref = (x.grad.clone(), w.grad.clone(), b.grad.clone())
    x.grad = w.grad = b.grad = None
    with fp8_training():
        y1 = linear(x, w, b)
    y1.backward(dy)                       # the backward keeps the path chosen in the forward
    assert y1.shape == y0.shape and w.grad.shape == w.shape
    # e4m3 has a 3-bit mantissa: a few percent of relative Frobenius error per GEMM
    assert _rel(y1, y0) < 0.05
    assert _rel(x.grad, ref[0]) < 0.06
    assert _rel(w.grad, ref[1]) < 0.06
    assert _rel(b.grad, ref[2]) < 0.01


def test_fp8_path_is_taken_only_inside_the_context_and_for_eligible_shapes():
    torch.manual_seed(1)
    w = torch.randn(256, 128) * 0.05
    x_ok, x_ragged = torch.randn(128, 256), torch.randn(100, 256)
    assert fp8_eligible(x_ok, w) and not fp8_eligible(x_ragged, w)
    assert not fp8_eligible(x_ok, torch.randn(256, 100)) and not fp8_eligible(x_ok, torch.randn(4, 256, 128))
    exact = x_ok @ w
    assert torch.equal(linear(x_ok, w), exact)                      # outside the context: plain path
    with fp8_training():
        assert torch.equal(linear(x_ragged, w), x_ragged @ w)       # ragged token count: plain path
        y = linear(x_ok, w)
        with fp8_training(False):
            assert torch.equal(linear(x_ok, w), exact)              # nested switch-off (the LM heads use it)
    assert not torch.equal(y, exact) and _rel(y, exact) < 0.05
    assert torch.equal(linear(x_ok, w), exact)                      # state restored
    assert _rel(fp8_linear(x_ok, w), exact) < 0.05


def test_small_mlp_trains_in_fp8_like_in_fp32():
    def run(fp8):
        torch.manual_seed(2)
        w1 = (torch.randn(128, 256) * 0.1).requires_grad_()
        w2 = (torch.randn(256, 128) * 0.1).requires_grad_()
        x = torch.randn(256, 128)
        target = torch.tanh(x @ (torch.randn(128, 128) * 0.2))
        losses = []
        for _ in range(30):
            with fp8_training(fp8):
                out = linear(torch.nn.functional.gelu(linear(x, w1)), w2)
            loss = ((out - target) ** 2).mean()
            loss.backward()
            with torch.no_grad():
                for p in (w1, w2):
                    p -= 0.5 * p.grad
                    p.grad = None
            losses.append(float(loss))
        return losses
    ref, got = run(False), run(True)
    assert got[-1] < 0.5 * got[0]
    assert abs(got[-1] - ref[-1]) < 0.15 * ref[-1] + 1e-3, (ref[-1], got[-1])


def test_fp8_quant_mx_reference_layouts():
    """Reference side of the one-pass quantiser: the transposed form equals quantising the transposed matrix, the
    scales are powers of two, and the packed exponent bytes sit where the tensor-core GEMM reads them
    (byte (r % 32) * 16 + ((r % 128) // 32) * 4 + j of the chunk of row block r // 128 and 128-wide K block)."""
    from jax_gpt_b200.ops.fp8 import fp8_gemm_ref, fp8_quant_mx
    torch.manual_seed(3)
    x = (torch.randn(256, 384) * torch.logspace(-1, 1, 384)[None, :]).to(torch.bfloat16)
    for block in (False, True):
        q, sf, sc = fp8_quant_mx(x, False, block)
        qt, sft, sct = fp8_quant_mx(x, True, block)
        q2, sf2, sc2 = fp8_quant_mx(x.t().contiguous(), False, block)
        assert torch.equal(qt.view(torch.uint8), q2.view(torch.uint8)) and torch.equal(sft, sf2) and torch.equal(sct, sc2)
        assert torch.equal(torch.exp2(torch.log2(sc).round()), sc)                     # powers of two
        assert sf.shape == (2, 3, 512) and sft.shape == (3, 2, 512) and sf.dtype == torch.uint8
        for r, kb in ((0, 0), (37, 1), (130, 2), (255, 0)):
            scale = sc[r // 128, kb] if block else sc[r, kb]
            byte = int(torch.log2(scale).round()) + 127
            off = (r % 32) * 16 + ((r % 128) // 32) * 4
            assert sf[r // 128, kb, off:off + 4].tolist() == [byte] * 4
    # de-quantised product stays close to the bf16 product
    a_q, _, a_s = fp8_quant_mx(x, False, False)
    w = (torch.randn(128, 384) * 0.1).to(torch.bfloat16)
    b_q, _, b_s = fp8_quant_mx(w, False, True)
    ref = x.float() @ w.float().t()
    got = fp8_gemm_ref(a_q, a_s, b_q, b_s)
    assert ((got - ref).norm() / ref.norm()).item() < 0.06

"""tcgen05 GEMM vs an fp32 torch reference: every operand layout, epilogue and odd shapes."""
import pytest
import torch

from tnn_b200.ops import _lib
from tnn_b200.ops.gemm import gemm, gelu_tanh, gelu_tanh_grad

pytestmark = pytest.mark.gpu


def _rand(*shape):
    return (torch.randn(*shape, device="cuda") * 0.5).to(torch.bfloat16)


def _close(got, ref, tol=2e-2):
    """Largest error against the largest value, and every element on its own: bf16 keeps 8 bits, so an element may
    be off by 2 % of itself plus 0.2 % of the largest value (fp32 accumulation, one rounding of the result) - an
    element that was dropped or zeroed fails even when it is small."""
    got, ref = got.float(), ref.float()
    err = (got - ref).abs().max().item()
    scale = ref.abs().max().item() + 1e-6
    assert err / scale < tol, f"rel err {err / scale:.4g}"
    bad = (got - ref).abs() > (2e-2 * ref.abs() + 2e-3 * scale)
    assert not bool(bad.any()), f"{int(bad.sum())} of {bad.numel()} elements off; worst {float(((got - ref).abs() / (ref.abs() + 2e-3 * scale)).max()):.3g}"


@pytest.mark.parametrize("M,N,K", [(128, 128, 64), (256, 256, 128), (384, 512, 320), (200, 136, 72),
                                   (1000, 264, 200), (64, 48, 40), (1024, 768, 768)])
@pytest.mark.parametrize("a_t,b_t", [(False, False), (False, True), (True, False), (True, True)])
def test_layouts(M, N, K, a_t, b_t):
    torch.manual_seed(0)
    a = _rand(K, M) if a_t else _rand(M, K)
    b = _rand(K, N) if b_t else _rand(N, K)
    out = gemm(a, b, a_t=a_t, b_t=b_t)
    _lib.check_status()
    ref = (a.t() if a_t else a).float() @ (b if b_t else b.t()).float()
    _close(out, ref)


@pytest.mark.parametrize("M,N,K", [(8192, 768, 256), (4096, 704, 192), (2048, 768, 128), (1024, 1000, 64)])
@pytest.mark.parametrize("a_t,b_t", [(False, False), (False, True), (True, True)])
def test_pair_kernel_tile_widths(M, N, K, a_t, b_t):
    """CTA-pair kernel: shapes where the wave heuristic picks 384-wide single-accumulator tiles (N = 768 / 704 with
    many rows) and shapes that stay on 256-wide ones, plus the forced 256-wide form, with bias + residual fused."""
    torch.manual_seed(2)
    a = _rand(K, M) if a_t else _rand(M, K)
    b = _rand(K, N) if b_t else _rand(N, K)
    bias, res = _rand(N), _rand(M, N)
    ref = (a.t() if a_t else a).float() @ (b if b_t else b.t()).float() + bias.float() + res.float()
    _close(gemm(a, b, a_t=a_t, b_t=b_t, bias=bias, residual=res), ref)
    _close(gemm(a, b, a_t=a_t, b_t=b_t, bias=bias, residual=res, force_bn=512), ref)
    _lib.check_status()


@pytest.mark.parametrize("bn", [128, 256])
def test_tile_variants(bn):
    a, b = _rand(512, 256), _rand(512, 256)
    out = gemm(a, b, force_bn=bn)
    _lib.check_status()
    _close(out, a.float() @ b.float().t())


def test_epilogues():
    torch.manual_seed(1)
    M, N, K = 300, 200, 136
    a, b, bias, res = _rand(M, K), _rand(N, K), _rand(N), _rand(M, N)
    base = a.float() @ b.float().t()
    _close(gemm(a, b, bias=bias), base + bias.float())
    z = torch.empty(M, N, dtype=torch.bfloat16, device="cuda")
    g = gemm(a, b, bias=bias, gelu=True, save_preact=z)
    _close(z, base + bias.float())
    _close(g, gelu_tanh(base + bias.float()))
    _close(gemm(a, b, dgelu_of=z), base * gelu_tanh_grad(z.float()))
    _close(gemm(a, b, relu=True), torch.relu(base))
    _close(gemm(a, b, bias=bias, residual=res), base + bias.float() + res.float())
    o32 = gemm(a, b, out_dtype=torch.float32)
    _close(o32, base, tol=1e-2)
    acc = res.clone()
    gemm(a, b, out=acc, accumulate=True)
    _close(acc, base + res.float())
    _lib.check_status()


@pytest.mark.parametrize("split_k", [0, 1, 3, 8])
def test_wgrad_atomic_split_k(split_k):
    torch.manual_seed(2)
    rows, n_out, n_in = 2048, 192, 320
    dy, x = _rand(rows, n_out), _rand(rows, n_in)
    dw = torch.ones(n_out, n_in, dtype=torch.float32, device="cuda")
    gemm(dy, x, a_t=True, b_t=True, out=dw, atomic=True, split_k=split_k)
    _lib.check_status()
    _close(dw, dy.float().t() @ x.float() + 1.0, tol=1e-2)


def test_padded_leading_dims_and_vocab_tail():
    torch.manual_seed(3)
    M, K, V, ldc = 256, 128, 1001, 1024
    h, w = _rand(M, K), _rand(V, K)
    buf = torch.zeros(M, ldc, dtype=torch.bfloat16, device="cuda")
    logits = buf[:, :V]
    gemm(h, w, out=logits)
    _close(logits, h.float() @ w.float().t())
    assert buf[:, V:].abs().max().item() == 0
    # dgrad over a K dimension that is not a multiple of the k-block and lives in a padded buffer
    dh = gemm(logits, w, b_t=True)
    _close(dh, logits.float() @ w.float())
    _lib.check_status()

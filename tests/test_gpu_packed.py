"""Packed FP16-piece operands (prad_packed): packing a matrix by rows, by columns and both at once,
with an activation's Forward or Backward evaluated on the fly, and products of packed operands --
every result against the CPU oracle's FP32 loops at the float tolerance."""
import numpy as np
import pytest

import oracle as O
from parallelreverseautodiff_b200 import _lib
from parallelreverseautodiff_b200 import engine as E
from util import assert_close, rng

pytestmark = pytest.mark.gpu
f = np.float32


def _absprod(a, b):
    return np.abs(a).astype(np.float64) @ np.abs(b).astype(np.float64)


@pytest.fixture(params=["0", "2"], ids=["one CTA per tile", "CTA pairs"])
def tile_engine(engine, request):
    """The engine with products of packed operands on one CTA per 128 x 256 tile, or on pairs of CTAs
    (tcgen05 cta_group::2) that share a 256 x 256 tile ("2": also for k below 1024, where the default
    would take single CTAs)."""
    engine.set_option("tc_pair", request.param)
    yield engine
    engine.set_option("tc_pair", "1")          # the default


@pytest.mark.parametrize("shape", [(257, 640, 300), (1024, 2048, 768), (2100, 4096, 520)])
def test_products_on_cta_pairs_match_single_ctas(engine, shape):
    """Several tiles per pair, ragged last tile rows and columns, split-K: the pair kernel adds the same block
    sums in the same order as the one-CTA kernel, so the results are bit-identical."""
    m, k, n = shape
    r = rng(m + n)
    X = r.standard_normal((m, k)).astype(f)
    Y = (r.standard_normal((k, n)) * 0.1).astype(f)
    PX = engine.packed(m, k, E.PACK_ROWS).pack(engine.upload(X))
    PY = engine.packed(k, n, E.PACK_COLS, 0, PX.blocks()[0]).pack(engine.upload(Y))
    outs = []
    for mode in ("0", "2"):
        engine.set_option("tc_pair", mode)
        out = engine.zeros((m, n), f)
        engine.gemm_packed(PX, E.PACK_ROWS, PY, E.PACK_COLS, out)
        outs.append(out.numpy())
    assert_close(outs[1], O.matmul_forward(X, Y), _absprod(X, Y), f"pair product {shape}")
    np.testing.assert_array_equal(outs[0], outs[1])
    # asking L2 for the row operand ahead of its loads changes nothing in the result (an option of the one-CTA kernel)
    engine.set_option("tc_pair", "0")
    engine.set_option("tc_prefetch", "16")
    out = engine.zeros((m, n), f)
    engine.gemm_packed(PX, E.PACK_ROWS, PY, E.PACK_COLS, out)
    engine.set_option("tc_prefetch", "0")
    engine.set_option("tc_pair", "1")          # the default
    np.testing.assert_array_equal(outs[0], out.numpy())


@pytest.mark.parametrize("blocks", [(0, 0), (128, 128), (256, 128), (128, 256), (256, 256)])
@pytest.mark.parametrize("shape", [(300, 200, 130), (512, 384, 256), (77, 1000, 33), (1, 40, 5), (260, 129, 257),
                                   (256, 96, 288)])
def test_products_of_packed_operands(tile_engine, shape, blocks):
    """C = X Y for X (m x k), Y (k x n) through every pairing of forms: X by rows, Y by columns; and the two
    backward shapes dX = dC Y^T (dC by rows, Y by rows), dY = X^T dC (X by columns, dC by columns)."""
    engine = tile_engine
    m, k, n = shape
    br, bc = blocks
    r = rng(m + k + n)
    X = r.standard_normal((m, k)).astype(f)
    Y = (r.standard_normal((k, n)) * 0.3).astype(f)
    dC = (r.standard_normal((m, n)) * 1e-4).astype(f)        # gradients are small numbers
    both = E.PACK_ROWS | E.PACK_COLS
    # block lengths of the forms that meet in one product must agree
    PX = engine.packed(m, k, both, br, bc).pack(engine.upload(X))
    PC = engine.packed(m, n, both, br, bc).pack(engine.upload(dC))
    PY = engine.packed(k, n, both, PC.blocks()[0], PX.blocks()[0]).pack(engine.upload(Y))
    bx, by, bcc = PX.blocks(), PY.blocks(), PC.blocks()
    assert bx[0] == by[1] and bcc[0] == by[0] and bx[1] == bcc[1]
    out = engine.empty((m, n), f)
    engine.gemm_packed(PX, E.PACK_ROWS, PY, E.PACK_COLS, out)
    assert_close(out.numpy(), O.matmul_forward(X, Y), _absprod(X, Y), f"packed forward {shape} {blocks}")
    dX_ref, dY_ref = O.matmul_backward(X, Y, dC)
    dX = engine.empty((m, k), f)
    engine.gemm_packed(PC, E.PACK_ROWS, PY, E.PACK_ROWS, dX)
    assert_close(dX.numpy(), dX_ref, _absprod(dC, Y.T), f"packed dA {shape} {blocks}")
    dY = engine.empty((k, n), f)
    engine.gemm_packed(PX, E.PACK_COLS, PC, E.PACK_COLS, dY)
    assert_close(dY.numpy(), dY_ref, _absprod(X.T, dC), f"packed dB {shape} {blocks}")
    # alpha, beta and a bias row
    base = r.standard_normal((m, n)).astype(f)
    bias = r.standard_normal((1, n)).astype(f)
    out2 = engine.upload(base)
    engine.gemm_packed(PX, E.PACK_ROWS, PY, E.PACK_COLS, out2, alpha=0.5, beta=2.0, bias=engine.upload(bias))
    want = (0.5 * O.matmul_forward(X, Y).astype(np.float64) + 2.0 * base + bias).astype(f)
    assert_close(out2.numpy(), want, _absprod(X, Y) + np.abs(base) + 1.0, f"packed alpha beta bias {shape} {blocks}")
    # a bias row alone (the forward product of a layer)
    out3 = engine.empty((m, n), f)
    engine.gemm_packed(PX, E.PACK_ROWS, PY, E.PACK_COLS, out3, alpha=0.25, bias=engine.upload(bias))
    want3 = (0.25 * O.matmul_forward(X, Y).astype(np.float64) + bias).astype(f)
    assert_close(out3.numpy(), want3, _absprod(X, Y) + 1.0, f"packed alpha bias {shape} {blocks}")


@pytest.mark.parametrize("shape", [(256, 4096, 130), (256, 4096, 128), (96, 16384, 288)])
def test_k_slices_and_their_sum_pass(engine, shape):
    """Few output tiles over a long k: the product runs as k slices into scratch and an ordered sum pass (four
    columns per thread when the output's rows are whole float4, one otherwise), with alpha and beta applied once."""
    m, k, n = shape
    r = rng(m + k + n)
    X = r.standard_normal((m, k)).astype(f)
    Y = (r.standard_normal((k, n)) * 0.1).astype(f)
    base = r.standard_normal((m, n)).astype(f)
    PX = engine.packed(m, k, E.PACK_ROWS).pack(engine.upload(X))
    PY = engine.packed(k, n, E.PACK_COLS, 0, PX.blocks()[0]).pack(engine.upload(Y))
    n0 = engine.launch_count()
    out = engine.upload(base)
    engine.gemm_packed(PX, E.PACK_ROWS, PY, E.PACK_COLS, out, alpha=0.5, beta=2.0)
    assert engine.launch_count() - n0 == 2          # the product and the sum pass
    want = (0.5 * O.matmul_forward(X, Y).astype(np.float64) + 2.0 * base).astype(f)
    assert_close(out.numpy(), want, _absprod(X, Y) + np.abs(base), f"sliced product {shape}")
    engine.set_option("tc_split_k", "off")
    try:
        whole = engine.upload(base)
        engine.gemm_packed(PX, E.PACK_ROWS, PY, E.PACK_COLS, whole, alpha=0.5, beta=2.0)
    finally:
        engine.set_option("tc_split_k", "on")
    assert_close(out.numpy(), whole.numpy(), _absprod(X, Y) + np.abs(base), f"sliced against whole {shape}")


@pytest.mark.parametrize("act", [E.ACT_GELU, E.ACT_LEAKY_RELU, E.ACT_TANH, E.ACT_SIGMOID, E.ACT_NONE])
def test_activation_written_in_packed_form(engine, act):
    """y = act(x) and dx = dy * act'(saved) packed on the fly: the FP32 copies are bit-identical to the
    stand-alone activation kernels, and products of the packed results match the oracle's."""
    r = rng(9)
    m, k, n = 384, 520, 260
    x = r.standard_normal((m, k)).astype(f)
    dy = (r.standard_normal((m, k)) * 1e-3).astype(f)
    W = (r.standard_normal((k, n)) * 0.1).astype(f)
    xd, dyd = engine.upload(x), engine.upload(dy)
    both = E.PACK_ROWS | E.PACK_COLS
    PW = engine.packed(k, n, both, 128, 128).pack(engine.upload(W))
    # forward
    P = engine.packed(m, k, both)
    y = engine.empty((m, k), f)
    P.act_forward(act, xd, y, 0.01)
    y_alone = engine.act_forward(act, xd, 0.01).numpy() if act != E.ACT_NONE else x
    np.testing.assert_array_equal(y.numpy(), y_alone)
    out = engine.empty((m, n), f)
    engine.gemm_packed(P, E.PACK_ROWS, PW, E.PACK_COLS, out)
    ref_y = {E.ACT_GELU: O.gelu_forward, E.ACT_LEAKY_RELU: lambda v: O.leaky_relu_forward(v, f(0.01)), E.ACT_TANH: O.tanh_forward,
             E.ACT_SIGMOID: O.sigmoid_forward, E.ACT_NONE: lambda v: v}[act](x)
    assert_close(out.numpy(), O.matmul_forward(ref_y, W), _absprod(ref_y, W), f"act {act} forward packed product")
    # backward: the saved tensor is the input for GELU / LeakyReLU, the output for Tanh and Sigmoid (whose value at
    # the zeros beyond a partly filled column tile is not zero: those must not reach the padding of the operand)
    saved = ref_y if act in (E.ACT_TANH, E.ACT_SIGMOID) else x
    dx = engine.empty((m, k), f)
    P.act_backward(act, engine.upload(saved) if act != E.ACT_NONE else None, dyd, dx, 0.01)
    dx_alone = engine.act_backward(act, engine.upload(saved), dyd, 0.01).numpy() if act != E.ACT_NONE else dy
    np.testing.assert_array_equal(dx.numpy(), dx_alone)
    ref_dx = {E.ACT_GELU: O.gelu_backward, E.ACT_LEAKY_RELU: lambda s, d: O.leaky_relu_backward(s, d, f(0.01)),
              E.ACT_TANH: O.tanh_backward, E.ACT_SIGMOID: O.sigmoid_backward, E.ACT_NONE: lambda s, d: d}[act](saved, dy)
    # weight-gradient shape: (k x m) (m x n'), both by columns
    G = (r.standard_normal((m, n)) * 1e-3).astype(f)
    PG = engine.packed(m, n, both).pack(engine.upload(G))
    dWt = engine.empty((k, n), f)
    engine.gemm_packed(P, E.PACK_COLS, PG, E.PACK_COLS, dWt)
    assert_close(dWt.numpy(), O.matmul_backward(ref_dx, W, G)[1], _absprod(ref_dx.T, G), f"act {act} backward packed dW")
    # without an FP32 copy the operand is the same, except that GELU is then evaluated in short arithmetic
    # (fused multiply-adds, tanh from exp2 and a reciprocal): equal within the same bound
    P2 = engine.packed(m, k, both)
    P2.act_backward(act, engine.upload(saved) if act != E.ACT_NONE else None, dyd, None, 0.01)
    dWt2 = engine.empty((k, n), f)
    engine.gemm_packed(P2, E.PACK_COLS, PG, E.PACK_COLS, dWt2)
    if act == E.ACT_GELU:
        assert_close(dWt2.numpy(), O.matmul_backward(ref_dx, W, G)[1], _absprod(ref_dx.T, G), f"act {act} backward packed dW, no copy")
    else:
        np.testing.assert_array_equal(dWt2.numpy(), dWt.numpy())
    P3 = engine.packed(m, k, both)
    P3.act_forward(act, xd, None, 0.01)
    out3 = engine.empty((m, n), f)
    engine.gemm_packed(P3, E.PACK_ROWS, PW, E.PACK_COLS, out3)
    assert_close(out3.numpy(), O.matmul_forward(ref_y, W), _absprod(ref_y, W), f"act {act} forward packed product, no copy")


def test_loss_gradient_formed_inside_the_packing_pass(engine):
    """prad_mse_act_backward_pack == prad_mse_backward followed by prad_act_backward_pack, bit for bit."""
    r = rng(12)
    m, k = 300, 260
    z = r.standard_normal((m, k)).astype(f)
    out = O.gelu_forward(z)
    t = r.standard_normal((m, k)).astype(f)
    zd, od, td = engine.upload(z), engine.upload(out), engine.upload(t)
    both = E.PACK_ROWS | E.PACK_COLS
    P1, P2 = engine.packed(m, k, both), engine.packed(m, k, both)
    dx1, dx2 = engine.empty((m, k), f), engine.empty((m, k), f)
    g = engine.mse_backward(od, td, rows_total=4 * m)
    P1.act_backward(E.ACT_GELU, zd, g, dx1)
    P2.mse_act_backward(E.ACT_GELU, zd, od, td, 4 * m, dx2)
    np.testing.assert_array_equal(dx1.numpy(), dx2.numpy())
    assert_close(dx2.numpy(), O.gelu_backward(z, O.mse_backward(out, t, rows_total=4 * m)), 1e-6, "mse + gelu backward packed")
    W = engine.packed(k, 128, both, 128, 128).pack(engine.upload((r.standard_normal((k, 128)) * 0.1).astype(f)))
    a, b = engine.empty((m, 128), f), engine.empty((m, 128), f)
    engine.gemm_packed(P1, E.PACK_ROWS, W, E.PACK_COLS, a)
    engine.gemm_packed(P2, E.PACK_ROWS, W, E.PACK_COLS, b)
    np.testing.assert_array_equal(a.numpy(), b.numpy())


def test_block_scales_follow_the_data_range(engine):
    """Rows and columns whose magnitudes differ by 30 decades between blocks keep their 22 bits: every
    block has its own scale."""
    r = rng(4)
    m, k, n = 256, 512, 256
    X = r.standard_normal((m, k)).astype(np.float64)
    Y = r.standard_normal((k, n)).astype(np.float64)
    X *= 10.0 ** r.integers(-12, 12, (m, 1))                 # whole rows of X scaled
    X[:, 256:] *= 1e-6                                        # and the second k block much smaller
    Y[256:, :] *= 1e6
    X, Y = X.astype(f), Y.astype(f)
    PX = engine.packed(m, k, E.PACK_ROWS, 256, 0).pack(engine.upload(X))
    PY = engine.packed(k, n, E.PACK_COLS, 0, 256).pack(engine.upload(Y))
    out = engine.empty((m, n), f)
    engine.gemm_packed(PX, E.PACK_ROWS, PY, E.PACK_COLS, out)
    assert_close(out.numpy(), O.matmul_forward(X, Y), _absprod(X, Y), "block scales")


def test_packed_shape_rules(engine):
    A = engine.packed(64, 96, E.PACK_ROWS)
    B = engine.packed(80, 32, E.PACK_COLS)                   # k = 80, A has k = 96
    out = engine.empty((64, 32), f)
    with pytest.raises(_lib.PradError) as e:                 # not packed yet
        engine.gemm_packed(A, E.PACK_ROWS, B, E.PACK_COLS, out)
    assert e.value.status == _lib.ERR_INVALID
    A.pack(engine.zeros((64, 96), f))
    B.pack(engine.zeros((80, 32), f))
    with pytest.raises(_lib.PradError) as e:
        engine.gemm_packed(A, E.PACK_ROWS, B, E.PACK_COLS, out)
    assert e.value.status == _lib.ERR_SHAPE and "do not match" in str(e.value)
    with pytest.raises(_lib.PradError) as e:                 # A was created without the by-columns form
        engine.gemm_packed(A, E.PACK_COLS, B, E.PACK_COLS, out)
    assert e.value.status == _lib.ERR_INVALID
    with pytest.raises(_lib.PradError):
        engine.packed(8, 8, E.PACK_ROWS, 64, 0)              # block lengths are 128 or 256

"""Parity of the CUDA kernels, called through the C-ABI, with the golden fixtures (outputs of the
reference's own CPU code) and with the C oracle on seeded inputs.

Bars: dilation / erosion forward is BIT-EXACT (values compared with array_equal) for every merge,
padding and dtype, and so are the packed winner indices; gradients and smorph are compared within the
tolerances stated beside each assertion (summation order differs from the reference, whose own weight
gradient is not reproducible run to run)."""
import hashlib

import numpy as np
import pytest
import torch

import workloads as WL
from oracle import oracle as O

pytestmark = pytest.mark.gpu

MERGES = ("max", "min", "sum", "mean", "identity")


@pytest.fixture(scope="module")
def C():
    import _cabi
    return _cabi


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def flip(w):
    return np.ascontiguousarray(w[..., ::-1, ::-1])


def grad_tol(dtype, scale=1.0):
    # fp32: the reference's own CPU<->CUDA bar (rtol 1e-4), atol scaled to the magnitude of the sums
    return dict(rtol=1e-4, atol=1e-5 * scale) if dtype == np.float32 else dict(rtol=1e-12, atol=1e-12 * scale)


def test_morph_golden_fixtures(C, manifest, golden):
    data = golden("morph_small")
    for case in manifest["morph_small"]:
        k = case["key"]
        x, w, gy = data[k + "_x"], data[k + "_w"], data[k + "_gy"]
        op, merge, padding, pv = case["op"], case["merge"], case["padding"], case["padding_value"]
        wk = w if op == "dilation" else flip(w)
        y = C.morpho_forward(op, dev(x), dev(wk), merge, padding, pv)
        assert np.array_equal(y.cpu().numpy(), data[k + "_y"]), f"forward not bit-exact: {case}"
        gx, gw = C.morpho_backward(op, dev(x), dev(wk), dev(gy), merge, padding, pv)
        gw = gw.cpu().numpy()
        if op == "erosion":
            gw = flip(gw)
        tol = grad_tol(x.dtype, scale=float(np.abs(gy).sum()) / 100)
        np.testing.assert_allclose(gx.cpu().numpy(), data[k + "_gx"], **grad_tol(x.dtype), err_msg=str(case))
        np.testing.assert_allclose(gw, data[k + "_gw"], **tol, err_msg=str(case))


@pytest.mark.parametrize("dtype", [np.float32, np.float64])
@pytest.mark.parametrize("op", ["dilation", "erosion"])
def test_morph_exhaustive_small_shapes(C, op, dtype):
    """Every H, W in 1..6 (plus sizes around the 64 x 32 tile), k in {1, 2, 3, 4, 5}, all merges, two paddings,
    against the oracle: forward bit-exact, winner indices identical."""
    rng = np.random.default_rng(5)
    shapes = [(h, w) for h in range(1, 7) for w in range(1, 7)] + [(31, 63), (32, 64), (33, 65), (40, 130)]
    for (H, W) in shapes:
        for (kH, kW) in ((1, 1), (3, 3), (2, 3), (5, 5), (4, 1)) if H <= 6 else ((3, 3), (5, 4), (7, 7)):
            for merge in MERGES:
                Ci, Co = (3, 3) if merge == "identity" else (2, 5)
                x = rng.integers(-3, 4, (2, Ci, H, W)).astype(dtype) if (H + W) % 2 else rng.standard_normal((2, Ci, H, W)).astype(dtype)
                w = rng.standard_normal((Co, 1 if merge == "identity" else Ci, kH, kW)).astype(dtype).round(1)
                for padding, pv in (("replicate", 0.0), ("constant", 0.5), ("geodesic", 0.0)):
                    want, want_idx = O.morpho_forward(op, x, w, merge, padding, pv, with_index=True)
                    got, got_idx = C.morpho_forward(op, dev(x), dev(w), merge, padding, pv, with_index=True)
                    assert np.array_equal(got.cpu().numpy(), want), (op, merge, padding, H, W, kH, kW)
                    if merge in ("max", "min"):
                        assert np.array_equal(got_idx.cpu().numpy(), want_idx), (op, merge, padding, H, W, kH, kW)


@pytest.mark.parametrize("dtype", [np.float32, np.float64])
@pytest.mark.parametrize("k", [3, 5, 7, 11, (9, 9), (6, 3)])
def test_morph_kernel_sizes_forward_and_backward(C, k, dtype):
    """Specialised widths (3, 5, 7, 11) and the any-size path, larger channel counts, against the oracle."""
    rng = np.random.default_rng(11)
    kH, kW = (k, k) if isinstance(k, int) else k
    for op in ("dilation", "erosion"):
        for merge in MERGES:
            Ci, Co = (6, 6) if merge == "identity" else (5, 7)
            x = rng.standard_normal((2, Ci, 37, 70)).astype(dtype)
            w = (0.3 * rng.standard_normal((Co, 1 if merge == "identity" else Ci, kH, kW))).astype(dtype)
            gy = rng.standard_normal((2, Co, 37, 70)).astype(dtype)
            for padding in ("replicate", "zero"):
                want = O.morpho_forward(op, x, w, merge, padding)
                got = C.morpho_forward(op, dev(x), dev(w), merge, padding)
                assert np.array_equal(got.cpu().numpy(), want), (op, merge, padding, k)
                wgx, wgw = O.morpho_backward(op, x, w, gy, merge, padding)
                gx, gw = C.morpho_backward(op, dev(x), dev(w), dev(gy), merge, padding)
                np.testing.assert_allclose(gx.cpu().numpy(), wgx, **grad_tol(dtype, 10), err_msg=str((op, merge, padding, k)))
                np.testing.assert_allclose(gw.cpu().numpy(), wgw, **grad_tol(dtype, 100), err_msg=str((op, merge, padding, k)))


def test_saved_indices_equal_recomputed(C):
    """MAX / MIN backward from the saved winners equals the backward that recomputes them into the
    workspace (the reference's save_indices=True / False equivalence)."""
    rng = np.random.default_rng(3)
    x = rng.standard_normal((3, 4, 45, 83)).astype(np.float32)
    w = rng.standard_normal((6, 4, 5, 5)).astype(np.float32)
    gy = rng.standard_normal((3, 6, 45, 83)).astype(np.float32)
    for op in ("dilation", "erosion"):
        for merge in ("max", "min"):
            y, idx = C.morpho_forward(op, dev(x), dev(w), merge, "replicate", with_index=True)
            _, want_idx = O.morpho_forward(op, x, w, merge, "replicate", with_index=True)
            assert np.array_equal(idx.cpu().numpy(), want_idx)
            a = C.morpho_backward(op, dev(x), dev(w), dev(gy), merge, "replicate", idx=idx)
            b = C.morpho_backward(op, dev(x), dev(w), dev(gy), merge, "replicate", idx=None)
            np.testing.assert_allclose(a[0].cpu().numpy(), b[0].cpu().numpy(), rtol=1e-5, atol=1e-5)
            np.testing.assert_allclose(a[1].cpu().numpy(), b[1].cpu().numpy(), rtol=1e-4, atol=1e-3)
            wgx, wgw = O.morpho_backward(op, x, w, gy, merge, "replicate")
            np.testing.assert_allclose(a[0].cpu().numpy(), wgx, rtol=1e-4, atol=1e-5)
            np.testing.assert_allclose(a[1].cpu().numpy(), wgw, rtol=1e-4, atol=1e-3)


@pytest.mark.parametrize("dtype", [np.float32, np.float64])
def test_winner_index_with_many_input_channels(C, dtype):
    """The tiled tap search stages the windows of a GROUP of input channels in shared memory; with more channels than
    fit (70 in double at 5 x 5: three groups) every pixel must still be searched exactly once, in the group that holds
    its winning channel. Indices and values against the oracle, both operations, both merges."""
    rng = np.random.default_rng(23)
    x = rng.standard_normal((2, 70, 21, 40)).astype(dtype)
    w = (0.5 * rng.standard_normal((3, 70, 5, 5))).astype(dtype)
    for op in ("dilation", "erosion"):
        for merge in ("max", "min"):
            want, want_idx = O.morpho_forward(op, x, w, merge, "replicate", with_index=True)
            got, got_idx = C.morpho_forward(op, dev(x), dev(w), merge, "replicate", with_index=True)
            assert np.array_equal(got.cpu().numpy(), want), (op, merge)
            assert np.array_equal(got_idx.cpu().numpy(), want_idx), (op, merge)


def test_ties_route_to_first_tap_and_channel_zero(C):
    """All-equal input: tap (0, 0) and channel 0 take every gradient; with replicate padding grad_weight
    receives all 25 contributions of a 5 x 5 image but grad_input only those whose tap (0, 0) is inside."""
    x = torch.zeros(1, 2, 5, 5, device="cuda")
    w = torch.zeros(1, 2, 3, 3, device="cuda")
    gy = torch.ones(1, 1, 5, 5, device="cuda")
    gx, gw = C.morpho_backward("dilation", x, w, gy, "max", "replicate")
    assert gw[0, 0, 0, 0].item() == 25 and gw.sum().item() == 25
    assert gx[0, 0].sum().item() == 16 and gx[0, 1].abs().sum().item() == 0
    gx, gw = C.morpho_backward("erosion", x, w, gy, "sum", "zero")
    assert gw[0, :, 0, 0].tolist() == [-25.0, -25.0] and gx.sum().item() == 32


@pytest.mark.parametrize("dtype", [np.float32, np.float64])
def test_negative_zero_inputs(C, dtype):
    """Inputs that hold -0.0. A candidate x + w is -0.0 only where x is -0.0 (and w a zero), so the sign of a zero
    extremum is the only thing that can differ. SUM and MEAN merges start from +0.0, which absorbs the sign of a zero
    channel extremum, and are bit-identical to the reference's rule (compared on raw bits). For MAX / MIN / IDENTITY
    the reference keeps the FIRST of several zero candidates (strict comparison), the hardware max / min instruction
    orders -0 < +0: the results are equal as numbers everywhere, the raw bits may differ only where the result is a
    zero, and the winner indices are the reference's."""
    rng = np.random.default_rng(41)
    bits = np.uint32 if dtype == np.float32 else np.uint64
    x = rng.choice(np.array([-0.0, 0.0, -0.0, 0.0, -1.0, 0.5], dtype), size=(2, 3, 19, 37))
    gy = rng.standard_normal((2, 3, 19, 37)).astype(dtype)
    for op in ("dilation", "erosion"):
        for merge in MERGES:
            w = rng.choice(np.array([0.0, -0.0, -0.25], dtype), size=(3, 1 if merge == "identity" else 3, 3, 3))
            want, want_idx = O.morpho_forward(op, x, w, merge, "zero", with_index=True)
            got, got_idx = C.morpho_forward(op, dev(x), dev(w), merge, "zero", with_index=True)
            got = got.cpu().numpy()
            assert np.array_equal(got, want), (op, merge)
            differs = got.view(bits) != want.view(bits)
            if merge in ("sum", "mean"):
                assert not differs.any(), (op, merge)
            else:
                assert (want[differs] == 0).all(), (op, merge)
            if merge in ("max", "min"):
                assert np.array_equal(got_idx.cpu().numpy(), want_idx), (op, merge)
            wgx, wgw = O.morpho_backward(op, x, w, gy, merge, "zero")
            gx, gw = C.morpho_backward(op, dev(x), dev(w), dev(gy), merge, "zero")
            np.testing.assert_allclose(gx.cpu().numpy(), wgx, **grad_tol(dtype, 10), err_msg=str((op, merge)))
            np.testing.assert_allclose(gw.cpu().numpy(), wgw, **grad_tol(dtype, 100), err_msg=str((op, merge)))


@pytest.mark.parametrize("merge", ["sum", "mean", "max", "min", "identity"])
@pytest.mark.parametrize("k", [3, 5, 7])
def test_fused_dilation_erosion_pass_is_bit_identical(C, merge, k):
    """mc_morpho_pair_forward (the two halves of sigma_layer, morphocore/functional/sigma_layer.py:73-83, in one pass) against
    two mc_morpho_forward calls, erosion with the flipped structuring element as morphocore/functional/erosion.py:89 passes it:
    bit-identical outputs for every merge and border it covers, partial tiles and a width that is not a multiple of four
    included; the cases it does not cover answer MC_ERR_UNSUPPORTED and launch nothing."""
    g = torch.Generator().manual_seed(77 + k)
    co, ci = (6, 6) if merge == "identity" else (5, 7)
    for shape, padding, value in (((2, ci, 70, 100), "replicate", 0.0), ((1, ci, 33, 68), "zero", 0.0), ((2, ci, 64, 64), "constant", 0.25)):
        x = torch.randn(shape, generator=g).cuda()
        w = (0.3 * torch.randn((co, 1 if merge == "identity" else ci, k, k), generator=g)).cuda()
        pair = C.morpho_pair_forward(x, w, merge, padding, value)
        assert pair is not None
        yd = C.morpho_forward("dilation", x, w, merge, padding, value)
        ye = C.morpho_forward("erosion", x, torch.flip(w, dims=(-2, -1)).contiguous(), merge, padding, value)
        assert torch.equal(pair[0], yd)
        assert torch.equal(pair[1], ye)
    x = torch.randn((1, ci, 40, 40), generator=g).cuda()
    w = (0.3 * torch.randn((co, 1 if merge == "identity" else ci, k, k), generator=g)).cuda()
    assert C.morpho_pair_forward(x, w, merge, "geodesic") is None                       # the fill value differs between the two
    assert C.morpho_pair_forward(x.double(), w.double(), merge) is None                 # float only
    w4 = (0.3 * torch.randn((co, 1 if merge == "identity" else ci, 4, 4), generator=g)).cuda()
    assert C.morpho_pair_forward(x, w4, merge) is None                                  # 3 x 3, 5 x 5, 7 x 7 only
    assert C.morpho_pair_forward(x[..., :37].contiguous(), w, merge) is None            # rows that TMA cannot address (pitch not 16 bytes)


def test_per_sample_weights(C):
    """weight_batch_stride: one structuring element per batch element equals running each element alone,
    and grad_weight is the sum over the batch."""
    rng = np.random.default_rng(9)
    x = rng.standard_normal((3, 2, 20, 33)).astype(np.float32)
    w5 = rng.standard_normal((3, 4, 2, 3, 3)).astype(np.float32)
    gy = rng.standard_normal((3, 4, 20, 33)).astype(np.float32)
    for merge in ("sum", "max"):
        y = C.morpho_forward("dilation", dev(x), dev(w5), merge)
        gx, gw = C.morpho_backward("dilation", dev(x), dev(w5), dev(gy), merge)
        gw_sum = np.zeros((4, 2, 3, 3), np.float32)
        for b in range(3):
            yb = O.morpho_forward("dilation", x[b:b + 1], w5[b], merge)
            assert np.array_equal(y[b:b + 1].cpu().numpy(), yb)
            gxb, gwb = O.morpho_backward("dilation", x[b:b + 1], w5[b], gy[b:b + 1], merge)
            np.testing.assert_allclose(gx[b:b + 1].cpu().numpy(), gxb, rtol=1e-4, atol=1e-5)
            gw_sum += gwb
        np.testing.assert_allclose(gw.cpu().numpy(), gw_sum, rtol=1e-4, atol=1e-3)


def smorph_tols(dtype, alpha0):
    # values: rtol 1e-4 / atol 1e-5 in fp32 (the stated bar), 1e-12 / 1e-12 in fp64 (measured worst deviation from
    # the oracle over these cases: 4.4e-14 of the largest value, 2.3e-14 of the largest gradient). Gradients multiply
    # the rounding of exp() by alpha, so their tolerance grows with |alpha| beyond 10.
    amp = max(1.0, abs(alpha0) / 10.0)
    if dtype == np.float32:
        return dict(rtol=1e-4, atol=1e-5), dict(rtol=1e-4 * amp, atol=3e-5 * amp)
    return dict(rtol=1e-12, atol=1e-12), dict(rtol=1e-12 * amp, atol=1e-12 * amp)


def test_smorph_golden_fixtures(C, manifest, golden):
    data = golden("smorph_small")
    for case in manifest["smorph_small"]:
        k = case["key"]
        x, w, alpha, gy = data[k + "_x"], data[k + "_w"], data[k + "_alpha"], data[k + "_gy"]
        merge = case["merge"]
        wt = O.smorph_weight(w, alpha, merge)
        ytol, gtol = smorph_tols(x.dtype, case["alpha0"])
        y = C.smorph_forward(dev(x), dev(wt), dev(alpha), merge)
        np.testing.assert_allclose(y.cpu().numpy(), data[k + "_y"], **ytol, err_msg=str(case))
        gx, gwt, ga = C.smorph_backward(dev(x), dev(wt), dev(alpha), y, dev(gy), merge)
        np.testing.assert_allclose(gx.cpu().numpy(), data[k + "_gx"], **gtol, err_msg=str(case))
        # operator-level gradients of w~ and alpha against the oracle (the fixture holds the gradients of
        # the user-level w and alpha, checked through autograd in test_gpu_autograd.py)
        ogx, ogw, oga = O.smorph_backward(x, wt, alpha, gy, merge)
        wtol = dict(rtol=gtol["rtol"], atol=gtol["atol"] * 30)
        np.testing.assert_allclose(gwt.cpu().numpy(), ogw, **wtol, err_msg=str(case))
        np.testing.assert_allclose(ga.cpu().numpy().reshape(-1), oga.reshape(-1), **wtol, err_msg=str(case))


def mask_ambiguous_winners(gy, x, w, alpha, merge):
    """MAX / MIN merges share the gradient between the channels whose soft extremum lies within 1e-6 of
    the merged value: a step function of the channel outputs. Where the runner-up is closer than 1e-5
    the last bits of exp() decide which side of the step a pixel falls on, in the reference as well, so
    those pixels get a zero output gradient in the comparison."""
    if merge not in ("max", "min"):
        return gy
    Ci = x.shape[1]
    outs = np.stack([O.smorph_forward(x[:, i:i + 1], w[:, i:i + 1], alpha[:, i:i + 1], "sum") for i in range(Ci)], 0)
    srt = np.sort(outs, 0)
    gap = (srt[1] - srt[0]) if merge == "min" else (srt[-1] - srt[-2])
    gy = gy.copy()
    gy[gap < 1e-5] = 0
    return gy


@pytest.mark.parametrize("dtype", [np.float32, np.float64])
@pytest.mark.parametrize("k", [3, 5, 7, (4, 3), 11])
def test_smorph_against_oracle(C, k, dtype):
    rng = np.random.default_rng(21)
    kH, kW = (k, k) if isinstance(k, int) else k
    for merge in MERGES:
        Ci, Co = (4, 4) if merge == "identity" else (3, 5)
        x = rng.standard_normal((2, Ci, 35, 67)).astype(dtype)
        w = (0.2 * rng.standard_normal((Co, 1 if merge == "identity" else Ci, kH, kW))).astype(dtype)
        gy = rng.standard_normal((2, Co, 35, 67)).astype(dtype)
        for a0 in (-8.0, -1.0, 0.0, 2.0, 30.0):
            ashape = (Co,) if merge == "identity" else (Co, Ci)
            alpha = (a0 + 0.1 * rng.standard_normal(ashape)).astype(dtype)
            if a0 == 0.0:
                alpha[...] = 0.0
            ytol, gtol = smorph_tols(dtype, a0)
            want = O.smorph_forward(x, w, alpha, merge)
            y = C.smorph_forward(dev(x), dev(w), dev(alpha), merge)
            np.testing.assert_allclose(y.cpu().numpy(), want, **ytol, err_msg=str((merge, k, a0)))
            g = mask_ambiguous_winners(gy, x, w, alpha, merge)
            # Gradients are checked against the oracle run in double on the same (float) inputs: its float run is
            # itself up to one full tolerance away from the double one at |alpha| = 8 (measured: 7e-5 on grad_input of
            # the max merge, 7 x 7), so a float-to-float comparison would test the oracle's rounding, not the kernel's.
            f64 = np.float64
            wgx, wgw, wga = O.smorph_backward(x.astype(f64), w.astype(f64), alpha.astype(f64), g.astype(f64), merge)
            gx, gw, ga = C.smorph_backward(dev(x), dev(w), dev(alpha), y, dev(g), merge)
            np.testing.assert_allclose(gx.cpu().numpy(), wgx, **gtol, err_msg=str((merge, k, a0)))
            sums = dict(rtol=gtol["rtol"], atol=gtol["atol"] * 100)
            np.testing.assert_allclose(gw.cpu().numpy(), wgw, **sums, err_msg=str((merge, k, a0)))
            np.testing.assert_allclose(ga.cpu().numpy().reshape(-1), wga.reshape(-1), **sums, err_msg=str((merge, k, a0)))


def sha(t):
    return hashlib.sha256(t.cpu().numpy().tobytes()).hexdigest()


def entry(manifest, key):
    return next(m for m in manifest["full_size"] if m["key"] == key)


@pytest.mark.parametrize("case", [
    # kernel, image, alphas, spread of x
    (3, 224, "uniform", 1.0), (3, 97, "per_pair", 1.0), (3, 61, "extreme", 1.0), (3, 130, "per_pair", 30.0),
    (5, 128, "per_pair", 1.0), (7, 128, "uniform_negative", 1.0), (7, 70, "extreme", 3.0)])
@pytest.mark.parametrize("merge", ["sum", "mean", "identity"])
def test_smorph_factorised_forward_matches_double(C, case, merge):
    """The float forward pass of the sum / mean / identity merges replaces exp(|alpha| (u_k - ref)) by the product of a
    per-pixel and a per-tap factor wherever |alpha| * (range of x in a warp's block + range of w) allows it, and
    falls back to the max-subtracting form elsewhere (large |alpha|, wide-spread inputs). Both must agree with the
    double kernel, which always subtracts the maximum: partial tiles, borders, alpha = 0, signs mixed within one
    output channel, and ranges on both sides of the switch."""
    k, hw, kind, spread = case
    g = torch.Generator().manual_seed(1234 + k + hw)
    co, ci = (6, 6) if merge == "identity" else (6, 5)
    x = (spread * torch.randn((2, ci, hw, hw + 3), generator=g)).cuda()
    w = (0.3 * torch.randn((co, 1 if merge == "identity" else ci, k, k), generator=g)).cuda()
    pairs = (co,) if merge == "identity" else (co, ci)
    if kind == "uniform":
        a = torch.full(pairs, 2.0)
    elif kind == "uniform_negative":
        a = torch.full(pairs, -8.0)
    elif kind == "per_pair":
        a = 3.0 * torch.randn(pairs, generator=g)
    else:
        values = torch.tensor([-1000.0, -40.0, -6.0, -0.5, 0.0, -1e-8, 1e-7, 1e-4, 3.0, 25.0, 400.0])
        a = values[torch.randint(0, len(values), pairs, generator=g)]
    a = a.cuda()
    y = C.smorph_forward(x, w, a, merge)
    ref = C.smorph_forward(x.double(), w.double(), a.double(), merge)
    assert torch.isfinite(y).all()
    # rtol 1e-4 / atol 1e-5 per channel output (the bar of the other float smorph tests), scaled by the number of
    # channels a sum adds up
    scale = ci if merge == "sum" else 1
    torch.testing.assert_close(y.double(), ref, rtol=1e-4, atol=1e-5 * scale * max(1.0, spread))


@pytest.mark.parametrize("case", [
    # kernel, image, alphas, spread of x
    (3, 224, "uniform", 1.0), (3, 97, "per_pair", 1.0), (3, 61, "extreme", 1.0), (3, 130, "per_pair", 30.0), (3, 100, "offset", 1.0),
    # widths that are multiples of four take the 3 x 3 kernel's fast channel loop (gradients staged by cp.async)
    (3, 221, "uniform", 1.0), (3, 125, "offset", 1.0), (3, 93, "per_pair", 30.0),
    (5, 128, "uniform", 1.0), (5, 97, "per_pair", 1.0), (5, 61, "extreme", 1.0), (7, 128, "uniform_negative", 1.0),
    (7, 131, "per_pair", 1.0), (7, 70, "extreme", 3.0), (7, 100, "per_pair", 30.0)])
@pytest.mark.parametrize("merge", ["sum", "mean", "identity"])
def test_smorph_factorised_backward_matches_double(C, case, merge):
    """The float backward pass of 5 x 5 and 7 x 7 structuring elements (sum / mean / identity merges) recomputes the
    sums S and N of a pair from the factorised form wherever the ranges allow it, the 3 x 3 one takes its exponentials
    relative to a bound of the thread's patch instead of the pixel's maximum, and both subtract the maximum elsewhere.
    All must agree with the double kernel, which always subtracts the maximum: interior and border blocks, partial
    tiles, alpha = 0 and alphas too small for the bounded form's scaled units, signs mixed within one input channel,
    ranges on both sides of the switch, inputs far from zero, grad_output rows aligned for cp.async or not."""
    k, hw, kind, spread = case
    g = torch.Generator().manual_seed(4321 + k + hw)
    co, ci = (6, 6) if merge == "identity" else (6, 5)
    x = (spread * torch.randn((2, ci, hw, hw + 3), generator=g)).cuda()
    if kind == "offset":   # activations of a deep layer: unit spread around 100
        x = 100.0 + x
    w = (0.3 * torch.randn((co, 1 if merge == "identity" else ci, k, k), generator=g)).cuda()
    gy = torch.randn((2, co, hw, hw + 3), generator=g).cuda()
    pairs = (co,) if merge == "identity" else (co, ci)
    if kind == "uniform":
        a = torch.full(pairs, 2.0)
    elif kind == "uniform_negative":
        a = torch.full(pairs, -8.0)
    elif kind == "per_pair":
        a = 3.0 * torch.randn(pairs, generator=g)
    elif kind == "offset":
        a = 2.0 + 0.5 * torch.randn(pairs, generator=g)
    else:
        values = torch.tensor([-1000.0, -40.0, -6.0, -0.5, 0.0, -1e-8, 1e-7, 1e-4, 3.0, 25.0, 400.0])
        a = values[torch.randint(0, len(values), pairs, generator=g)]
    a = a.cuda()
    y = C.smorph_forward(x, w, a, merge)
    gx, gw, ga = C.smorph_backward(x, w, a, y, gy, merge)
    yd = C.smorph_forward(x.double(), w.double(), a.double(), merge)
    rx, rw, ra = C.smorph_backward(x.double(), w.double(), a.double(), yd, gy.double(), merge)
    for t in (gx, gw, ga):
        assert torch.isfinite(t).all()
    # Rounding of exp() is multiplied by |alpha| in the gradients (see smorph_tols); sums over the image are compared
    # relative to their largest element.
    amp = max(1.0, float(a.abs().max()) / 10.0)
    torch.testing.assert_close(gx.double(), rx, rtol=1e-4 * amp, atol=3e-5 * amp * max(1.0, spread))
    torch.testing.assert_close(gw.double(), rw, rtol=1e-4 * amp, atol=1e-4 * amp * float(rw.abs().max()))
    torch.testing.assert_close(ga.double(), ra, rtol=1e-4 * amp, atol=1e-4 * amp * float(ra.abs().max()))


def test_smorph_3x3_random_shapes_against_double(C):
    """Sixty random 3 x 3 problems (1-3 images of up to 90 x 160 pixels, widths that are multiples of four so that the fast
    channel loop of the backward kernel runs, 1-9 channels, sum / mean / identity merges, inputs spread over 0.1 to 30 units
    around 0, 50 or -200, alphas up to +-25 with zeros mixed in): the float kernels against the double kernels. The parameter
    gradients are sums over the image of terms of both signs, so their error is held against the sum of the terms'
    magnitudes (the same backward pass on |grad_output|), the input gradient and the output against their largest element."""
    import random
    random.seed(5)
    g = torch.Generator().manual_seed(5)
    for _ in range(60):
        merge = random.choice(["sum", "mean", "identity"])
        B, H, W = random.randint(1, 3), random.randint(3, 90), 4 * random.randint(1, 40)
        ci = random.randint(1, 9)
        co = ci if merge == "identity" else random.randint(1, 9)
        spread, offset = random.choice([0.1, 1.0, 1.0, 5.0, 30.0]), random.choice([0.0, 0.0, 50.0, -200.0])
        x = (offset + spread * torch.randn((B, ci, H, W), generator=g)).cuda()
        w = (random.choice([0.05, 0.3, 2.0]) * torch.randn((co, 1 if merge == "identity" else ci, 3, 3), generator=g)).cuda()
        pairs = (co,) if merge == "identity" else (co, ci)
        a = (random.choice([0.5, 2.0, 8.0]) * torch.randn(pairs, generator=g)).cuda()
        if random.random() < 0.3:
            a[(torch.rand(pairs, generator=g) < 0.3).cuda()] = 0.0
        gy = torch.randn((B, co, H, W), generator=g).cuda()
        y = C.smorph_forward(x, w, a, merge)
        yd = C.smorph_forward(x.double(), w.double(), a.double(), merge)
        gx, gw, ga = C.smorph_backward(x, w, a, y, gy, merge)
        rx, rw, ra = C.smorph_backward(x.double(), w.double(), a.double(), yd, gy.double(), merge)
        _, sw, sa = C.smorph_backward(x.double(), w.double(), a.double(), yd, gy.double().abs(), merge)
        where = f"{merge} {(B, ci, co, H, W)} spread {spread} offset {offset}"
        amp = max(1.0, float(a.abs().max()) / 10.0)   # rounding of exp() is multiplied by |alpha| in the gradients
        for t in (y, gx, gw, ga):
            assert torch.isfinite(t).all(), where
        scale = ci if merge == "sum" else 1
        assert float((y.double() - yd).abs().max()) <= 1e-4 * float(yd.abs().max()) + 1e-5 * scale * max(1.0, spread), where
        assert float((gx.double() - rx).abs().max()) <= 1e-4 * amp * max(float(rx.abs().max()), 1e-6), where
        assert float((gw.double() - rw).abs().max()) <= 1e-4 * amp * float(sw.abs().max()), where
        assert float((ga.double() - ra).abs().max()) <= 1e-4 * amp * float(sa.abs().max()), where


@pytest.mark.parametrize("merge", ["max", "min"])
@pytest.mark.parametrize("k", [3, 5])
def test_smorph_winner_merges_at_scale(C, merge, k):
    """MAX / MIN merges of smorph on a larger problem (16 input channels, 8 output channels, several tiles with partial
    ones): the float kernels against the double kernels. Only the channels within 1e-6 of the merged value receive
    gradient, shared equally (csrc/cpp/smorph_cpu_kernels.hxx:507-519): pixels whose runner-up channel is closer than 1e-5
    are excluded from the gradient comparison, as in test_smorph_against_oracle, because rounding decides their side."""
    g = torch.Generator().manual_seed(99 + k)
    B, Ci, Co, H, W = 2, 16, 8, 96, 130
    x = torch.randn((B, Ci, H, W), generator=g).cuda()
    w = (0.3 * torch.randn((Co, Ci, k, k), generator=g)).cuda()
    a = (2.0 * torch.randn((Co, Ci), generator=g)).cuda()
    gy = torch.randn((B, Co, H, W), generator=g).cuda()
    xd, wd, ad = x.double(), w.double(), a.double()
    per_channel = torch.stack([C.smorph_forward(xd[:, i:i + 1].contiguous(), wd[:, i:i + 1].contiguous(), ad[:, i:i + 1].contiguous(), "sum")
                               for i in range(Ci)])
    ordered = per_channel.sort(0).values
    gap = (ordered[1] - ordered[0]) if merge == "min" else (ordered[-1] - ordered[-2])
    gy = torch.where(gap < 1e-5, torch.zeros_like(gy), gy)
    y = C.smorph_forward(x, w, a, merge)
    yd = C.smorph_forward(xd, wd, ad, merge)
    torch.testing.assert_close(y.double(), yd, rtol=1e-4, atol=1e-5)
    gx, gw, ga = C.smorph_backward(x, w, a, y, gy, merge)
    rx, rw, ra = C.smorph_backward(xd, wd, ad, yd, gy.double(), merge)
    amp = max(1.0, float(a.abs().max()) / 10.0)
    torch.testing.assert_close(gx.double(), rx, rtol=1e-4 * amp, atol=3e-5 * amp)
    torch.testing.assert_close(gw.double(), rw, rtol=1e-4 * amp, atol=1e-4 * amp * float(rw.abs().max()))
    torch.testing.assert_close(ga.double(), ra, rtol=1e-4 * amp, atol=1e-4 * amp * float(ra.abs().max()))


@pytest.mark.parametrize("dtype", [np.float32, np.float64])
@pytest.mark.parametrize("k", [3, 5, (4, 3), 11])
def test_smorph_scm_against_oracle(C, k, dtype):
    """Smorph with the smooth channel merge through the C-ABI: output, the four gradients, partial tiles, betas of
    both signs, zero and large."""
    kh, kw = (k, k) if isinstance(k, int) else k
    rng = np.random.default_rng(77 + kh * kw)
    B, Ci, Co, H, W = 2, 5, 4, 37, 70
    x = rng.standard_normal((B, Ci, H, W)).astype(dtype)
    wt = (0.4 * rng.standard_normal((Co, Ci, kh, kw))).astype(dtype)
    alpha = (2.0 * rng.standard_normal((Co, Ci))).astype(dtype)
    beta = np.array([-20.0, -0.7, 0.0, 3.0], dtype=dtype)
    gy = rng.standard_normal((B, Co, H, W)).astype(dtype)
    want_y = O.smorph_scm_forward(x, wt, alpha, beta)
    want = O.smorph_scm_backward(x, wt, alpha, beta, gy)
    xs, ws, al, bt, gs = (torch.from_numpy(t).cuda() for t in (x, wt, alpha, beta, gy))
    y = C.smorph_scm_forward(xs, ws, al, bt)
    tol = dict(rtol=1e-4, atol=1e-5) if dtype == np.float32 else dict(rtol=1e-12, atol=1e-12)
    np.testing.assert_allclose(y.cpu().numpy(), want_y, **tol)
    got = C.smorph_scm_backward(xs, ws, al, bt, y, gs)
    gtol = dict(rtol=2e-3, atol=2e-3) if dtype == np.float32 else dict(rtol=1e-11, atol=1e-11)
    for name, a, b in zip(("gx", "gw", "galpha", "gbeta"), got, want):
        scale = max(1.0, float(np.abs(b).max()))
        np.testing.assert_allclose(a.cpu().numpy().reshape(b.shape), b, rtol=gtol["rtol"], atol=gtol["atol"] * scale, err_msg=name)


def test_smorph_scm_rejects_other_merges(C):
    x = torch.randn(1, 2, 8, 8, device="cuda")
    w = torch.randn(2, 2, 3, 3, device="cuda")
    a = torch.zeros(2, 2, device="cuda")
    with pytest.raises(RuntimeError, match="mc_smorph_scm"):
        C.smorph_forward(x, w, a, "smooth")


def test_cfg1_full_size_bit_exact(C, manifest):
    c = WL.cfg1()
    y = C.morpho_forward("dilation", c["x"].cuda(), c["w"].cuda(), "max", "replicate")
    assert sha(y) == entry(manifest, "cfg1")["y_sha256"]


def test_cfg2_full_size(C, manifest, golden):
    """Config 2 at full size: forward SHA-256 equals the reference's; grad_weight and sampled grad_input
    within rtol 1e-4 (atol scaled to the sums)."""
    data = golden("full_size")
    c = WL.cfg2()
    x, wk, gy = c["x"].cuda(), c["w"].flip((-2, -1)).contiguous().cuda(), c["gy"].cuda()
    y = C.morpho_forward("erosion", x, wk, "sum", "replicate")
    assert sha(y) == entry(manifest, "cfg2")["y_sha256"]
    gx, gw = C.morpho_backward("erosion", x, wk, gy, "sum", "replicate")
    gw = gw.flip((-2, -1)).cpu().numpy()
    np.testing.assert_allclose(gw, data["cfg2_gw"], rtol=1e-4, atol=0.05)
    np.testing.assert_allclose(gx.reshape(-1)[torch.from_numpy(data["cfg2_gx_pos"]).cuda()].cpu().numpy(), data["cfg2_gx_val"], rtol=1e-4, atol=1e-4)
    # size-independent property: every output pixel sends its gradient to exactly one tap per pair
    assert abs(gw.sum() / (-16 * c["gy"].double().sum().item()) - 1) < 1e-3


def weight_grad_fixture(data, key):
    """The reference's user-level weight gradient of a config 3 case: whole, or at sampled positions."""
    if key + "_gw" in data.files:
        return None, data[key + "_gw"].reshape(-1)
    return data[key + "_gw_pos"], data[key + "_gw_val"]


@pytest.mark.parametrize("alpha", WL.CFG3_ALPHAS)
def test_cfg3_full_size(C, golden, alpha):
    """Config 3 at full size. Operator level through the C-ABI: sampled outputs and input gradients. Then the public
    call (tanh re-parametrisation and autograd included): the weight gradient and the alpha gradient of every pair
    against the reference's, rtol 1e-4 with atol 1e-4 of the largest entry (each entry sums 262 144 pixels x 16 images
    in float, in an order that differs from the reference's)."""
    import morphocore_b200.functional as F
    data = golden("full_size")
    key = f"cfg3_a{alpha:g}"
    c = WL.cfg3(alpha)
    wt = torch.from_numpy(O.smorph_weight(c["w"].numpy(), c["alpha"].numpy(), "mean")).cuda()
    x, a, gy = c["x"].cuda(), c["alpha"].cuda(), c["gy"].cuda()
    y = C.smorph_forward(x, wt, a, "mean")
    pos = torch.from_numpy(data[key + "_pos"]).cuda()
    np.testing.assert_allclose(y.reshape(-1)[pos].cpu().numpy(), data[key + "_y_val"], rtol=1e-4, atol=1e-5)
    gx, gwt, ga = C.smorph_backward(x, wt, a, y, gy, "mean")
    np.testing.assert_allclose(gx.reshape(-1)[pos].cpu().numpy(), data[key + "_gx_val"], rtol=1e-4, atol=1e-5)
    assert torch.isfinite(gwt).all() and torch.isfinite(ga).all()
    del y, gx, gwt, ga

    xr, wr, ar = x.requires_grad_(True), c["w"].cuda().requires_grad_(True), a.requires_grad_(True)
    out = F.smorph(xr, wr, ar, channel_merge_mode="mean")
    out.backward(gy)
    np.testing.assert_allclose(xr.grad.reshape(-1)[pos].cpu().numpy(), data[key + "_gx_val"], rtol=1e-4, atol=1e-5)
    wpos, want = weight_grad_fixture(data, key)
    got = wr.grad.reshape(-1).cpu().numpy()
    got = got if wpos is None else got[wpos]
    np.testing.assert_allclose(got, want, rtol=1e-4, atol=1e-4 * max(float(np.abs(want).max()), 1e-3), err_msg="grad_weight")
    want = data[key + "_galpha"]
    np.testing.assert_allclose(ar.grad.cpu().numpy(), want, rtol=1e-4, atol=1e-4 * max(float(np.abs(want).max()), 1e-3), err_msg="grad_alpha")


@pytest.mark.parametrize("op", ["dilation", "erosion"])
def test_cfg4_full_size_bit_exact(C, manifest, golden, op):
    """Config 4 at full size (8, 64, 512, 512), fp64, identity merge: the forward SHA-256 equals the reference's, the
    whole weight gradient and 8192 sampled input gradients agree to 1e-12 (relative to the magnitude of the sums for
    the weight gradient, whose entries each add 2 097 152 terms). The reduced case pins the same on partial sums."""
    data, full = golden("full_size"), golden("cfg4_full")
    c = WL.cfg4(op)
    w = c["w"] if op == "dilation" else c["w"].flip((-2, -1)).contiguous()
    x, w, gy = c["x"].cuda(), w.cuda(), c["gy"].cuda()
    y = C.morpho_forward(op, x, w, "identity", "replicate")
    assert sha(y) == entry(manifest, f"cfg4_{op}")["y_sha256"]
    del y
    gx, gw = C.morpho_backward(op, x, w, gy, "identity", "replicate")
    if op == "erosion":
        gw = gw.flip((-2, -1))
    np.testing.assert_allclose(gw.cpu().numpy(), full[f"cfg4_{op}_gw"], rtol=1e-12, atol=1e-12 * float(c["gy"].abs().sum()) / 64)
    np.testing.assert_allclose(gx.reshape(-1)[torch.from_numpy(full[f"cfg4_{op}_gx_pos"]).cuda()].cpu().numpy(),
                               full[f"cfg4_{op}_gx_val"], rtol=1e-12, atol=1e-12)
    # size-independent property: every output pixel sends its gradient to exactly one tap
    total = gw.sum().item() * (-1.0 if op == "erosion" else 1.0)
    assert abs(total / c["gy"].sum().item() - 1) < 1e-9
    del x, w, gy, gx, gw
    c = WL.cfg4(op, B=2, C=8, HW=256)
    w = c["w"] if op == "dilation" else c["w"].flip((-2, -1)).contiguous()
    x, w, gy = c["x"].cuda(), w.cuda(), c["gy"].cuda()
    y = C.morpho_forward(op, x, w, "identity", "replicate")
    assert sha(y) == entry(manifest, f"cfg4s_{op}")["y_sha256"]
    gx, gw = C.morpho_backward(op, x, w, gy, "identity", "replicate")
    if op == "erosion":
        gw = gw.flip((-2, -1))
    # fp64: 1e-12 relative to the magnitude of the sums
    np.testing.assert_allclose(gw.cpu().numpy(), data[f"cfg4s_{op}_gw"], rtol=1e-12, atol=1e-12 * float(c["gy"].abs().sum()))
    np.testing.assert_allclose(gx.reshape(-1)[torch.from_numpy(data[f"cfg4s_{op}_gx_pos"]).cuda()].cpu().numpy(),
                               data[f"cfg4s_{op}_gx_val"], rtol=1e-12, atol=1e-12)


@pytest.mark.parametrize("dtype", [np.float32, np.float64])
def test_tma_staged_shapes_all_paddings(C, dtype):
    """Widths whose rows are 16-byte aligned take the TMA staging path: partial tiles (72, 100, 132 wide),
    many input channels (several double-buffered chunks, a partial last chunk), every border rule, both
    operations, forward bit-exact and indices identical; smorph with both alpha signs in one call."""
    rng = np.random.default_rng(17)
    for (H, W, Ci, Co, k) in ((33, 72, 11, 5, 3), (40, 100, 9, 6, 5), (31, 132, 7, 4, 7)):
        x = rng.standard_normal((2, Ci, H, W)).astype(dtype)
        w = (0.3 * rng.standard_normal((Co, Ci, k, k))).astype(dtype)
        for op in ("dilation", "erosion"):
            for padding, pv in (("replicate", 0.0), ("zero", 0.0), ("geodesic", 0.0), ("constant", -0.75)):
                for merge in ("sum", "max", "min", "mean"):
                    want, want_idx = O.morpho_forward(op, x, w, merge, padding, pv, with_index=True)
                    got, got_idx = C.morpho_forward(op, dev(x), dev(w), merge, padding, pv, with_index=True)
                    assert np.array_equal(got.cpu().numpy(), want), (op, merge, padding, H, W, k)
                    if merge in ("max", "min"):
                        assert np.array_equal(got_idx.cpu().numpy(), want_idx), (op, merge, padding, H, W, k)
        alpha = rng.standard_normal((Co, Ci)).astype(dtype) * 3     # both signs: two windows per channel
        ytol, gtol = smorph_tols(dtype, 3.0)
        for merge in ("sum", "max"):
            want = O.smorph_forward(x, w, alpha, merge)
            y = C.smorph_forward(dev(x), dev(w), dev(alpha), merge)
            np.testing.assert_allclose(y.cpu().numpy(), want, **ytol, err_msg=str((merge, H, W, k)))
        neg = -np.abs(alpha)                                        # one sign only, negative: a single window filled with +1e30
        want = O.smorph_forward(x, w, neg, "mean")
        y = C.smorph_forward(dev(x), dev(w), dev(neg), "mean")
        np.testing.assert_allclose(y.cpu().numpy(), want, **ytol)
        gy = rng.standard_normal(want.shape).astype(dtype)
        wgx, wgw, wga = O.smorph_backward(x, w, neg, gy, "mean")
        gx, gw, ga = C.smorph_backward(dev(x), dev(w), dev(neg), y, dev(gy), "mean")
        np.testing.assert_allclose(gx.cpu().numpy(), wgx, **gtol)
        np.testing.assert_allclose(gw.cpu().numpy(), wgw, rtol=gtol["rtol"], atol=gtol["atol"] * 100)
    assert C.lib.mc_device_error_count() == 0, "a bounded wait on a TMA copy timed out"


def test_bounded_wait_runs_out_and_is_counted(C):
    """The time-out path of the TMA kernels without a fault: one thread block waits 2 ms for a copy that nobody
    issues, gives up, counts itself and returns. The context stays usable (a forward pass runs right after) and the
    counter reads one more than before; it is then set back so that the session ends at zero."""
    import time
    before = C.lib.mc_device_error_count()
    assert before >= 0
    t0 = time.perf_counter()
    C.check(C.lib.mc_selftest_wait_timeout(2_000_000, C.stream()))
    torch.cuda.synchronize()
    assert time.perf_counter() - t0 < 5.0
    assert C.lib.mc_device_error_count() == before + 1
    c = WL.cfg1()
    y = C.morpho_forward("dilation", c["x"].cuda(), c["w"].cuda(), "max", "replicate")
    assert torch.isfinite(y).all()
    assert C.lib.mc_device_error_count() == before + 1
    C.check(C.lib.mc_device_error_reset())
    assert C.lib.mc_device_error_count() == 0


def test_results_are_reproducible_run_to_run(C):
    """Forward outputs and winner indices are bitwise reproducible; gradients accumulate with atomics and
    agree to rounding."""
    c = WL.cfg2(B=2)
    x, wk, gy = c["x"].cuda(), c["w"].cuda(), c["gy"].cuda()
    a, ia = C.morpho_forward("erosion", x, wk, "max", "replicate", with_index=True)
    b, ib = C.morpho_forward("erosion", x, wk, "max", "replicate", with_index=True)
    assert torch.equal(a, b) and torch.equal(ia, ib)
    g1 = C.morpho_backward("erosion", x, wk, gy, "sum", "replicate")
    g2 = C.morpho_backward("erosion", x, wk, gy, "sum", "replicate")
    # up to 32 x 25 float atomics per element, in an order that changes from run to run
    torch.testing.assert_close(g1[0], g2[0], rtol=1e-4, atol=1e-4)
    torch.testing.assert_close(g1[1], g2[1], rtol=1e-4, atol=1e-2)

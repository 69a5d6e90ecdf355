"""The index arithmetic of the row-staged tcgen05 kernels, restated in NumPy and checked against the
oracle on the CPU.  A convolution with stride 1 and "same" padding is computed the way
`csrc/tc_conv_rows.cuh` does it: image rows padded to Wp = W + 2*PW pixels are laid end to end with
PH zero rows after every image; a tile is 128 consecutive positions of that padded linear space; the
rows a tile needs are staged once (rows outside the image are zeros, as the copy engine fills them)
and every filter tap reads the same staged buffer at an offset of whole pixels.  The weight gradient
uses the same space with the position as reduction index and groups of four horizontal taps.  These
tests pin the formulas (first staged row, number of staged rows, tap offsets, which positions are
real pixels) for shapes the GPU tests do not all cover."""
import numpy as np
import pytest

from oracle import ops as O

TILE = 128


def _stage_rows(x_nhwc, v_lo, nr, hv, pw):
    """Rows v_lo .. v_lo+nr-1 of the virtual row space (image n = v // hv, row h = v % hv), each padded
    by pw zero pixels on both sides; rows with h >= H or outside the batch are zeros."""
    n, h, w, c = x_nhwc.shape
    wp = w + 2 * pw
    buf = np.zeros((nr * wp, c), x_nhwc.dtype)
    for r in range(nr):
        v = v_lo + r
        img, row = (v // hv, v % hv) if v >= 0 else (-1, v + hv)
        if 0 <= img < n and row < h:
            buf[r * wp + pw: r * wp + pw + w] = x_nhwc[img, row]
    return buf


def _row_staged_conv(x, wt, ph, pw, tiles_per_item=1):
    n, cin, h, w = x.shape
    cout, _, kh, kw = wt.shape
    xn = np.ascontiguousarray(x.transpose(0, 2, 3, 1)).astype(np.float64)
    wp, hv = w + 2 * pw, h + ph
    q_total = n * hv * wp
    span = TILE * tiles_per_item
    out = np.zeros((n, h, w, cout))
    for q0 in range(0, q_total, span):
        v_lo = q0 // wp - ph
        nr = (q0 + span - 1) // wp + ph - v_lo + 1
        assert nr <= (wp - 1 + span - 1) // wp + 1 + 2 * ph          # what the stage is sized for
        buf = _stage_rows(xn, v_lo, nr, hv, pw)
        col = q0 % wp
        acc = np.zeros((span, cout))
        for a in range(kh):
            for b in range(kw):
                start = col + a * wp + b - pw                          # the descriptor's first staged pixel
                assert start >= -pw and start + span <= nr * wp + pw  # stays inside the stage's lead / tail
                lo, hi = max(start, 0), min(start + span, nr * wp)
                rows = np.zeros((span, cin))
                rows[lo - start: hi - start] = buf[lo:hi]
                acc += rows @ wt[:, :, a, b].T.astype(np.float64)
        for m in range(span):
            q = q0 + m
            v, wpos = divmod(q, wp)
            img, row = divmod(v, hv)
            if q < q_total and row < h and pw <= wpos < w + pw:
                out[img, row, wpos - pw] = acc[m]
    return out.transpose(0, 3, 1, 2)


@pytest.mark.parametrize("cfg", [(2, 3, 5, 7, 4, 3, 3), (1, 2, 32, 32, 3, 3, 3), (3, 2, 9, 11, 2, 5, 3), (2, 1, 16, 16, 2, 1, 7), (2, 2, 6, 130, 2, 3, 3)])
@pytest.mark.parametrize("tiles_per_item", [1, 2])
def test_forward_through_staged_rows_matches_oracle(cfg, tiles_per_item):
    n, cin, h, w, cout, kh, kw = cfg
    rng = np.random.default_rng(sum(cfg))
    x = rng.standard_normal((n, cin, h, w)).astype(np.float32)
    wt = rng.standard_normal((cout, cin, kh, kw)).astype(np.float32)
    ph, pw = kh // 2, kw // 2
    got = _row_staged_conv(x, wt, ph, pw, tiles_per_item)
    want = O.conv2d_forward(x, wt, None, (1, 1), (ph, pw))
    assert np.allclose(got, want, rtol=1e-5, atol=1e-5)


@pytest.mark.parametrize("cfg", [(2, 3, 5, 7, 4, 3, 3), (1, 2, 20, 36, 3, 5, 5), (2, 2, 9, 11, 2, 3, 7)])
def test_data_gradient_is_the_same_walk_with_mirrored_taps(cfg):
    n, cin, h, w, cout, kh, kw = cfg
    rng = np.random.default_rng(sum(cfg) + 1)
    x = rng.standard_normal((n, cin, h, w)).astype(np.float32)
    wt = rng.standard_normal((cout, cin, kh, kw)).astype(np.float32)
    dy = rng.standard_normal((n, cout, h, w)).astype(np.float32)
    ph, pw = kh // 2, kw // 2
    # dX = dY convolved with the filter rotated by 180 degrees, input and output channels swapped
    mirrored = np.ascontiguousarray(wt[:, :, ::-1, ::-1].transpose(1, 0, 2, 3))
    got = _row_staged_conv(dy, mirrored, ph, pw)
    want = O.conv2d_backward(dy, x, wt, False, (1, 1), (ph, pw))[0]
    assert np.allclose(got, want, rtol=1e-5, atol=1e-5)


@pytest.mark.parametrize("cfg", [(2, 3, 5, 7, 4, 3, 3), (1, 2, 20, 36, 3, 5, 5), (3, 2, 9, 11, 2, 3, 7), (1, 1, 32, 32, 2, 3, 1)])
def test_weight_gradient_through_staged_panels_matches_oracle(cfg):
    """K = positions in blocks of 128; X rows v0-PH .. and dY rows v0 .. staged per block; one 'MMA' covers
    four horizontal taps (kw = 4g .. 4g+3) of one filter row, taps beyond the filter are dropped."""
    n, cin, h, w, cout, kh, kw = cfg
    rng = np.random.default_rng(sum(cfg) + 2)
    x = rng.standard_normal((n, cin, h, w)).astype(np.float32)
    dy = rng.standard_normal((n, cout, h, w)).astype(np.float32)
    ph, pw = kh // 2, kw // 2
    xn = np.ascontiguousarray(x.transpose(0, 2, 3, 1)).astype(np.float64)
    dn = np.ascontiguousarray(dy.transpose(0, 2, 3, 1)).astype(np.float64)
    wp, hv = w + 2 * pw, h + ph
    q_total = n * hv * wp
    groups = (kw + 3) // 4
    acc = np.zeros((kh, groups, 4, cin, cout))
    for q0 in range(0, q_total, TILE):
        v0 = q0 // wp
        nr_y = (q0 + TILE - 1) // wp - v0 + 1
        nr_x = nr_y + 2 * ph
        xb = _stage_rows(xn, v0 - ph, nr_x, hv, pw)
        yb = _stage_rows(dn, v0, nr_y, hv, pw)        # same padding: padding positions carry zero gradient
        col = q0 % wp
        ypart = yb[col: col + TILE]
        assert ypart.shape[0] == TILE                 # the dY rows always cover the block
        for a in range(kh):
            for g in range(groups):
                for j in range(4):
                    start = col + a * wp + 4 * g + j - pw
                    assert start >= -pw and start + TILE <= nr_x * wp + 16   # inside the panel's lead / tail
                    lo, hi = max(start, 0), min(start + TILE, nr_x * wp)
                    rows = np.zeros((TILE, cin))
                    rows[lo - start: hi - start] = xb[lo:hi]
                    acc[a, g, j] += rows.T @ ypart
    got = np.zeros((cout, cin, kh, kw))
    for a in range(kh):
        for b in range(kw):
            got[:, :, a, b] = acc[a, b // 4, b % 4].T
    want = O.conv2d_backward(dy, x, np.zeros((cout, cin, kh, kw), np.float32), False, (1, 1), (ph, pw))[1]
    assert np.allclose(got, want, rtol=1e-5, atol=1e-4)

"""The randn oracle on the host: Philox4x32-10 against the published known-answer vectors, the output layout of the
reference's kernel (``src/quark/kernels/randn/kernel.py:200-254``) as shift properties, and the moments."""

import numpy as np

from oracle import ops

# counter, key, output: the known-answer vectors shipped with the Philox authors' implementation
KAT = [
    ((0, 0, 0, 0), (0, 0), (0x6627E8D5, 0xE169C58D, 0xBC57AC4C, 0x9B00DBD8)),
    ((0xFFFFFFFF,) * 4, (0xFFFFFFFF,) * 2, (0x408F276D, 0x41C83B0E, 0xA20BC7C6, 0x6D5451FD)),
    ((0x243F6A88, 0x85A308D3, 0x13198A2E, 0x03707344), (0xA4093822, 0x299F31D0), (0xD16CFE09, 0x94FDCCEB, 0x5001E420, 0x24126EA1)),
]


def test_philox_known_answers():
    for ctr, key, want in KAT:
        got = ops.philox4x32_10(np.array(ctr, np.uint32), np.array(key, np.uint32))
        assert tuple(int(x) for x in got) == want
    # vectorised over a leading axis
    got = ops.philox4x32_10(np.array([k[0] for k in KAT], np.uint32), np.array([k[1] for k in KAT], np.uint32))
    assert [tuple(int(x) for x in row) for row in got] == [k[2] for k in KAT]


def test_layout_and_counter_arithmetic():
    a = ops.randn(3 * 2048, 0)
    # a block uses 512 consecutive counters: moving the offset by 512 moves the stream by one block
    np.testing.assert_array_equal(ops.randn(2 * 2048, 512), a[2048:])
    # ... and by 128 moves it by one pass of a block: 4 x 128 values further on
    b = ops.randn(2048, 128)
    np.testing.assert_array_equal(b[: 3 * 512], a[512:2048])
    # the stride multiplies the offset; the reference's meaning is stride 1
    np.testing.assert_array_equal(ops.randn(2048, 2, counter_stride=256), a[2048:4096])
    # ragged length: a prefix of the padded draw
    np.testing.assert_array_equal(ops.randn(1000, 0), a[:1000])
    # thread t of pass g writes its four normals 128 apart: element 0 and 128 come from the same Philox call
    w = ops.philox4x32_10(np.array([0, 0, 0xDEADBEEF, 0xBADC0FFE], np.uint32), np.array([0xDEADBEEF, 0xBADC0FFE], np.uint32))
    u = (w >> 8).astype(np.float32) * np.float32(2.0**-24) + np.float32(2.0**-25)
    r = np.sqrt(-2.0 * np.log(np.float64(u[0])))
    np.testing.assert_allclose([a[0], a[128]], [r * np.cos(2 * np.pi * np.float64(u[1])), r * np.sin(2 * np.pi * np.float64(u[1]))], rtol=1e-5, atol=1e-6)
    # other seeds, another stream
    assert not np.array_equal(ops.randn(2048, 0, seed0=1), a[:2048])


def test_moments_and_range():
    z = ops.randn(1 << 18, 7)
    assert abs(float(z.mean())) < 0.01 and abs(float(z.std()) - 1.0) < 0.01
    assert abs(float((z**3).mean())) < 0.03 and abs(float((z**4).mean()) - 3.0) < 0.06
    assert np.all(np.isfinite(z)) and float(np.abs(z).max()) < 5.9  # sqrt(-2 ln 2^-25) = 5.887
    zb = ops.randn(4096, 7, dtype="bf16")
    assert zb.dtype == np.uint16 and zb.shape == (4096,)

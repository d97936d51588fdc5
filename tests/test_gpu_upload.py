"""Weight upload with the ggml -> device-regions permutation done on the device (ac_b200_weight_upload): the regions
must hold exactly the bytes the CPU codec produces, so the read-back guarantee of the reference
(tests/ameva_qmm_check.cpp:184-196: get_tensor returns the uploaded bytes) is unchanged."""
import time

import numpy as np
import pytest

from conftest import load_pkg
from helpers import I2_S, Q4_0, Q4_K, Q8_0, make_weights

pytestmark = pytest.mark.gpu
pkg = load_pkg()
rt, qmm = pkg.runtime, pkg.qmm


@pytest.fixture(scope="module")
def ctx():
    c = rt.init()
    yield c
    c.destroy()


@pytest.mark.parametrize("t,N,K", [(Q4_0, 5, 96), (Q4_0, 4096, 4096), (Q8_0, 3, 32), (Q8_0, 257, 1024), (Q4_K, 1, 256),
                                   (Q4_K, 300, 2048), (Q8_0, 11008, 4096), (Q4_K, 28672, 8192), (I2_S, 640, 2560)])
def test_device_repack_leaves_the_bytes_of_the_cpu_codec(ctx, t, N, K):
    """Tiny and ragged tensors (fewer blocks than one tile of the kernel, a last tile that is not full), tensors of one
    staging chunk and of several (47.9 MB and 132 MB of ggml blocks against 32 MB chunks), and the dense I2_S copy."""
    blocks, _ = make_weights(t, N, K, N + K)
    blocks = np.ascontiguousarray(blocks, np.uint8).reshape(-1)
    total, s_off = rt.device_layout(t, N, K)
    want = rt.repack_to_device(t, blocks, N, K)
    pad = 4096                      # the tensor sits at an offset inside a larger buffer whose other bytes must survive
    buf = ctx.buffer(pad + total + 128)
    buf.fill(0xA5)
    t0 = time.perf_counter()
    buf.upload_weight(t, blocks, N, K, offset=pad)
    dt = time.perf_counter() - t0
    got = buf.read(np.uint8, total, pad)
    nblk = N * K // (256 if t == Q4_K else 32) if t != I2_S else 0
    if t != I2_S:   # the padding between the payload and the scale regions is not written by either path
        q_end = nblk * {Q4_0: 16, Q8_0: 32, Q4_K: 128}[t]
        assert np.array_equal(got[:q_end], want[:q_end])
        assert np.array_equal(got[s_off:], want[s_off:])
        assert (got[q_end:s_off] == 0xA5).all()
    else:
        assert np.array_equal(got, want)
    assert (buf.read(np.uint8, pad, 0) == 0xA5).all() and (buf.read(np.uint8, 128, pad + total) == 0xA5).all()
    if blocks.size > (8 << 20):
        print(f"upload of {blocks.size / 1e6:.1f} MB of ggml blocks ({qmm.TYPE_NAMES.get(t, t)}): {blocks.size / dt / 1e9:.2f} GB/s "
              f"end to end from pageable host memory")
    buf.destroy()
    # and through the weight object: read-back returns the uploaded blocks, whole and as a row range
    w = qmm.QuantWeight.from_ggml(ctx, t, blocks, N, K)
    assert np.array_equal(w.to_ggml(), blocks)
    if N >= 3:
        per_row = blocks.size // N
        assert np.array_equal(w.to_ggml(1, 2), blocks[per_row:3 * per_row])
    w.destroy()


def test_upload_argument_checks(ctx):
    blocks, _ = make_weights(Q4_0, 8, 256, 1)
    blocks = np.ascontiguousarray(blocks, np.uint8).reshape(-1)
    total, _ = rt.device_layout(Q4_0, 8, 256)
    buf = ctx.buffer(total + 64)
    with pytest.raises(rt.AmevaComputeError) as e:
        buf.upload_weight(Q4_0, blocks, 8, 256, offset=32)
    assert e.value.code == rt.AC_ERR_BUFFER_ALIGNMENT_INVALID
    with pytest.raises(rt.AmevaComputeError) as e:
        buf.upload_weight(Q4_0, blocks, 8, 256, offset=128)          # does not fit behind the offset
    assert e.value.code == rt.AC_ERR_INVALID_BUFFER_SIZE
    with pytest.raises(rt.AmevaComputeError) as e:
        buf.upload_weight(Q4_0, blocks, 8, 250)                       # K is not whole blocks
    assert e.value.code == rt.AC_ERR_INVALID_SHAPE
    with pytest.raises(rt.AmevaComputeError):
        buf.upload_weight(14, blocks, 8, 256)                         # a type outside the path
    buf.destroy()

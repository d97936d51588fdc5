"""Index arithmetic of the streamed GEMV's shared-memory reads (csrc/gemv_bulk.cu), restated on the CPU.

The kernel stages the int8 activations with their 16-byte pieces permuted (piece p stored at p ^ ((p >> 3) & 3)) and lets
the upper four lanes of every eight read the two halves of their 32-byte weight chunk in the opposite order. These tests
check, for every lane and loop iteration, that (a) each lane still multiplies the weight bytes with the activations that
belong to them, and (b) every 128-bit shared-memory load phase (eight consecutive lanes) touches eight different 16-byte
bank groups, i.e. is free of bank conflicts."""
import numpy as np
import pytest


def swz_piece(p):
    return p ^ ((p >> 3) & 3)


def lane_consts(lane):
    h, sw = (lane >> 2) & 1, (lane >> 1) & 3
    return h, sw, (16 * h, 16 * (h ^ 1)), [16 * ((i ^ h) ^ sw) for i in range(4)]


@pytest.mark.parametrize("K,M", [(256, 1), (4096, 3), (8192, 8), (2304 * 4, 2)])
def test_q4k_lane_reads_its_own_activations(K, M):
    stride = (K + 511) & ~511                      # staged row pitch: the permutation is per 512 bytes
    act = np.arange(M * K, dtype=np.int64).reshape(M, K)           # element id stands for the int8 value
    staged = np.full(M * stride, -1, np.int64)
    for m in range(M):
        for w in range(K // 16):                   # the staging loop of the kernel
            dst = swz_piece(m * (stride // 16) + w)
            staged[16 * dst:16 * dst + 16] = act[m, 16 * w:16 * w + 16]
    C = K // 64
    for lane in range(32):
        h, sw, (wo0, wo1), ao = lane_consts(lane)
        for c in range(lane, C, 32):
            assert (c >> 2) & 1 == h and (c >> 1) & 3 == sw        # loop-invariant per lane, as the kernel assumes
            for m in range(M):
                base = m * stride + 64 * c
                A = [staged[base + ao[i]:base + ao[i] + 16] for i in range(4)]
                # x0 = half h of the chunk (weights 16h..16h+15 of each sub-block), x1 = the other half.
                # dlo pairs (x0 & 15) with A0 and (x1 & 15) with A1; dhi pairs (x0 >> 4) with A2 and (x1 >> 4) with A3.
                want = act[m, 64 * c:64 * c + 64]
                lo, hi = want[:32], want[32:]                      # sub-block 2k, sub-block 2k+1
                assert np.array_equal(A[0], lo[16 * h:16 * h + 16])
                assert np.array_equal(A[1], lo[16 * (h ^ 1):16 * (h ^ 1) + 16])
                assert np.array_equal(A[2], hi[16 * h:16 * h + 16])
                assert np.array_equal(A[3], hi[16 * (h ^ 1):16 * (h ^ 1) + 16])


def bank_groups(addresses):
    return [(a // 16) % 8 for a in addresses]


def test_q4k_loads_are_bank_conflict_free():
    for first_lane in range(0, 32, 8):             # a 128-bit load is served eight lanes at a time
        lanes = range(first_lane, first_lane + 8)
        for it in range(4):
            cs = [lane + 32 * it for lane in lanes]
            for which in range(2):                 # the two weight halves
                addrs = [32 * c + lane_consts(lane)[2][which] for c, lane in zip(cs, lanes)]
                assert len(set(bank_groups(addrs))) == 8
            for i in range(4):                     # the four activation pieces
                addrs = [64 * c + lane_consts(lane)[3][i] for c, lane in zip(cs, lanes)]
                assert len(set(bank_groups(addrs))) == 8
    # for contrast: the straightforward order collides (each phase hits four bank groups twice / two groups four times)
    assert len(set(bank_groups([32 * c for c in range(8)]))) == 4
    assert len(set(bank_groups([64 * c for c in range(8)]))) == 2


def test_per32_types_read_permuted_activations_without_conflicts():
    """Q4_0 / Q8_0: lane u reads the 32 activation bytes of unit u as pieces 2u and 2u+1 through the permutation."""
    for first in range(0, 32, 8):
        for half in range(2):
            addrs = [16 * swz_piece(2 * u + half) for u in range(first, first + 8)]
            assert len(set(bank_groups(addrs))) == 8
    # and the permutation is a bijection inside every 64 bytes, so every piece is still found
    for base in range(0, 1024, 4):
        assert sorted(swz_piece(base + i) for i in range(4)) == [base + i for i in range(4)]

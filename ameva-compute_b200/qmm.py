"""Host side of the quantized MUL_MAT path: weight upload into the device layout, the shape contract, the choice of
kernel by M, and the dispatch sequence (activation quantize -> GEMV / GEMM) recorded into an ac_runtime batch.

Mirrors, for this path only, what the reference's ggml plugin does on the host
(adapters/llama/ggml-ameva/ggml-ameva.cpp: ``mul_mat_qmm_reason`` :1326-1377, ``ameva_mmq_plan`` :2486-2503,
``enc_mul_mat`` :3607-3804, ``enc_mul_mat_mmq`` :2540, ``enc_mul_mat_mmvq`` :2704; weight repack on upload,
ggml-ameva-buffer.cpp:300-330, 390-416) and the BitNet engine's ``RecordNormQ8`` / ``RecordGemv``
(adapters/bitnet/src/core/ac_bitnet_engine.cpp:253-288). Anything the kernels cannot run is refused with a reason
(``MulMatUnsupported``): there is no CPU path behind this module.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import numpy as np

from . import runtime as rt

GGML_TYPE_Q4_0, GGML_TYPE_Q8_0, GGML_TYPE_Q4_K, GGML_TYPE_I2_S = 2, 8, 12, 36
# kept on the device as Q8_0 regions: d * (q5 - 16) and d * kvalues_iq4nl[q4] are d * int8 (registry.cu, decode_block)
GGML_TYPE_Q5_0, GGML_TYPE_IQ4_NL = 6, 20
DEVICE_TYPE = {GGML_TYPE_Q5_0: GGML_TYPE_Q8_0, GGML_TYPE_IQ4_NL: GGML_TYPE_Q8_0}
# Q6_K: the 6-bit weights decoded to int8 at upload (256 payload bytes per block), scales[16] + d kept (18 bytes); one
# kernel, ameva_mmvqb_q6_K, over Q8_K activations (gemv_q6k.cu); more than 8 activation rows: ameva_mmtc_b8
GGML_TYPE_Q6_K = 14
# Q5_K likewise: q5 decoded to bytes (256 per block), the block's first 16 bytes (d, dmin, packed scales) kept as the
# scale record; ameva_mmvqb_q5_K
GGML_TYPE_Q5_K = 13
# IQ4_XS: kvalues_iq4nl[q4] decoded to int8, the block's first 8 bytes (d, scales_h, scales_l) kept; ameva_mmvqb_iq4_xs
GGML_TYPE_IQ4_XS = 23
# Q4_1 / Q5_1 (d * q + m per 32): q decoded to bytes, (d, m) kept as a 4-byte record; ameva_mmvq_q4_1 / _q5_1 over the
# per-32 activations (whose records carry the sum of q8 the m term needs)
GGML_TYPE_Q4_1, GGML_TYPE_Q5_1 = 3, 7
# Q3_K / Q2_K: q3 (-4..3) / q2 (0..3) decoded to bytes; scales[12] + d (14 bytes) / scales[16], d, dmin (20 bytes) kept;
# ameva_mmvqb_q3_K / _q2_K
GGML_TYPE_Q2_K, GGML_TYPE_Q3_K = 10, 11
BYTE_DECODED = (GGML_TYPE_Q6_K, GGML_TYPE_Q5_K, GGML_TYPE_IQ4_XS, GGML_TYPE_Q4_1, GGML_TYPE_Q5_1, GGML_TYPE_Q3_K,
                GGML_TYPE_Q2_K)   # one GEMV kernel each, one tensor-core kernel for all (ameva_mmtc_b8), no fused variants
BYTE_SIGNED = (GGML_TYPE_Q6_K, GGML_TYPE_IQ4_XS, GGML_TYPE_Q3_K)   # payload bytes are int8 (the others: 0..255)
TYPE_NAMES = {GGML_TYPE_Q4_0: "q4_0", GGML_TYPE_Q8_0: "q8_0", GGML_TYPE_Q4_K: "q4_K", GGML_TYPE_I2_S: "i2_s",
              GGML_TYPE_Q6_K: "q6_K", GGML_TYPE_Q5_K: "q5_K", GGML_TYPE_IQ4_XS: "iq4_xs", GGML_TYPE_Q4_1: "q4_1",
              GGML_TYPE_Q5_1: "q5_1", GGML_TYPE_Q3_K: "q3_K", GGML_TYPE_Q2_K: "q2_K"}
BLOCK = {GGML_TYPE_Q4_0: 32, GGML_TYPE_Q8_0: 32, GGML_TYPE_Q4_K: 256, GGML_TYPE_I2_S: 128, GGML_TYPE_Q6_K: 256,
         GGML_TYPE_Q5_K: 256, GGML_TYPE_IQ4_XS: 256, GGML_TYPE_Q4_1: 32, GGML_TYPE_Q5_1: 32, GGML_TYPE_Q3_K: 256,
         GGML_TYPE_Q2_K: 256}
Q_BYTES = {GGML_TYPE_Q4_0: 16, GGML_TYPE_Q8_0: 32, GGML_TYPE_Q4_K: 128, GGML_TYPE_Q6_K: 256, GGML_TYPE_Q5_K: 256,
           GGML_TYPE_IQ4_XS: 256, GGML_TYPE_Q4_1: 32, GGML_TYPE_Q5_1: 32, GGML_TYPE_Q3_K: 256,
           GGML_TYPE_Q2_K: 256}   # payload bytes per block
S_BYTES = {GGML_TYPE_Q4_0: 2, GGML_TYPE_Q8_0: 2, GGML_TYPE_Q4_K: 16, GGML_TYPE_Q6_K: 18, GGML_TYPE_Q5_K: 16,
           GGML_TYPE_IQ4_XS: 8, GGML_TYPE_Q4_1: 4, GGML_TYPE_Q5_1: 4, GGML_TYPE_Q3_K: 14,
           GGML_TYPE_Q2_K: 20}     # scale bytes per block
PER_256 = (GGML_TYPE_Q4_K, GGML_TYPE_Q6_K, GGML_TYPE_Q5_K, GGML_TYPE_IQ4_XS, GGML_TYPE_Q3_K, GGML_TYPE_Q2_K)   # types whose activations are quantized per 256 (Q8_K records)
PER_32 = (GGML_TYPE_Q4_0, GGML_TYPE_Q8_0, GGML_TYPE_Q4_1, GGML_TYPE_Q5_1)         # per 32 (fp16 d | int16 sum per block)
FUSED_QUANT_MAX_K = 16384          # the fused kernels keep the quantized row in shared memory


def mma_gemv_fits(M: int, K: int) -> bool:
    """Q4_K, M <= 8: whether ameva_mmvm_q4_K can hold the M activation rows (plus one row of zeros), their per-block
    records, its partial sums and two ring stages per warp in 227 KB of shared memory (M = 8: K <= 14592)."""
    rows = M + 1
    return K % 256 == 0 and rows * (K + 32) + rows * (K // 256) * 20 + 16384 + 16 + 2 * 16 * 2304 <= 227 * 1024


GEMV_MAX_M = 8   # decode GEMV serves M <= 8 (ggml-ameva.cpp:3607-3804 sends 2 <= M < 8 to the GEMV family as well)
AB_BYTES = 48

ROUND_NEAREST_EVEN, ROUND_TIES_AWAY = 0, 1
Q8K_GGML, Q8K_AMEVA = 0, 1


EPILOGUE_ADD, EPILOGUE_SWIGLU_GATE, EPILOGUE_SWIGLU_UP = 1, 2, 3


def plan(ggml_type: int, M: int, N: int, K: int, flags: int = 0) -> int:
    """The library's kernel choice for a shape (rt.PATH_*), or rt.PATH_NONE for a shape outside the contract. The policy
    itself lives in the C library (ac_b200_mul_mat_plan), shared with the ggml plugin."""
    try:
        return rt.mul_mat_plan(ggml_type, M, N, K, flags)
    except rt.AmevaComputeError:
        return rt.PATH_NONE


def streamed_pays(ggml_type: int, M: int, N: int, K: int) -> bool:
    """Whether the library's policy sends this decode shape to the streamed GEMV (ameva_mmvs_*)."""
    return 1 <= M <= GEMV_MAX_M and plan(ggml_type, M, N, K) == rt.PATH_GEMV_STREAMED


def weight_exponent(ggml_type: int, blocks: np.ndarray, N: int, K: int) -> int:
    """The magnitude of a weight tensor as a power of two (2^w_exp brings its largest |w| into [1, 2)), computed once per
    tensor at upload (ac_b200_weight_exponent). The tensor-core GEMM dequantizes weights to fp16: tensors whose magnitudes
    fp16 does not hold comfortably (rt.weight_range_extreme) stay on the integer kernels at every M."""
    return rt.weight_exponent(ggml_type, blocks, N, K)


class MulMatUnsupported(Exception):
    """The op is outside the contract; the message is the reason (the reference logs it once per (op, type, reason))."""


def unsupported_reason(ggml_type: int, M: int, N: int, K: int) -> Optional[str]:
    """Shape contract (mul_mat_qmm_reason, ggml-ameva.cpp:1326-1377, narrowed to the four types built here)."""
    ggml_type = DEVICE_TYPE.get(ggml_type, ggml_type)
    if ggml_type not in TYPE_NAMES:
        return f"weight type {ggml_type} not built"
    if M <= 0 or N <= 0 or K <= 0:
        return "empty operand"
    if K % BLOCK[ggml_type]:
        return f"K={K} is not a multiple of the {TYPE_NAMES[ggml_type]} block ({BLOCK[ggml_type]})"
    if K % 4 or (K * 4) % 16:
        return "activation rows must be 16-byte aligned"
    if N * K >= 2 ** 32 or M * max(N, K) >= 2 ** 32:
        return "32-bit indexing"
    return None


@dataclass
class WeightView:
    """Rows [row0, row0 + rows) of an uploaded weight (what a rank of a row-sharded projection owns)."""
    weight: "QuantWeight"
    row0: int
    rows: int


class QuantWeight:
    """A weight matrix [N][K] in the device layout. ``from_ggml`` repacks ggml blocks on upload; ``to_ggml`` returns the
    uploaded bytes exactly, whole or by row range (read-back guarantee of tests/ameva_qmm_check.cpp:184-196)."""

    def __init__(self, ctx: rt.Context, ggml_type: int, N: int, K: int, buf: rt.Buffer, s_off: int,
                 scale: float = 1.0, w_exp: int = 0) -> None:
        self.ggml_type = ggml_type                          # what was uploaded and what to_ggml returns
        ggml_type = DEVICE_TYPE.get(ggml_type, ggml_type)   # the type whose regions and kernels serve it
        self.ctx, self.type, self.N, self.K, self.buf, self.s_off, self.scale = ctx, ggml_type, N, K, buf, s_off, scale
        self.w_exp = w_exp   # see weight_exponent
        self.fp16_ok = not rt.weight_range_extreme(w_exp)

    @classmethod
    def from_ggml(cls, ctx: rt.Context, ggml_type: int, blocks: np.ndarray, N: int, K: int,
                  scale: float = 1.0, host_repack: bool = False) -> "QuantWeight":
        """Uploads ggml blocks into the device regions. The permutation runs on the device, fed from pinned staging
        chunks (ac_b200_weight_upload); host_repack=True permutes on the CPU first (ac_b200_repack_to_device) and
        writes the result, which is what a caller with its own staging does. Both leave the same bytes."""
        why = unsupported_reason(ggml_type, 1, N, K)
        if why:
            raise MulMatUnsupported(why)
        blocks = np.ascontiguousarray(blocks, dtype=np.uint8).reshape(-1)
        if blocks.size != rt.ggml_nbytes(ggml_type, N, K):
            raise MulMatUnsupported(f"expected {rt.ggml_nbytes(ggml_type, N, K)} bytes of ggml blocks, got {blocks.size}")
        total, s_off = rt.device_layout(ggml_type, N, K)
        w_exp = weight_exponent(ggml_type, blocks, N, K)
        if host_repack:
            buf = ctx.buffer(total, rt.repack_to_device(ggml_type, blocks, N, K))
        else:
            buf = ctx.buffer(total)
            try:
                buf.upload_weight(ggml_type, blocks, N, K)
            except Exception:
                buf.destroy()
                raise
        return cls(ctx, ggml_type, N, K, buf, s_off, scale, w_exp)

    def to_ggml(self, row0: int = 0, rows: Optional[int] = None) -> np.ndarray:
        rows = self.N - row0 if rows is None else rows
        nblk_row = self.K // BLOCK[self.type]
        if self.type == GGML_TYPE_I2_S:
            return self.buf.read(np.uint8, rows * self.K // 4, row0 * self.K // 4)
        qb, sb = Q_BYTES[self.type], S_BYTES[self.type]
        q = self.buf.read(np.uint8, rows * nblk_row * qb, row0 * nblk_row * qb)
        s = self.buf.read(np.uint8, rows * nblk_row * sb, self.s_off + row0 * nblk_row * sb)
        pad = (-q.size) % 64   # the codec expects the payload region padded to 64 bytes before the scales
        dev = np.concatenate([q, np.zeros(pad, np.uint8), s])
        return rt.repack_from_device(self.ggml_type, dev, rows, self.K)

    def view(self, row0: int, rows: int) -> WeightView:
        if row0 < 0 or rows <= 0 or row0 + rows > self.N:
            raise MulMatUnsupported("row range outside the weight")
        return WeightView(self, row0, rows)

    def destroy(self) -> None:
        self.buf.destroy()


def _bindings_for(view: WeightView):
    """(Q binding, S binding) of a row range; offsets must meet the runtime's 64-byte binding alignment."""
    w = view.weight
    nblk_row = w.K // BLOCK[w.type]
    if w.type == GGML_TYPE_I2_S:
        off = view.row0 * w.K // 4
        if off % 64:
            raise MulMatUnsupported("row range does not start on a 64-byte boundary")
        return (w.buf, off, view.rows * w.K // 4), None
    qb, sb = Q_BYTES[w.type], S_BYTES[w.type]
    qo, so = view.row0 * nblk_row * qb, w.s_off + view.row0 * nblk_row * sb
    if qo % 64 or so % 64:
        raise MulMatUnsupported("row range does not start on a 64-byte boundary of the payload / scale regions")
    return (w.buf, qo, view.rows * nblk_row * qb), (w.buf, so, view.rows * nblk_row * sb)


def _record_rms_norm_quantize(ctx, batch, ggml_type, M, K, x, y, aq, ad, ah, ae, mode, eps, weight, x_offset, y_offset,
                              w_offset):
    """ameva_rms_norm_quant_a8 / a8b: y = rms_norm(x) [* weight] written as f32, and y quantized into (aq, ad[, ah, ae])."""
    if ggml_type not in PER_32 and ggml_type not in PER_256:
        raise MulMatUnsupported("the fused RMS norm + quantize serves the per-32 and per-256 activation schemes")
    if K > 32768:
        raise MulMatUnsupported("the fused RMS norm + quantize keeps a row in registers: K <= 32768")
    name = "ameva_rms_norm_quant_a8b" if ggml_type in PER_256 else "ameva_rms_norm_quant_a8"
    wb = (weight, w_offset, K * 4) if weight is not None else (x, x_offset)
    write_h = ah is not None
    binds = [(x, x_offset), wb, (y, y_offset, M * K * 4), aq, ad, ah if write_h else aq, ae if write_h else aq]
    push = [M, K, K, mode, int(np.float32(eps).view(np.uint32)), 1 if weight is not None else 0, 1 if write_h else 0]
    batch.dispatch(ctx.kernel(name), binds, push, (M, 1, 1))
    batch.barrier()


class MulMat:
    """dst[M][N] (fp32) = activations[M][K] (fp32) x weight[N][K]^T for one weight (or row range) and a maximum M.

    Owns the scratch the path needs (quantized activations and their scales), sized once for ``max_m``; ``record``
    appends the dispatch sequence to a batch; ``run`` is record + submit + wait. ``path`` reports which kernels ran.
    """

    def __init__(self, ctx: rt.Context, weight, max_m: int, *, round_mode: int = ROUND_NEAREST_EVEN,
                 q8k_mode: int = Q8K_GGML, dump_block_sums: bool = False, exact: bool = False,
                 streamed: Optional[bool] = None, fused_quantize: bool = False, mma: Optional[bool] = None,
                 gemm_flags: int = 0) -> None:
        self.ctx = ctx
        # launch switches of the tensor-core GEMM (rt.GEMM_ONE_TILE_PER_UNIT for hosts that share the GPU with other
        # work, rt.GEMM_ONE_ACCUMULATOR to keep M > 256 on the kernel with one accumulator per CTA pair)
        self.gemm_flags = gemm_flags
        # M <= 8 over Q4_K: the GEMV on the warp-level integer tensor instruction (ameva_mmvm_q4_K). None = with 2..8
        # activation rows wherever they fit; True also takes a single row; False never.
        self.mma = mma
        # M <= 8: stage the weight rows in shared memory by bulk copies (ameva_mmvs_*). None = where it measures faster
        # than the register-staged kernels (see streamed_pays); True / False force the choice.
        self.streamed = streamed
        # M == 1 of a small projection: one launch that quantizes the row inside the GEMV (ameva_mmv*_fq); same bits.
        # On request: in replayed batches, where the quantize kernel's launch already overlaps (programmatic dependent
        # launch), the two kernels measure faster (5.3 vs 6.0 us on 4096 x 4096 Q4_0); it saves a host launch otherwise.
        self.fused_quantize = fused_quantize
        self.view = weight if isinstance(weight, WeightView) else weight.view(0, weight.N)
        w = self.view.weight
        why = unsupported_reason(w.type, max_m, self.view.rows, w.K)
        if why:
            raise MulMatUnsupported(why)
        self.type, self.N, self.K, self.max_m = w.type, self.view.rows, w.K, max_m
        if w.type in BYTE_DECODED and dump_block_sums:
            raise MulMatUnsupported("no kernel writes the per-block sums of a Q6_K / Q5_K product")
        self.round_mode, self.q8k_mode, self.dump = round_mode, q8k_mode, dump_block_sums
        # exact = keep every M on the dp4a kernels (exact per-block int32 sums); otherwise M > 8 runs on tensor cores,
        # unless the weights' magnitudes are outside what their fp16 form holds comfortably
        self.exact = exact or dump_block_sums or not w.fp16_ok
        # the GEMM stages weights and scales with TMA: whole 128-byte operand rows, whole 16-byte scale groups per row
        self.tc_ok = self.K % (128 if self.type == GGML_TYPE_I2_S else 256) == 0
        self.qbind, self.sbind = _bindings_for(self.view)
        K = self.K
        self.aq = ctx.buffer(max_m * K)
        if self.type in PER_32:
            self.ad = ctx.buffer(max_m * (K // 32) * 4)
        elif self.type in PER_256:
            self.ad = ctx.buffer(max_m * (K // 256) * AB_BYTES)
        else:
            self.ad = ctx.buffer(max_m * 8)
            self.y = ctx.buffer(max_m * K * 4)     # bitnet_norm_q8 writes the fp32 activations it quantized
            self.qeo = ctx.buffer(64)              # emulated-dot operand: not produced (range too small on purpose)
        self.ah = self.ae = None
        if max_m > GEMV_MAX_M and not self.exact and self.tc_ok and self.type != GGML_TYPE_I2_S:
            self.ah = ctx.buffer(max_m * K * 2)    # fp16(q * d * s_m): the activation operand of the tensor-core GEMM
            self.ae = ctx.buffer(max_m * 4)        # 1 / s_m per token row (power-of-two range factors, see act_quant.cu)
        # the byte-decoded types' GEMM reads an fp16 (scale, offset) pair per 16 weights: written once, here, from the
        # weight's scale records (64 bytes per 256 weights)
        self.h = None
        if self.ah is not None and self.type in BYTE_DECODED:
            self.h = ctx.buffer(self.N * (K // 16) * 4)
            batch = ctx.batch(4)
            try:
                batch.dispatch(ctx.kernel("ameva_mmtc_scales"), [self.sbind, self.h], [self.type, self.N, K],
                               ((self.N * (K // 256) + 255) // 256, 1, 1))
                ev = batch.submit()
                try:
                    ev.wait()
                finally:
                    ev.destroy()
            finally:
                batch.destroy()
        self.sums = None
        self.path = ""

    # -- scratch accounting (graph_compute reserves the max over nodes, ggml-ameva.cpp:5382-5422)
    def scratch_bytes(self) -> int:
        return self.aq.size_bytes + self.ad.size_bytes + (self.ah.size_bytes + self.ae.size_bytes if self.ah else 0)

    def _sum_shape(self, M: int):
        if self.type in (GGML_TYPE_Q4_0, GGML_TYPE_Q8_0):
            return (M, self.N, self.K // 32)
        if self.type == GGML_TYPE_Q4_K:
            return (M, self.N, self.K // 256, 2)
        return None

    def streamed_pays(self, M: int) -> bool:
        return streamed_pays(self.type, M, self.N, self.K)

    def record(self, batch: rt.Batch, x: rt.Buffer, dst: rt.Buffer, M: int, *, x_offset: int = 0, dst_offset: int = 0,
               dst_stride: Optional[int] = None, quantize: bool = True, peers=None, epilogue=None) -> None:
        """x: fp32 [M][K] at byte x_offset; dst: fp32 rows dst_stride floats apart at byte dst_offset.

        peers: buffers of other ranks (opened with Context.open_ipc) that receive the same output range at the same
        offset and stride: the kernel's epilogue stores every tile to the local dst and to each peer, which is the
        output exchange of a row-sharded projection fused into the mul_mat (no separate all-gather).

        epilogue: (mode, e, out) with f32 buffers of N elements, M == 1 only: besides dst the kernel writes
        out = dst + e (EPILOGUE_ADD), silu(dst) * e (EPILOGUE_SWIGLU_GATE) or silu(e) * dst (EPILOGUE_SWIGLU_UP), the
        fusion the reference's graph engine applies to token-generation MUL_MATs (ggml-ameva.cpp:2272-2279,
        4345-4378)."""
        if M <= 0 or M > self.max_m:
            raise MulMatUnsupported(f"M={M} outside 1..{self.max_m}")
        ctx, K, N = self.ctx, self.K, self.N
        dst_stride = N if dst_stride is None else dst_stride
        t = self.type
        use_tc = M > GEMV_MAX_M and not self.exact and self.tc_ok
        peers = list(peers or [])
        # One activation row of a projection small enough to be launch-bound: the GEMV quantizes the row itself (every
        # CTA repeats the quantize, so larger projections keep the separate kernel). The scratch AQ/AD stay unwritten.
        if (quantize and M == 1 and self.fused_quantize and t in (GGML_TYPE_Q4_0, GGML_TYPE_Q8_0, GGML_TYPE_Q4_K)
                and not self.dump and self.streamed is not True and not peers and epilogue is None
                and plan(t, 1, N, K, rt.PLAN_HOST_LAUNCH) == rt.PATH_GEMV_FQ and x_offset % 64 == 0
                and dst_offset % 64 == 0):
            fam = "ameva_mmvqb" if t == GGML_TYPE_Q4_K else "ameva_mmvq"
            mode = self.q8k_mode if t == GGML_TYPE_Q4_K else self.round_mode
            self.path = "mmvq-fq"
            batch.dispatch(ctx.kernel(f"{fam}_{TYPE_NAMES[t]}_fq"), [self.qbind, self.sbind, (x, x_offset), (dst, dst_offset)],
                           [N, K, mode], ((N + 15) // 16, 1, 1))
            return
        if quantize:
            if t in PER_32:
                binds = [(x, x_offset), self.aq, self.ad] + ([self.ah, self.ae] if use_tc else [])
                batch.dispatch(ctx.kernel("ameva_quant_a8_f16" if use_tc else "ameva_quant_a8"), binds,
                               [M, K, K, self.round_mode], ((M * (K // 32) * 8 + 255) // 256, 1, 1))
            elif t in PER_256:
                binds = [(x, x_offset), self.aq, self.ad] + ([self.ah, self.ae] if use_tc else [])
                batch.dispatch(ctx.kernel("ameva_quant_a8b_f16" if use_tc else "ameva_quant_a8b"), binds,
                               [M, K, K, self.q8k_mode], ((M * (K // 256) * 32 + 255) // 256, 1, 1))
            else:
                batch.dispatch(ctx.kernel("bitnet_norm_q8"),
                               [(x, x_offset), (x, x_offset), (x, x_offset), self.y, self.aq, self.ad, self.qeo],
                               [K, 0, 0, 0], (M, 1, 1))
            batch.barrier()
        if self.dump:
            shp = self._sum_shape(M)
            if shp is not None and self.sums is None:
                self.sums = ctx.buffer(int(np.prod(self._sum_shape(self.max_m))) * 4)
        # kernel choice by M (ameva_mmq_plan / enc_mul_mat): M <= 8 -> streaming GEMV; larger M -> tcgen05 GEMM; the exact
        # mode (and K that is not a whole number of 128-byte operand rows) walks larger M in chunks of 8 through the GEMV
        if len(peers) > 7:
            raise MulMatUnsupported("at most 7 peers")
        # The shared-memory-streamed GEMV carries the peer exchange for every scaled type, so it always runs with peers.
        want_streamed = self.streamed if self.streamed is not None else (self.streamed_pays(M) and epilogue is None)
        streamed = (not use_tc and M <= GEMV_MAX_M and t != GGML_TYPE_I2_S and t not in BYTE_DECODED and K % 256 == 0 and not self.dump
                    and not self.exact and (want_streamed or bool(peers)))
        if peers and not (use_tc and t != GGML_TYPE_I2_S and t not in BYTE_DECODED) and not streamed:
            raise MulMatUnsupported("the fused peer exchange is built for the tensor-core GEMM of the scaled types and "
                                    "the streamed GEMV (K a multiple of 256)")
        if use_tc:
            self.path = "mmtc"
            grid = ((M + 255) // 256, (N + 127) // 128, 1)
            if peers:
                self.path = "mmtc+peer-stores"
                outs = [(dst, dst_offset)] + [(pb, dst_offset) for pb in peers]
                outs += [(dst, dst_offset)] * (8 - len(outs))
                batch.dispatch(ctx.kernel(f"ameva_mmtc_{TYPE_NAMES[t]}_mp"), [self.qbind, self.sbind, self.ah] + outs + [self.ae],
                               [M, N, K, dst_stride, self.gemm_flags, len(peers)], grid)
                return
            if t in BYTE_DECODED:
                batch.dispatch(ctx.kernel("ameva_mmtc_b8"), [self.qbind, self.h, self.ah, (dst, dst_offset), self.ae],
                               [M, N, K, dst_stride, self.gemm_flags, 1 if t in BYTE_SIGNED else 0], grid)
            elif t == GGML_TYPE_I2_S:
                push = [M, N, K, dst_stride, int(np.float32(self.view.weight.scale).view(np.uint32))]
                batch.dispatch(ctx.kernel("bitnet_gemm_i2_s"), [self.qbind, self.aq, (dst, dst_offset), self.ad], push,
                               grid)
            else:
                batch.dispatch(ctx.kernel(f"ameva_mmtc_{TYPE_NAMES[t]}"),
                               [self.qbind, self.sbind, self.ah, (dst, dst_offset), self.ae],
                               [M, N, K, dst_stride, self.gemm_flags], grid)
            return
        if epilogue is not None and (M != 1 or t == GGML_TYPE_I2_S or t in BYTE_DECODED or self.dump or peers):
            raise MulMatUnsupported("the fused epilogue is built for one activation row of a Q4_0 / Q8_0 / Q4_K product")
        use_mma = (t == GGML_TYPE_Q4_K and 1 <= M <= GEMV_MAX_M and mma_gemv_fits(M, K) and not self.dump and not peers
                   and epilogue is None and self.streamed is not True
                   and (self.mma is True or (self.mma is None and plan(t, M, N, K) == rt.PATH_GEMV_MMA)))
        if self.mma is True and not use_mma and not use_tc:
            raise MulMatUnsupported("ameva_mmvm_q4_K serves Q4_K with up to 8 activation rows that fit shared memory")
        if use_mma and not use_tc:
            self.path = "mmvm"
            batch.dispatch(ctx.kernel("ameva_mmvm_q4_K"), [self.qbind, self.sbind, self.aq, self.ad, (dst, dst_offset)],
                           [M, N, K, dst_stride], ((N + 15) // 16, 1, 1))
            return
        if streamed and epilogue is None:
            # weight rows staged in shared memory by bulk copies, several stages ahead of the dot products; also carries
            # the output exchange of a row-sharded projection (every output row stored to every rank)
            self.path = "mmvs+peer-stores" if peers else "mmvs"
            outs = [(dst, dst_offset)] + [(pb, dst_offset) for pb in peers]
            outs += [(dst, dst_offset)] * (8 - len(outs))
            batch.dispatch(ctx.kernel(f"ameva_mmvs_{TYPE_NAMES[t]}"), [self.qbind, self.sbind, self.aq, self.ad] + outs,
                           [M, N, K, dst_stride, len(peers), 0], ((N + 15) // 16, 1, 1))
            return
        self.path = "mmvq" if M <= GEMV_MAX_M else "mmvq-chunks"
        for m0 in range(0, M, GEMV_MAX_M):
            mc = min(GEMV_MAX_M, M - m0)
            d_off = dst_offset + m0 * dst_stride * 4
            if t == GGML_TYPE_I2_S:
                name = "bitnet_gemv_i2_s_l32w1"
                push = [K, N, int(np.float32(self.view.weight.scale).view(np.uint32)), 0, mc, dst_stride]
                binds = [self.qbind, (self.aq, m0 * K), (dst, d_off), (self.ad, m0 * 8)]
            else:
                fam = "ameva_mmvqb" if t in PER_256 else "ameva_mmvq"
                name = f"{fam}_{TYPE_NAMES[t]}" + ("_dump" if self.dump else "")
                push = [mc, N, K, dst_stride]
                per_row = (K // 32) * 4 if t not in PER_256 else (K // 256) * AB_BYTES
                binds = [self.qbind, self.sbind, (self.aq, m0 * K), (self.ad, m0 * per_row), (dst, d_off)]
                if self.dump:
                    per_m = int(np.prod(self._sum_shape(1))) * 4
                    binds.append((self.sums, m0 * per_m))
                if epilogue is not None:
                    mode, e_buf, out_buf = epilogue
                    name += "_ep"
                    binds += [e_buf, out_buf]
                    push = push + [int(mode)]
            for b in binds:
                if isinstance(b, tuple) and b[1] % 64:
                    raise MulMatUnsupported(f"binding offset {b[1]} of {name} is not 64-byte aligned")
            batch.dispatch(ctx.kernel(name), binds, push, ((N + 15) // 16, 1, 1))

    def run(self, x: rt.Buffer, dst: rt.Buffer, M: int, **kw) -> float:
        """Record, submit, wait. Returns the GPU time of the batch in microseconds."""
        batch = self.ctx.batch(64 + (M + GEMV_MAX_M - 1) // GEMV_MAX_M)   # (the exact path walks M in chunks of 8 rows)
        try:
            self.record(batch, x, dst, M, **kw)
            ev = batch.submit()
            try:
                ev.wait()
                return ev.gpu_duration_us()
            finally:
                ev.destroy()
        finally:
            batch.destroy()

    def read_block_sums(self, M: int) -> np.ndarray:
        shp = self._sum_shape(M)
        return self.sums.read(np.int32, int(np.prod(shp))).reshape(shp)

    def record_rms_norm_quantize(self, batch: rt.Batch, x: rt.Buffer, y: rt.Buffer, M: int, *, eps: float,
                                 weight: Optional[rt.Buffer] = None, x_offset: int = 0, y_offset: int = 0,
                                 w_offset: int = 0) -> None:
        """RMS norm of M rows of x (times the weight row, if given) written to y, and y quantized into this product's
        scratch by the same kernel: follow with ``record(batch, y, dst, M, quantize=False)``. Replaces RMS_NORM (+ MUL)
        and the quantize kernel of the MUL_MAT that consumes the result (three launches become one)."""
        use_tc = M > GEMV_MAX_M and not self.exact and self.tc_ok
        mode = self.q8k_mode if self.type in PER_256 else self.round_mode
        _record_rms_norm_quantize(self.ctx, batch, self.type, M, self.K, x, y, self.aq, self.ad,
                                  self.ah if use_tc else None, self.ae if use_tc else None, mode, eps, weight, x_offset,
                                  y_offset, w_offset)

    def read_quantized(self, M: int):
        """The activation scratch of the last run, in oracle-comparable form."""
        K = self.K
        q = self.aq.read(np.int8, M * K).reshape(M, K)
        if self.type in PER_32:
            ad = self.ad.read(np.uint32, M * (K // 32)).reshape(M, K // 32)
            return q, (ad & 0xFFFF).astype(np.uint16), (ad >> 16).astype(np.uint16).view(np.int16)
        if self.type in PER_256:
            ab = self.ad.read(np.uint8, M * (K // 256) * AB_BYTES).reshape(M, K // 256, AB_BYTES)
            bsums = np.ascontiguousarray(ab[:, :, :32]).view(np.int16)
            d = np.ascontiguousarray(ab[:, :, 32:36]).view(np.float32)[..., 0]
            return q, d, bsums
        act = self.ad.read(np.uint32, M * 2).reshape(M, 2)
        return q, act[:, 0].copy().view(np.float32), act[:, 1].copy().view(np.int32)

    def destroy(self) -> None:
        for name in ("aq", "ad", "ah", "ae", "h", "y", "qeo", "sums"):
            b = getattr(self, name, None)
            if b is not None:
                b.destroy()


class MulMatGroup:
    """One activation row against several weight matrices that share it (the q / k / v or the gate / up projections of a
    decoder layer), as ONE launch, every output bit-equal to the separate launches. The reference quantizes such a shared
    src1 once and reuses it (adapters/llama/ggml-ameva/ggml-ameva.cpp:2154-2158, 2738-2749); on B200 the launches
    themselves are what a small projection pays for, so they are merged too. fused_quantize=True: the row is quantized
    by every CTA inside that launch (one launch in all, K <= FUSED_QUANT_MAX_K: for hosts that launch kernel by kernel);
    False: the quantize kernel runs once before it (faster on the device, any K). Up to four matrices of one type and K,
    every N a multiple of 2; anything else is refused (callers fall back to one MulMat per matrix)."""

    def __init__(self, ctx: rt.Context, weights, *, round_mode: int = ROUND_NEAREST_EVEN, q8k_mode: int = Q8K_GGML,
                 fused_quantize: bool = True) -> None:
        views = [w if isinstance(w, WeightView) else w.view(0, w.N) for w in weights]
        if not 1 <= len(views) <= 4:
            raise MulMatUnsupported("a group holds one to four weight matrices")
        t, K = views[0].weight.type, views[0].weight.K
        if t not in (GGML_TYPE_Q4_0, GGML_TYPE_Q8_0, GGML_TYPE_Q4_K):
            raise MulMatUnsupported("grouped launches are built for Q4_0 / Q8_0 / Q4_K")
        for v in views:
            if v.weight.type != t or v.weight.K != K:
                raise MulMatUnsupported("the matrices of a group share the type and K")
            why = unsupported_reason(t, 1, v.rows, K)
            if why:
                raise MulMatUnsupported(why)
            if v.rows % 2:
                raise MulMatUnsupported("grouped launches need an even number of weight rows per matrix")
        if fused_quantize and K > FUSED_QUANT_MAX_K:
            raise MulMatUnsupported(f"K={K} above {FUSED_QUANT_MAX_K}: the quantized row does not fit shared memory")
        self.ctx, self.type, self.K, self.views = ctx, t, K, views
        self.mode = q8k_mode if t == GGML_TYPE_Q4_K else round_mode
        self.binds = [_bindings_for(v) for v in views]
        self.fq = fused_quantize
        self.path = "mmvqg-fq" if fused_quantize else "mmvqg"
        self.aq = self.ad = None
        if not fused_quantize:
            self.aq = ctx.buffer(K)
            self.ad = ctx.buffer((K // 256) * AB_BYTES if t == GGML_TYPE_Q4_K else (K // 32) * 4)

    def record(self, batch: rt.Batch, x: rt.Buffer, dsts, *, x_offset: int = 0, dst_offsets=None,
               quantize: bool = True) -> None:
        """x: fp32 [K] at byte x_offset (64-byte aligned); dsts[j]: fp32 [N_j] at byte dst_offsets[j]. quantize=False
        (two-kernel form only) reuses the row quantized by the previous record."""
        if len(dsts) != len(self.views):
            raise MulMatUnsupported("one destination per matrix")
        offs = list(dst_offsets or [0] * len(dsts))
        if x_offset % 64 or any(o % 64 for o in offs):
            raise MulMatUnsupported("binding offsets must be 64-byte aligned")
        binds = []
        for j in range(4):
            jj = j if j < len(self.views) else 0
            q, s_ = self.binds[jj]
            binds += [q, s_, (dsts[jj], offs[jj], self.views[jj].rows * 4)]
        ns = [v.rows for v in self.views] + [0] * (4 - len(self.views))
        fam = "ameva_mmvqgb" if self.type == GGML_TYPE_Q4_K else "ameva_mmvqg"
        total = sum(v.rows for v in self.views)
        if self.fq:
            binds.append((x, x_offset, self.K * 4))
            batch.dispatch(self.ctx.kernel(f"{fam}_{TYPE_NAMES[self.type]}_fq"), binds,
                           [self.K, self.mode, len(self.views)] + ns, ((total + 15) // 16, 1, 1))
            return
        if quantize:
            qk = "ameva_quant_a8b" if self.type == GGML_TYPE_Q4_K else "ameva_quant_a8"
            batch.dispatch(self.ctx.kernel(qk), [(x, x_offset, self.K * 4), self.aq, self.ad],
                           [1, self.K, self.K, self.mode], (1, 1, 1))
            batch.barrier()
        binds += [self.aq, self.ad]
        batch.dispatch(self.ctx.kernel(f"{fam}_{TYPE_NAMES[self.type]}"), binds, [self.K, 0, len(self.views)] + ns,
                       ((total + 15) // 16, 1, 1))

    def record_rms_norm_quantize(self, batch: rt.Batch, x: rt.Buffer, y: rt.Buffer, *, eps: float,
                                 weight: Optional[rt.Buffer] = None, x_offset: int = 0, y_offset: int = 0,
                                 w_offset: int = 0) -> None:
        """The row's RMS norm (times the weight row) written to y and quantized into the group's scratch in one kernel
        (two-kernel form only): follow with ``record(batch, y, dsts, quantize=False)``."""
        if self.fq:
            raise MulMatUnsupported("the group quantizes inside its launch: build it with fused_quantize=False")
        _record_rms_norm_quantize(self.ctx, batch, self.type, 1, self.K, x, y, self.aq, self.ad, None, None, self.mode, eps,
                                  weight, x_offset, y_offset, w_offset)

    def run(self, x: rt.Buffer, dsts, **kw) -> float:
        batch = self.ctx.batch(8)
        try:
            self.record(batch, x, dsts, **kw)
            ev = batch.submit()
            try:
                ev.wait()
                return ev.gpu_duration_us()
            finally:
                ev.destroy()
        finally:
            batch.destroy()

    def destroy(self) -> None:
        for b in (self.aq, self.ad):
            if b is not None:
                b.destroy()
        self.aq = self.ad = None


def q8_0_blocks_from_scratch(q: np.ndarray, d_bits: np.ndarray) -> np.ndarray:
    """Reassembles ggml Q8_0 block bytes (fp16 d + 32 int8) from the SoA scratch, for byte comparison with a CPU
    quantizer."""
    M, K = q.shape
    U = K // 32
    out = np.empty((M, U, 34), np.uint8)
    out[:, :, 0:2] = d_bits.astype(np.uint16).reshape(M, U, 1).view(np.uint8)
    out[:, :, 2:] = q.reshape(M, U, 32).view(np.uint8)
    return out.reshape(M, U * 34)


def q8_K_blocks_from_scratch(q: np.ndarray, d: np.ndarray, bsums: np.ndarray) -> np.ndarray:
    """Reassembles ggml Q8_K block bytes (float d, 256 int8, 16 int16 bsums) from the SoA scratch."""
    M, K = q.shape
    B = K // 256
    out = np.empty((M, B, 292), np.uint8)
    out[:, :, 0:4] = d.astype(np.float32).reshape(M, B, 1).view(np.uint8)
    out[:, :, 4:260] = q.reshape(M, B, 256).view(np.uint8)
    out[:, :, 260:] = np.ascontiguousarray(bsums.reshape(M, B, 16)).view(np.uint8)
    return out.reshape(M, B * 292)


class PeerExchange:
    """The output side of a row-sharded mul_mat on the ranks of one box (one process per GPU).

    Every rank owns a full [M][N] fp32 output and a small flag array, both exported to the other ranks
    (``handles()`` -> exchange with any out-of-band channel -> ``connect()``). Three ways to assemble the output, none of
    them with a collective library in the data path:
      * fused: ``MulMat.record(..., peers=ex.peers)`` stores each rank's rows into every rank's output from the kernel's
        epilogue; ``record_barrier`` appends the cross-GPU barrier after which the local output is complete;
      * decode sizes (M <= 8): the mul_mat writes locally and ``record_push`` appends one kernel that copies the rank's
        slice to every peer and is the barrier as well;
      * prefill sizes: the mul_mat runs in chunks of token rows; after each chunk ``record_copy`` hands the rank's column
        block of those rows to the copy engines (one queue per peer, beside the compute stream), so the transfer of a
        chunk overlaps the mul_mat of the next; ``record_join`` + ``record_barrier`` close the step."""

    def __init__(self, ctx: rt.Context, rank: int, world: int, out_bytes: int) -> None:
        if not 2 <= world <= 8 or not 0 <= rank < world:
            raise MulMatUnsupported("PeerExchange needs 2..8 ranks")
        self.ctx, self.rank, self.world = ctx, rank, world
        self.out = ctx.buffer(out_bytes)
        self.flags = ctx.buffer(512)     # words 0..63: ameva_peer_barrier; words 64..127: ameva_peer_push_barrier
        self.flags.fill(0)
        self.epoch = 0
        self.peer_out, self.peer_flags = {}, {}

    def handles(self):
        return (self.out.export_ipc(), self.flags.export_ipc(), self.out.size_bytes)

    def connect(self, all_handles) -> None:
        """all_handles[r] = handles() of rank r."""
        for r, (oh, fh, nbytes) in enumerate(all_handles):
            if r != self.rank:
                self.peer_out[r] = self.ctx.open_ipc(oh, nbytes)
                self.peer_flags[r] = self.ctx.open_ipc(fh, 512)

    @property
    def peers(self):
        return [self.peer_out[r] for r in sorted(self.peer_out)]

    def _by_rank(self, own, others, offset=0, size=None):
        return [((own if r == self.rank or r >= self.world else others[r]), offset, size) for r in range(8)]

    def record_barrier(self, batch: rt.Batch) -> None:
        """The kernel counts its own uses (epoch 0), so a recorded step can be replayed."""
        batch.dispatch(self.ctx.kernel("ameva_peer_barrier"), self._by_rank(self.flags, self.peer_flags, 0, 256),
                       [self.rank, self.world, 0], (1, 1, 1))

    def record_push(self, batch: rt.Batch, M: int, stride: int, row0: int, rows: int) -> None:
        """M <= 8: copy rows [row0, row0 + rows) of every token row of the local output to all peers and wait until the
        peers' slices have arrived (one kernel; `stride` = floats between token rows)."""
        binds = self._by_rank(self.flags, self.peer_flags, 256, 256) + self._by_rank(self.out, self.peer_out)
        batch.dispatch(self.ctx.kernel("ameva_peer_push_barrier"), binds,
                       [self.rank, self.world, 0, M, stride, row0, rows], (self.world - 1, 1, 1))

    def record_copy(self, batch: rt.Batch, m0: int, mc: int, stride: int, row0: int, rows: int) -> None:
        """Token rows [m0, m0 + mc): queue the copy of this rank's column block to every peer on the copy engines."""
        off = (m0 * stride + row0) * 4
        if off % 64:
            raise MulMatUnsupported("the column block of a rank must start on a 64-byte boundary")
        size = ((mc - 1) * stride + rows) * 4
        peers = self.peers
        binds = [(self.out, off, size)] + [(p, off, size) for p in peers] + [(self.out, off, size)] * (7 - len(peers))
        batch.dispatch(self.ctx.kernel("ameva_peer_copy"), binds, [mc, rows * 4, stride * 4, len(peers)], (1, 1, 1))

    def record_join(self, batch: rt.Batch) -> None:
        batch.dispatch(self.ctx.kernel("ameva_peer_join"), [(self.flags, 0, 64)], [], (1, 1, 1))

    def destroy(self) -> None:
        for b in list(self.peer_out.values()) + list(self.peer_flags.values()) + [self.out, self.flags]:
            b.destroy()
        self.peer_out, self.peer_flags = {}, {}

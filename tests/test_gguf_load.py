"""GGUF files as the source of mul_mat weights: directory parsing, tensor sizing with the I2_S trailer, every failure the
reference's loader reports (src/amuda/amuda_gguf.c:203-330, 334-647, 659-681 of the reference), and (GPU) the upload of
a weight from the mapping into the device layout. Files are written by the writer below and, for the block types gguf-py
knows, by gguf-py's GGUFWriter as an independent producer."""
import importlib
import os
import struct

import numpy as np
import pytest

from helpers import I2_S, Q4_0, Q4_K, Q8_0, make_acts, make_weights, max_normalised_error, oracle_mul_mat

pkg = importlib.import_module("ameva-compute_b200")
rt = pkg.runtime
gg = importlib.import_module("ameva-compute_b200.gguf")

U8, I8, U16, I16, U32, I32, F32, BOOL, STR, ARR, U64, I64, F64 = range(13)


def _s(b):
    b = b.encode() if isinstance(b, str) else b
    return struct.pack("<Q", len(b)) + b


def _value(vtype, v):
    fmt = {U8: "<B", I8: "<b", U16: "<H", I16: "<h", U32: "<I", I32: "<i", F32: "<f", BOOL: "<B", U64: "<Q", I64: "<q",
           F64: "<d"}
    if vtype == STR:
        return _s(v)
    if vtype == ARR:
        et, items = v
        return struct.pack("<IQ", et, len(items)) + b"".join(_value(et, i) for i in items)
    return struct.pack(fmt.get(vtype, "<I"), v)   # (an unknown value type is written as four bytes)


def write_gguf(path, kv, tensors, version=3, alignment=None, magic=0x46554747, tail_cut=0, counts=None):
    """kv: [(key, vtype, value)]; tensors: [(name, ggml_type, ne, bytes)]. Returns the data offsets used."""
    if alignment is not None:
        kv = list(kv) + [("general.alignment", U32, alignment)]
    al = alignment or 32
    nt, nkv = counts or (len(tensors), len(kv))
    out = struct.pack("<IIQQ", magic, version, nt, nkv)
    for k, vt, v in kv:
        out += _s(k) + struct.pack("<I", vt) + _value(vt, v)
    offs, off = [], 0
    for name, t, ne, data in tensors:
        out += _s(name) + struct.pack("<I", len(ne)) + b"".join(struct.pack("<Q", d) for d in ne)
        out += struct.pack("<IQ", t, off)
        offs.append(off)
        off += (len(data) + al - 1) // al * al
    out += b"\0" * ((-len(out)) % al)
    for (_, _, _, data), o in zip(tensors, offs):
        out += bytes(data) + b"\0" * ((-len(data)) % al)
    with open(path, "wb") as f:
        f.write(out[:len(out) - tail_cut] if tail_cut else out)
    return offs


LLAMA_KV = [("general.architecture", STR, "llama"), ("llama.context_length", U32, 4096),
            ("llama.embedding_length", U64, 512), ("llama.block_count", U32, 2), ("llama.feed_forward_length", U32, 1024),
            ("llama.attention.head_count", U32, 8), ("llama.attention.head_count_kv", U32, 2),
            ("llama.attention.layer_norm_rms_epsilon", F32, 1e-5), ("llama.rope.freq_base", F32, 10000.0),
            ("llama.vocab_size", U32, 32000), ("tokenizer.ggml.tokens", ARR, (STR, ["a", "bc", "def"])),
            ("tokenizer.ggml.scores", ARR, (F32, [0.0, 1.0, 2.0])), ("other.nested", ARR, (ARR, [(U8, [1, 2]), (U8, [3])])),
            ("llama.rope.dimension_count", U32, 64), ("general.name", STR, "tiny")]


def test_the_library_exports_what_the_header_declares():
    import ctypes
    import re
    from conftest import ROOT
    header = open(os.path.join(ROOT, "include", "amuda_gguf_b200.h")).read()
    declared = set(re.findall(r"\b(ac_(?:gguf|b200_gguf)_[a-z0-9_]+)\s*\(", header))
    assert declared == {"ac_gguf_open", "ac_gguf_get_tensor", "ac_gguf_get_tensor_scale", "ac_gguf_close",
                        "ac_b200_gguf_tensor_size", "ac_b200_gguf_device_size", "ac_b200_gguf_upload_tensor"}
    lib = ctypes.CDLL(rt.LIB_PATH)
    for name in declared:
        assert hasattr(lib, name), name


def test_tensor_sizes_follow_the_block_table_and_the_i2s_trailer():
    table = {0: (1, 4), 1: (1, 2), 2: (32, 18), 3: (32, 20), 6: (32, 22), 7: (32, 24), 8: (32, 34), 9: (32, 40),
             10: (256, 84), 11: (256, 110), 12: (256, 144), 13: (256, 176), 14: (256, 210), 15: (256, 292)}
    for t, (elems, nbytes) in table.items():
        assert gg.tensor_size(t, [4096, 11008]) == 4096 * 11008 // elems * nbytes
        assert gg.tensor_size(t, [elems + 1]) == 2 * nbytes          # a partial block counts as a whole one
        assert gg.tensor_size(t, [elems, 3, 2, 5]) == 30 * nbytes
    assert gg.tensor_size(I2_S, [2560, 6912]) == 2560 * 6912 // 4 + 32
    assert gg.tensor_size(I2_S, [5]) == 2 + 32
    for bad, code in (((I2_S, [0, 4]), "BINARY_CORRUPTED"), ((2, [1 << 40, 1 << 40]), "BINARY_CORRUPTED"),
                      ((5, [32]), "DEVICE_NOT_SUPPORTED"), ((0, [1 << 63, 2]), "BINARY_CORRUPTED"),
                      ((0, [1 << 62]), "BINARY_CORRUPTED")):
        with pytest.raises(rt.AmevaComputeError, match=code):
            gg.tensor_size(*bad)
    with pytest.raises(rt.AmevaComputeError, match="INVALID_ARGUMENT"):
        gg.tensor_size(0, [])


def test_directory_metadata_and_scale(tmp_path):
    q4, _ = make_weights(Q4_0, 8, 64, 1)
    i2, scale = make_weights(I2_S, 4, 128, 2)
    trailer = struct.pack("<f", scale) + b"\0" * 28
    f32 = np.arange(6, dtype=np.float32)
    p = str(tmp_path / "m.gguf")
    offs = write_gguf(p, LLAMA_KV, [("blk.0.attn_q.weight", Q4_0, [64, 8], q4.tobytes()),
                                    ("blk.0.ffn_up.weight", I2_S, [128, 4], i2.tobytes() + trailer),
                                    ("output_norm.weight", 0, [6], f32.tobytes())], alignment=64)
    with gg.GgufFile(p) as f:
        c = f.config
        assert (f.version, c.arch, c.context_length, c.embedding_length, c.block_count) == (3, b"llama", 4096, 512, 2)
        assert (c.feed_forward_length, c.head_count, c.head_count_kv, c.vocab_size) == (1024, 8, 2, 32000)
        assert c.rms_norm_eps == np.float32(1e-5) and c.rope_freq_base == 10000.0
        assert list(f.tensors) == ["blk.0.attn_q.weight", "blk.0.ffn_up.weight", "output_norm.weight"]
        t = f.tensors["blk.0.ffn_up.weight"]
        assert (t.n_dims, list(t.ne)[:2], t.type, t.offset, t.size_bytes) == (2, [128, 4], I2_S, offs[1], 128 + 32)
        assert np.array_equal(f.data("blk.0.attn_q.weight"), np.frombuffer(q4.tobytes(), np.uint8))
        assert np.array_equal(f.data("output_norm.weight").view(np.float32), f32)
        assert f.scale("blk.0.ffn_up.weight") == np.float32(scale) and f.scale("output_norm.weight") == 1.0
        with pytest.raises(rt.AmevaComputeError, match="DEVICE_NOT_SUPPORTED"):
            f.scale("blk.0.attn_q.weight")
        assert f.tensor("blk.0.attn_q.weight").size_bytes == 8 * 2 * 18 and f.tensor("missing") is None


def test_version_2_and_a_name_longer_than_the_field(tmp_path):
    p = str(tmp_path / "v2.gguf")
    long = "x" * 80
    write_gguf(p, [("general.architecture", STR, "bitnet")], [(long, 1, [4], b"\0" * 8)], version=2)
    with gg.GgufFile(p) as f:
        assert f.version == 2 and list(f.tensors) == ["x" * 63]     # cut to the 64-byte field, as the reference does


@pytest.mark.parametrize("kwargs,tensors,code", [
    (dict(magic=0x46554746), None, "BINARY_CORRUPTED"),
    (dict(version=4), None, "DEVICE_NOT_SUPPORTED"),
    (dict(version=1), None, "DEVICE_NOT_SUPPORTED"),
    (dict(alignment=48), None, "BINARY_CORRUPTED"),
    (dict(alignment=0), None, "BINARY_CORRUPTED"),
    (dict(tail_cut=40), None, "BINARY_CORRUPTED"),                       # the last tensor reaches past the file
    (dict(counts=(70000, 1)), None, "BINARY_CORRUPTED"),
    (dict(counts=(1, 70000)), None, "BINARY_CORRUPTED"),
    (dict(), [("w", 5, [32], b"\0" * 32)], "DEVICE_NOT_SUPPORTED"),      # a type the sizing table does not have
    (dict(), [("w", 0, [4, 0], b"\0" * 16)], "BINARY_CORRUPTED"),        # a zero dimension
    (dict(), [("w", 0, [1, 1, 1, 1, 1], b"\0" * 4)], "BINARY_CORRUPTED"),  # five dimensions
    (dict(), [("w", 0, [1 << 40, 1 << 40], b"\0" * 4)], "BINARY_CORRUPTED"),
])
def test_failures_keep_the_reference_codes_and_leave_no_model(tmp_path, kwargs, tensors, code):
    p = str(tmp_path / "bad.gguf")
    write_gguf(p, [("general.architecture", STR, "llama")], tensors or [("w", 0, [16], b"\1" * 64)], **kwargs)
    with pytest.raises(rt.AmevaComputeError, match=code):
        gg.GgufFile(p)


def test_short_files_unknown_value_types_and_deep_nesting(tmp_path):
    p = str(tmp_path / "short.gguf")
    with open(p, "wb") as f:
        f.write(b"GGUF" + b"\0" * 10)
    with pytest.raises(rt.AmevaComputeError, match="BINARY_CORRUPTED"):
        gg.GgufFile(p)
    with pytest.raises(rt.AmevaComputeError, match="BINARY_CORRUPTED"):
        gg.GgufFile(str(tmp_path / "absent.gguf"))
    write_gguf(p, [("k", 13, 0)], [])                                    # value type 13 does not exist
    with pytest.raises(rt.AmevaComputeError, match="BINARY_CORRUPTED"):
        gg.GgufFile(p)
    nested = (U8, [1])
    for _ in range(20):
        nested = (ARR, [nested])
    write_gguf(p, [("deep", ARR, nested)], [])
    with pytest.raises(rt.AmevaComputeError, match="BINARY_CORRUPTED"):
        gg.GgufFile(p)
    write_gguf(p, [("s", STR, "y" * 70000)], [])                         # a string over the 65536-byte limit
    with pytest.raises(rt.AmevaComputeError, match="BINARY_CORRUPTED"):
        gg.GgufFile(p)
    write_gguf(p, [("general.architecture", STR, "llama")], [])          # no tensors: a valid, empty directory
    with gg.GgufFile(p) as f:
        assert f.tensors == {}


def test_a_file_written_by_gguf_py_reads_back(tmp_path):
    gguf = pytest.importorskip("gguf")
    q8, _ = make_weights(Q8_0, 16, 64, 3)
    q4k, _ = make_weights(Q4_K, 4, 512, 4)
    p = str(tmp_path / "py.gguf")
    w = gguf.GGUFWriter(p, "llama")
    w.add_uint32("llama.block_count", 7)
    w.add_float32("llama.rope.freq_base", 500000.0)
    w.add_tensor("a.weight", np.frombuffer(q8.tobytes(), np.uint8).reshape(16, -1), raw_dtype=gguf.GGMLQuantizationType.Q8_0)
    w.add_tensor("b.weight", np.frombuffer(q4k.tobytes(), np.uint8).reshape(4, -1), raw_dtype=gguf.GGMLQuantizationType.Q4_K)
    w.write_header_to_file()
    w.write_kv_data_to_file()
    w.write_tensors_to_file()
    w.close()
    with gg.GgufFile(p) as f:
        assert f.config.arch == b"llama" and f.config.block_count == 7 and f.config.rope_freq_base == 500000.0
        a, b = f.tensors["a.weight"], f.tensors["b.weight"]
        assert (list(a.ne)[:2], a.type, a.size_bytes) == ([64, 16], Q8_0, 16 * 2 * 34)
        assert (list(b.ne)[:2], b.type, b.size_bytes) == ([512, 4], Q4_K, 4 * 2 * 144)
        assert np.array_equal(f.data("a.weight"), np.frombuffer(q8.tobytes(), np.uint8))
        assert np.array_equal(f.data("b.weight"), np.frombuffer(q4k.tobytes(), np.uint8))


@pytest.mark.gpu
@pytest.mark.parametrize("t,N,K", [(Q4_0, 96, 1024), (Q8_0, 130, 512), (Q4_K, 64, 2048), (I2_S, 128, 256)])
def test_weight_from_the_mapping_to_the_device_layout_and_through_mul_mat(tmp_path, t, N, K):
    qmm = pkg.qmm
    blocks, scale = make_weights(t, N, K, 11)
    raw = np.frombuffer(np.asarray(blocks).tobytes(), np.uint8)
    data = raw.tobytes() + (struct.pack("<f", scale) + b"\0" * 28 if t == I2_S else b"")
    p = str(tmp_path / "w.gguf")
    write_gguf(p, [("general.architecture", STR, "llama")], [("pad", 0, [3], b"\0" * 12), ("w", t, [K, N], data)])
    ctx = rt.init()
    x = make_acts(3, K, 12)
    with gg.GgufFile(p) as f:
        w = f.mul_mat_weight(ctx, "w")
        assert np.array_equal(w.to_ggml(), raw) and w.scale == np.float32(scale)
        # the C entry point alone leaves the same bytes in its buffer
        rawbuf = f.upload_raw(ctx, "w")
        assert f.tensors["w"].ac_buf == rawbuf.handle
        assert np.array_equal(rawbuf.read(np.uint8), w.buf.read(np.uint8, rawbuf.size_bytes))
        rawbuf.destroy()
        with pytest.raises(qmm.MulMatUnsupported):
            f.mul_mat_weight(ctx, "pad")
    mm = qmm.MulMat(ctx, w, 3)
    xb, dst = ctx.buffer(data=x), ctx.buffer(3 * N * 4)
    mm.run(xb, dst, 3)
    want, _, _ = oracle_mul_mat(t, blocks, scale, x, N, K, want_sums=False)
    assert max_normalised_error(dst.read(np.float32).reshape(3, N), want) <= 1e-3
    for o in (mm, xb, dst, w):
        o.destroy()
    ctx.destroy()

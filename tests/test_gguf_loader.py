"""GGUF file -> weight store (qm_gguf_*): the parser against the rules of the reference's reader
(gguf/gguf.go:116-250, cases of gguf/gguf_test.go) on files written here byte by byte, and, on a
GPU, tensors streamed from a file into the store and dequantized bit for bit."""
import os
import struct

import numpy as np
import pytest

import lib_b200
from lib_b200 import _capi, synth
from oracle import oracle


def gguf_bytes(tensors, metadata=(), alignment=None, version=3, pad_data=True):
    """A GGUF v3 file: tensors = [(name, type_id, dims, data bytes)], metadata = [(key, type, packed value)]."""
    out = bytearray(b"GGUF")
    out += struct.pack("<I", version)
    meta = list(metadata)
    if alignment is not None:
        meta.append(("general.alignment", 4, struct.pack("<I", alignment)))
    out += struct.pack("<QQ", len(tensors), len(meta))
    for key, t, packed in meta:
        out += struct.pack("<Q", len(key)) + key.encode() + struct.pack("<I", t) + packed
    A = alignment or 32
    off = 0
    offsets = []
    for name, type_id, dims, data in tensors:
        out += struct.pack("<Q", len(name)) + name.encode() + struct.pack("<I", len(dims))
        for d in dims:
            out += struct.pack("<Q", d)
        out += struct.pack("<IQ", type_id, off)
        offsets.append(off)
        off = (off + len(data) + A - 1) // A * A
    if tensors:
        out += bytes((-len(out)) % A)
    data_offset = len(out)
    for (name, type_id, dims, data), o in zip(tensors, offsets):
        out += bytes(data_offset + o - len(out))
        out += bytes(data)
    if pad_data:
        out += bytes((-len(out)) % A)
    return bytes(out), data_offset


def string_value(s):
    return struct.pack("<Q", len(s)) + s.encode()


@pytest.fixture
def gguf_file(tmp_path):
    def make(name, blob):
        p = tmp_path / name
        p.write_bytes(blob)
        return str(p)
    return make


def test_open_reads_the_directory(gguf_file):
    q4k = synth.weights(12, 32, 512, seed=1)
    q80 = synth.weights(8, 5, 64, seed=2)
    meta = [("general.name", 8, string_value("tiny")), ("tiny.block_count", 4, struct.pack("<I", 2)),
            ("tokenizer.scores", 9, struct.pack("<IQ", 6, 3) + struct.pack("<fff", 1, 2, 3))]
    blob, data_offset = gguf_bytes([("blk.0.ffn_down.weight", 12, [512, 32], q4k), ("output.weight", 8, [64, 5], q80)], meta)
    g = _capi.GgufFile(gguf_file("a.gguf", blob))
    assert g.tensor_count() == 2
    name, type_id, dims, offset, nbytes = g.tensor_info(0)
    assert (name, type_id, dims) == ("blk.0.ffn_down.weight", 12, [512, 32])
    assert offset == data_offset and nbytes == oracle.TensorBytes(12, [512, 32]) == len(q4k)
    name, type_id, dims, offset, nbytes = g.tensor_info(1)
    assert (name, type_id, dims, nbytes) == ("output.weight", 8, [64, 5], len(q80))
    assert offset % 32 == 0 and offset >= data_offset + len(q4k)
    assert g.find("output.weight") == 1
    with pytest.raises(lib_b200.QmError):
        g.find("missing")
    g.close()


def test_alignment_key_moves_the_data_block(gguf_file):
    blob, data_offset = gguf_bytes([("w", 8, [32, 1], bytes(34))], alignment=64)
    g = _capi.GgufFile(gguf_file("b.gguf", blob))
    assert g.tensor_info(0)[3] == data_offset and data_offset % 64 == 0
    g.close()


@pytest.mark.parametrize("case", ["magic", "version", "truncated", "dup_tensor", "zero_dim", "five_dims", "bad_alignment",
                                  "unaligned_row", "offset_gap", "unknown_type", "outside_file"])
def test_malformed_files_are_refused(gguf_file, case):
    # gguf/gguf.go:116-250: each of these makes Read fail
    good = [("w", 8, [32, 2], bytes(68))]
    if case == "magic":
        blob = b"GGML" + gguf_bytes(good)[0][4:]
    elif case == "version":
        blob = gguf_bytes(good, version=2)[0]
    elif case == "truncated":
        blob = gguf_bytes(good)[0][:40]
    elif case == "dup_tensor":
        blob = gguf_bytes([("w", 8, [32, 1], bytes(34)), ("w", 8, [32, 1], bytes(34))])[0]
    elif case == "zero_dim":
        blob = gguf_bytes([("w", 8, [32, 0], b"")])[0]
    elif case == "five_dims":
        blob = gguf_bytes([("w", 8, [32, 1, 1, 1, 1], bytes(34))])[0]
    elif case == "bad_alignment":
        blob = gguf_bytes(good, alignment=12)[0]
    elif case == "unaligned_row":
        blob = gguf_bytes([("w", 8, [48, 1], bytes(51))])[0]
    elif case == "unknown_type":
        blob = gguf_bytes([("w", 4242, [32, 1], bytes(34))])[0]
    elif case == "outside_file":
        blob = gguf_bytes(good, pad_data=False)[0][:-8]
    else:  # offset_gap: the second tensor does not start where the first one ends (aligned)
        blob = bytearray(gguf_bytes([("a", 8, [32, 1], bytes(34)), ("b", 8, [32, 1], bytes(34))])[0])
        idx = blob.index(b"b" + struct.pack("<I", 2)) + 1 + 4 + 16 + 4   # name, ndims, dims, type -> offset field
        blob[idx:idx + 8] = struct.pack("<Q", 128)
        blob = bytes(blob) + bytes(256)
    with pytest.raises(lib_b200.QmError) as e:
        _capi.GgufFile(gguf_file(case + ".gguf", blob))
    assert e.value.code in (-3, -1)   # QM_ERR_FORMAT, or QM_ERR_COUNT for the row that is not block aligned


def test_written_file_is_what_ggufpy_reads(gguf_file):
    """The byte-by-byte writer above against the GGUF format's upstream Python reader."""
    gguf = pytest.importorskip("gguf", reason="gguf-py is not installed")
    q4k = synth.weights(12, 16, 256, seed=3)
    path = gguf_file("c.gguf", gguf_bytes([("blk.0.attn_q.weight", 12, [256, 16], q4k)], [("general.name", 8, string_value("t"))])[0])
    r = gguf.GGUFReader(path)
    t = r.tensors[0]
    assert t.name == "blk.0.attn_q.weight" and int(t.tensor_type) == 12
    assert bytes(np.asarray(t.data).reshape(-1).view(np.uint8)) == bytes(q4k)


@pytest.mark.gpu
def test_tensors_stream_into_the_store(ctx, devbuf, gguf_file):
    shapes = [("q4k", 12, 80, 1024), ("q80", 8, 37, 736), ("q40", 2, 64, 512), ("q2k", 10, 20, 512), ("iq2", 16, 20, 512)]
    raws = {n: synth.weights(f, r, c, seed=10 + i) for i, (n, f, r, c) in enumerate(shapes)}
    blob, _ = gguf_bytes([(n, f, [c, r], raws[n]) for n, f, r, c in shapes])
    g = _capi.GgufFile(gguf_file("d.gguf", blob))
    for i, (n, f, r, c) in enumerate(shapes):
        w = g.load_tensor(ctx, i)
        out = devbuf(nbytes=r * c * 4)
        ctx.dequantize(w, out.ptr)
        ctx.sync()
        want = oracle.Dequantize(f, raws[n], r * c)
        assert np.array_equal(out.get((r * c,)).view(np.uint32), want.view(np.uint32)), n
        w.free()
    # a row slice (a tensor-parallel rank's share), and two tensors stacked by rows into one entry
    w = g.load_tensor(ctx, 0, 16, 48)
    out = devbuf(nbytes=32 * 1024 * 4)
    ctx.dequantize(w, out.ptr)
    ctx.sync()
    want = oracle.Dequantize(12, raws["q4k"], 80 * 1024).reshape(80, 1024)[16:48]
    assert np.array_equal(out.get((32, 1024)).view(np.uint32), want.view(np.uint32))
    w.free()
    stacked = ctx.store_create(12, 160, 1024)
    g.load_rows(ctx, 0, 0, 80, stacked, 0)
    g.load_rows(ctx, 0, 0, 80, stacked, 80)
    out = devbuf(nbytes=160 * 1024 * 4)
    ctx.dequantize(stacked, out.ptr)
    ctx.sync()
    full = oracle.Dequantize(12, raws["q4k"], 80 * 1024).reshape(80, 1024)
    assert np.array_equal(out.get((160, 1024)).view(np.uint32), np.concatenate([full, full]).view(np.uint32))
    stacked.free()
    g.close()


@pytest.mark.gpu
def test_large_tensor_streams_in_chunks(ctx, gguf_file):
    """More rows than one 32 MiB staging chunk holds: both staging buffers and their events are reused."""
    rows, cols = 16384, 4096   # 37.7 MB of Q4_K
    raw = synth.weights(12, rows, cols, seed=77)
    g = _capi.GgufFile(gguf_file("e.gguf", gguf_bytes([("big", 12, [cols, rows], raw)])[0]))
    w = g.load_tensor(ctx, 0)
    x = synth.activations(1, cols, 5)
    y = ctx.matvec_host(w, x)
    ref = ctx.store_upload(12, rows, cols, raw)
    assert np.array_equal(y, ctx.matvec_host(ref, x))
    w.free()
    ref.free()
    g.close()

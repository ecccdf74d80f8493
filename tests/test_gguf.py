"""GGUF reader (include/fuelq_gguf.h) against an independent implementation of the format (gguf-py) and against
the parsing rules of the reference's `Content::read` (fuel-formats/src/gguf.rs:385-462). No GPU: header, metadata
and mapped tensor bytes only."""
import os
import struct

import numpy as np
import pytest

from fuel_b200 import gguf as G
from fuel_b200.ggml import GgmlDType as T
from oracle import oracle as O

gguf_py = pytest.importorskip("gguf")


def _blocks(ot, n, k, seed):
    w = np.random.Generator(np.random.PCG64(seed)).standard_normal((n, k), dtype=np.float32) * np.float32(0.02)
    return np.asarray(O.quantize(ot, w), dtype=np.uint8).reshape(-1)


@pytest.fixture(scope="module")
def tensors():
    return [("token_embd.weight", T.Q4K, (12, 256), _blocks(O.Q4K, 12, 256, 0)),
            ("blk.0.attn_q.weight", T.Q4K, (8, 512), _blocks(O.Q4K, 8, 512, 1)),
            ("blk.0.attn_v.weight", T.Q6K, (8, 512), _blocks(O.Q6K, 8, 512, 2)),
            ("blk.0.ffn_down.weight", T.Q8_0, (6, 96), _blocks(O.Q8_0, 6, 96, 3)),
            ("blk.0.attn_norm.weight", T.F32, (512,), np.arange(512, dtype=np.float32).view(np.uint8))]


def test_reads_what_gguf_py_writes(tmp_path, tensors):
    path = str(tmp_path / "a.gguf")
    w = gguf_py.GGUFWriter(path, "llama")
    w.add_uint32("llama.block_count", 1)
    w.add_float32("llama.attention.layer_norm_rms_epsilon", 1e-5)
    w.add_bool("some.flag", True)
    w.add_uint64("big", 2 ** 63 + 5)
    w.add_int32("neg", -7)
    w.add_string("general.name", "tiny")
    w.add_array("tokenizer.ggml.tokens", ["<s>", "a", "bc", ""])
    w.add_array("tokenizer.ggml.scores", [0.5, -1.0, 2.0])
    w.add_array("ints", [1, 2, 3])
    qt = gguf_py.GGMLQuantizationType
    for name, dt, shape, data in tensors:
        if dt == T.F32:
            w.add_tensor(name, data.view(np.float32).reshape(shape))
        else:
            rb = shape[-1] // dt.block_size() * dt.type_size()
            w.add_tensor(name, data.reshape(shape[0], rb), raw_dtype=qt(int(dt)))
    w.write_header_to_file()
    w.write_kv_data_to_file()
    w.write_tensors_to_file()
    w.close()

    with G.GgufFile(path) as f:
        assert f.version == 3 and f.alignment == 32 and f.tensor_data_offset % 32 == 0
        m = f.metadata
        assert m["general.architecture"] == "llama" and m["llama.block_count"] == 1 and m["some.flag"] is True
        assert m["big"] == 2 ** 63 + 5 and m["neg"] == -7 and m["general.name"] == "tiny"
        assert m["llama.attention.layer_norm_rms_epsilon"] == np.float32(1e-5)
        assert m["tokenizer.ggml.tokens"] == ["<s>", "a", "bc", ""]
        assert m["tokenizer.ggml.scores"].tolist() == [0.5, -1.0, 2.0] and m["ints"].tolist() == [1, 2, 3]
        assert set(f.tensor_infos) == {t[0] for t in tensors}
        for name, dt, shape, data in tensors:
            info = f.tensor_infos[name]
            assert info.ggml_dtype == dt and info.shape == shape and info.nbytes == data.size
            assert info.offset % 32 == 0
            assert np.array_equal(f.tensor_bytes(name), data)
        # the same offsets as the independent reader reports
        r = gguf_py.GGUFReader(path)
        for t in r.tensors:
            assert f.tensor_data_offset + f.tensor_infos[t.name].offset == t.data_offset


@pytest.mark.parametrize("version", [1, 2, 3])
@pytest.mark.parametrize("alignment", [None, 64])
def test_round_trip_of_every_version(tmp_path, tensors, version, alignment):
    path = str(tmp_path / "b.gguf")
    meta = [("llama.block_count", G.U32, 1), ("name\0\0", G.STRING, "x\0"), ("f", G.F64, 0.25), ("i8", G.I8, -3),
            ("u16", G.U16, 65535), ("i16", G.I16, -2), ("i64", G.I64, -2 ** 40), ("b", G.BOOL, 0),
            ("strs", G.ARRAY, (G.STRING, ["p", "qq\0"])), ("u8s", G.ARRAY, (G.U8, [1, 2, 255])),
            ("nested", G.ARRAY, (G.ARRAY, [(G.I32, [1, 2]), (G.STRING, ["z"])])), ("after", G.U32, 9)]
    G.write_gguf(path, meta, tensors, version=version, alignment=alignment)
    with G.GgufFile(path) as f:
        al = alignment or 32
        assert f.version == version and f.alignment == al and f.tensor_data_offset % al == 0
        m = f.metadata
        # trailing NULs of strings (keys too) are dropped on read (gguf.rs:78-81)
        assert m["name"] == "x" and m["strs"] == ["p", "qq"] and m["u8s"].tolist() == [1, 2, 255]
        assert m["f"] == 0.25 and m["i8"] == -3 and m["u16"] == 65535 and m["i16"] == -2 and m["i64"] == -2 ** 40 and m["b"] is False
        assert m["nested"] is None and m["after"] == 9  # an array of arrays is walked, what follows it still parses
        for name, dt, shape, data in tensors:
            info = f.tensor_infos[name]
            assert (info.ggml_dtype, info.shape, info.nbytes) == (dt, shape, data.size) and info.offset % al == 0
            assert np.array_equal(f.tensor_bytes(name), data)
    if version >= 2:  # gguf-py reads v2 and v3
        r = gguf_py.GGUFReader(path)
        got = {t.name: bytes(np.asarray(t.data).reshape(-1).view(np.uint8)) for t in r.tensors}
        for name, dt, shape, data in tensors:
            assert got[name] == data.tobytes()
    # the bytes of a whole file work like the path
    with G.GgufFile(open(path, "rb").read()) as f2:
        assert np.array_equal(f2.tensor_bytes(tensors[2][0]), tensors[2][3])


def _hdr(version=3, n_tensors=0, n_kv=0, magic=0x46554747):
    cnt = "<I" if version == 1 else "<Q"
    return struct.pack("<II", magic, version) + struct.pack(cnt, n_tensors) + struct.pack(cnt, n_kv)


def _s(s, version=3):
    return struct.pack("<I" if version == 1 else "<Q", len(s)) + s


def test_rejects_what_the_reference_rejects():
    with pytest.raises(G.GgufError, match="unknown magic 0x12345678"):
        G.GgufFile(_hdr(magic=0x12345678))
    G.GgufFile(_hdr(magic=0x47475546)).close()  # the tag in the other byte order is accepted (gguf.rs:29)
    for v in (0, 4):
        with pytest.raises(G.GgufError, match="unsupported magic/version"):
            G.GgufFile(struct.pack("<II", 0x46554747, v) + b"\0" * 16)
    with pytest.raises(G.GgufError, match="unexpected bool value 2"):
        G.GgufFile(_hdr(n_kv=1) + _s(b"k") + struct.pack("<IB", G.BOOL, 2))
    with pytest.raises(G.GgufError, match="unrecognized value-type"):
        G.GgufFile(_hdr(n_kv=1) + _s(b"k") + struct.pack("<II", 13, 0))
    with pytest.raises(G.GgufError, match="unknown dtype for tensor 4"):
        G.GgufFile(_hdr(n_tensors=1) + _s(b"t") + struct.pack("<IQIQ", 1, 32, 4, 0))
    with pytest.raises(G.GgufError) as e:
        G.GgufFile(os.path.join(os.sep, "nonexistent", "x.gguf"))
    assert e.value.status == 2


def test_alignment_rules():
    """general.alignment counts when it is U8/U16/U32 or a non-negative I8/I16/I32; anything else means 32
    (gguf.rs:443-451). The data offset is the header's end rounded up."""
    def image(vtype, value):
        return _hdr(n_kv=1) + _s(b"general.alignment") + struct.pack("<I", vtype) + struct.pack(G._PACK[vtype], value)
    for vtype, value, want in ((G.U8, 16, 16), (G.U16, 128, 128), (G.U32, 4096, 4096), (G.I8, 8, 8), (G.I32, 64, 64),
                               (G.I32, -64, 32), (G.U64, 64, 32), (G.I64, 64, 32), (G.F32, 64.0, 32)):
        with G.GgufFile(image(vtype, value)) as f:
            n = len(image(vtype, value))
            assert f.alignment == want and f.tensor_data_offset == (n + want - 1) // want * want
    with pytest.raises(G.GgufError, match="alignment"):
        G.GgufFile(image(G.U32, 0))


def test_repeated_names_keep_the_last_entry():
    img = (_hdr(n_tensors=2, n_kv=2) + _s(b"k") + struct.pack("<II", G.U32, 1) + _s(b"k") + struct.pack("<II", G.U32, 2)
           + _s(b"t") + struct.pack("<IQIQ", 1, 32, 0, 0) + _s(b"t") + struct.pack("<IQQIQ", 2, 4, 3, 0, 128))
    with G.GgufFile(img) as f:
        assert f.metadata == {"k": 2}
        assert list(f.tensor_infos) == ["t"] and f.tensor_infos["t"].shape == (3, 4) and f.tensor_infos["t"].offset == 128


def test_truncated_and_out_of_range_files_are_errors_not_faults(tmp_path, tensors):
    path = str(tmp_path / "c.gguf")
    G.write_gguf(path, [("a", G.ARRAY, (G.STRING, ["x", "y"])), ("n", G.U32, 3)], tensors[:2])
    img = open(path, "rb").read()
    with G.GgufFile(img) as f:
        header_end = f.tensor_data_offset
    for cut in range(0, header_end - 31):  # every prefix that ends inside the header
        with pytest.raises(G.GgufError):
            G.GgufFile(img[:cut])
    # the header is whole but the data is cut short: the table is readable, the affected tensor is refused
    with G.GgufFile(img[:len(img) - 1]) as f:
        assert np.array_equal(f.tensor_bytes(tensors[0][0]), tensors[0][3])
        with pytest.raises(G.GgufError, match="outside the file"):
            f.tensor_bytes(tensors[1][0])
    # absurd counts and lengths
    for bad in (_hdr(n_kv=2 ** 62), _hdr(n_tensors=2 ** 62), _hdr(n_kv=1) + struct.pack("<Q", 2 ** 63) + b"k",
                _hdr(n_kv=1) + _s(b"k") + struct.pack("<IIQ", G.ARRAY, G.U64, 2 ** 61),
                _hdr(n_tensors=1) + _s(b"t") + struct.pack("<I", 9),
                _hdr(n_tensors=1) + _s(b"t") + struct.pack("<IQQIQ", 2, 2 ** 40, 2 ** 40, 0, 0)):
        with pytest.raises(G.GgufError):
            G.GgufFile(bad)
    with G.GgufFile(img) as f, pytest.raises(KeyError, match="missing tensor"):
        f.tensor_info("nope")
    # sizes a hostile header can declare: an element count that is not whole blocks (would be truncated
    # silently), and dims whose byte size wraps 64 bits to something small (2^62 F32 elements -> 2^64 bytes)
    with pytest.raises(G.GgufError, match="whole number of blocks"):
        G.GgufFile(_hdr(n_tensors=1) + _s(b"t") + struct.pack("<IQIQ", 1, 300, int(T.Q4K), 0))
    with pytest.raises(G.GgufError, match="larger than the file"):
        G.GgufFile(_hdr(n_tensors=1) + _s(b"t") + struct.pack("<IQQIQ", 2, 2 ** 31, 2 ** 31, 0, 0))
    with pytest.raises(G.GgufError, match="larger than the file"):
        G.GgufFile(_hdr(n_tensors=1) + _s(b"t") + struct.pack("<IQIQ", 1, 2 ** 62, 0, 0) + b"\0" * 64)


def test_llama_loader_reads_architecture_and_checks_shapes(tmp_path):
    """Host logic of QLlama.from_gguf that needs no GPU: the architecture from the llama.* keys and tensor shapes, the
    element-count checks (fuel-core/src/lazy_quantized_llama.rs:271-277), tied embeddings, refused formats."""
    torch = pytest.importorskip("torch")
    import dataclasses
    from fuel_b200.llama import GgufWeights, LlamaConfig
    dim, ffn, vocab, layers = 256, 512, 64, 2

    def blob(t, n, k):
        return np.zeros(n * k // t.block_size() * t.type_size(), np.uint8)

    tensors = [("token_embd.weight", T.Q6K, (vocab, dim), blob(T.Q6K, vocab, dim)),
               ("output_norm.weight", T.F32, (dim,), np.zeros(dim * 4, np.uint8))]
    for li in range(layers):
        for nm, (n, k), t in (("attn_q", (dim, dim), T.Q4K), ("attn_k", (dim // 2, dim), T.Q4K), ("attn_v", (dim // 2, dim), T.Q6K),
                              ("attn_output", (dim, dim), T.Q8_0), ("ffn_gate", (ffn, dim), T.Q5K), ("ffn_up", (ffn, dim), T.Q5K),
                              ("ffn_down", (dim, ffn), T.Q8K if li == 1 else T.Q4_0)):
            tensors.append((f"blk.{li}.{nm}.weight", t, (n, k), blob(t, n, k)))
        for nm in ("attn_norm", "ffn_norm"):
            tensors.append((f"blk.{li}.{nm}.weight", T.F32, (dim,), np.zeros(dim * 4, np.uint8)))
    meta = [("general.architecture", G.STRING, "llama"), ("llama.block_count", G.U32, layers),
            ("llama.attention.head_count", G.U32, 2), ("llama.attention.head_count_kv", G.U32, 1),
            ("llama.attention.layer_norm_rms_epsilon", G.F32, 1e-6), ("llama.rope.freq_base", G.F32, 500000.0)]
    path = str(tmp_path / "arch.gguf")
    G.write_gguf(path, meta, tensors)
    w = GgufWeights(path, torch.device("cpu"))
    cfg = w.config(max_seq=128)
    assert cfg == LlamaConfig(dim=dim, n_layers=layers, n_heads=2, n_kv_heads=1, head_dim=128, ffn_dim=ffn, vocab=vocab,
                              norm_eps=float(np.float32(1e-6)), rope_theta=500000.0, max_seq=128)
    w.check(cfg)
    with pytest.raises(ValueError, match="elements, expected"):
        w.check(dataclasses.replace(cfg, n_kv_heads=2))
    assert w.dtype("attn_v", 0) == T.Q6K and w.dtype("ffn_gate", 1) == T.Q5K and w.dtype("ffn_down", 0) == T.Q4_0
    assert w.dtype("output", -1) == T.Q6K            # no output.weight: the head is the embedding table
    with pytest.raises(NotImplementedError, match="Q8K"):
        w.dtype("ffn_down", 1)
    with pytest.raises(KeyError, match="missing tensor"):
        w.dtype("attn_q", 2)
    w.file.close()
    G.write_gguf(path, [("general.architecture", G.STRING, "qwen3moe")] + meta[1:], tensors)
    with pytest.raises(ValueError, match="not the LLaMA layout"):
        GgufWeights(path, torch.device("cpu")).config()

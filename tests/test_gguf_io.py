"""GGUF v3 container reader: round trips through the writer and the reference's error cases
(tests/Test_GGUF.cpp's container tests: bad magic, wrong version, truncation, missing tensor, payload
out of range, unsupported shapes). CPU tests build tensors on the host; the GPU test runs a loaded
tensor through the GEMV and checks it against the CPU checker."""
import struct

import numpy as np
import pytest
import torch


def _file(kd, tmp_path, tensors, kv=None, name="m.gguf"):
    p = str(tmp_path / name)
    kd.write_gguf(p, kv or {}, tensors)
    return p


def test_round_trip_metadata_and_payloads(kd, tmp_path):
    pk = kd.ggml_pack
    w4 = pk.random_payload(kd.Q4_K, 5, 512, 1)
    w8 = pk.random_payload(kd.Q8_0, 3, 96, 2)
    norm = np.arange(7, dtype=np.float32)
    kv = {"general.architecture": "lfm2moe", "lfm2moe.block_count": 24, "lfm2moe.rope.freq_base": 1e6,
          "tokenizer.ggml.tokens": ["a", "bc", ""], "lfm2moe.flag": True, "neg": -5,
          "lfm2moe.head_count_kv": np.array([0, 8, 0, 8], dtype=np.int32)}
    p = _file(kd, tmp_path, [("blk.0.w", [512, 5], kd.Q4_K, w4), ("out.w", [96, 3], kd.Q8_0, w8),
                             ("norm", [7], 0, norm)], kv)
    f = kd.GgufFile(p)
    assert f.version == 3 and f.data_start % 32 == 0 and len(f.tensors) == 3
    assert f.get("general.architecture", str) == "lfm2moe"
    assert f.kv["lfm2moe.block_count"] == 24 and f.kv["neg"] == -5 and f.kv["lfm2moe.flag"] is True
    assert f.kv["lfm2moe.rope.freq_base"] == pytest.approx(1e6)
    assert f.kv["tokenizer.ggml.tokens"] == ["a", "bc", ""]
    assert np.array_equal(f.kv["lfm2moe.head_count_kv"], [0, 8, 0, 8])
    with pytest.raises(RuntimeError, match="KV not found"):
        f.get("general.architecture", int)
    t = f.tensor("blk.0.w")
    assert (t.rows(), t.cols(), t.dtype, t.nbytes, t.numel) == (5, 512, kd.Q4_K, 5 * 2 * 144, 5 * 512)
    assert np.array_equal(f.payload(t), w4.reshape(-1))
    assert np.array_equal(f.payload(f.tensor("out.w")), w8.reshape(-1))
    n = f.tensor("norm")
    assert (n.rows(), n.cols()) == (1, 7)
    assert np.array_equal(f.payload(n).view(np.float32), norm)
    assert all(x.offset % 32 == 0 for x in f.tensors)
    assert f.has_tensor("norm") and not f.has_tensor("nope")
    with pytest.raises(RuntimeError, match="tensor not found"):
        f.tensor("nope")
    f.close()


def test_load_quant_weight_on_host(kd, tmp_path):
    w6 = kd.ggml_pack.random_payload(kd.Q6_K, 4, 256, 3)
    ex = kd.ggml_pack.random_payload(kd.Q4_K, 3 * 6, 256, 4)          # 3 experts x 6 rows
    p = _file(kd, tmp_path, [("w6", [256, 4], kd.Q6_K, w6), ("ex", [256, 6, 3], kd.Q4_K, ex),
                             ("f", [8, 2], 0, np.zeros(16, np.float32))])
    f = kd.GgufFile(p)
    w = kd.load_quant_weight(f, f.tensor("w6"), device="cpu")
    assert (w.dtype, w.rows, w.cols, w.bytes()) == (kd.Q6_K, 4, 256, 4 * 210)
    assert np.array_equal(w.data.numpy(), w6.reshape(-1))
    with pytest.raises(RuntimeError, match="unsupported dtype"):
        kd.load_quant_weight(f, f.tensor("f"), device="cpu")
    with pytest.raises(RuntimeError, match="only 1-D/2-D"):
        kd.load_quant_weight(f, f.tensor("ex"), device="cpu")
    with pytest.raises(RuntimeError, match="3-D"):
        kd.load_expert_weights(f, f.tensor("w6"), device="cpu")
    ws = kd.load_expert_weights(f, f.tensor("ex"), device="cpu")
    assert len(ws) == 3 and all((e.rows, e.cols, e.dtype) == (6, 256, kd.Q4_K) for e in ws)
    per = 6 * 144
    flat = ex.reshape(-1)
    for e, q in enumerate(ws):
        assert np.array_equal(q.data.numpy(), flat[e * per:(e + 1) * per])
        assert (q.data.data_ptr() - ws[0].data.data_ptr()) % 256 == 0


def _header(version=3, n_tensors=0, n_kv=0, magic=b"GGUF"):
    return magic + struct.pack("<IQQ", version, n_tensors, n_kv)


def _s(s):
    return struct.pack("<Q", len(s)) + s


@pytest.mark.parametrize("blob,msg", [
    (b"GGUF", "too small"),
    (_header(magic=b"GGML") + b"\0" * 8, "bad magic"),
    (_header(version=2) + b"\0" * 8, "unsupported version"),
    (_header(n_kv=1) + _s(b"k") + struct.pack("<I", 99) + b"\0" * 16, "bad metadata type"),
    (_header(n_kv=1) + _s(b"k") + struct.pack("<I", 8) + struct.pack("<Q", 1000), "truncated"),
    (_header(n_tensors=1) + _s(b"t") + struct.pack("<I", 5) + b"\0" * 64, "bad n_dims"),
    (_header(n_tensors=1) + _s(b"t") + struct.pack("<IQIQ", 1, 256, 77, 0), "unknown dtype"),
    (_header(n_tensors=1) + _s(b"t") + struct.pack("<IQIQ", 1, 100, 12, 0), "multiple of block"),
    (_header(n_tensors=1) + _s(b"t") + struct.pack("<IQIQ", 1, 256, 12, 0) + b"\0" * 64, "payload out of range"),
    (_header(n_tensors=3) + _s(b"t") + struct.pack("<IQIQ", 1, 256, 12, 0), "truncated"),
])
def test_malformed_files_raise(kd, tmp_path, blob, msg):
    p = tmp_path / "bad.gguf"
    p.write_bytes(blob)
    with pytest.raises(RuntimeError, match=msg):
        kd.GgufFile(str(p))


def test_missing_file_raises(kd, tmp_path):
    with pytest.raises(RuntimeError, match="cannot open"):
        kd.GgufFile(str(tmp_path / "absent.gguf"))


def test_size_mismatch_is_caught(kd, tmp_path):
    w = kd.ggml_pack.random_payload(kd.Q4_K, 2, 256, 5)
    p = _file(kd, tmp_path, [("w", [256, 2], kd.Q4_K, w)])
    f = kd.GgufFile(p)
    t = f.tensor("w")
    t.nbytes -= 144                      # a corrupted info record
    with pytest.raises(RuntimeError, match="size mismatch"):
        kd.load_quant_weight(f, t, device="cpu")


@pytest.mark.gpu
@pytest.mark.parametrize("dtype_name", ["Q4_K", "Q5_K", "Q6_K", "Q8_0"])
def test_loaded_weight_runs_the_gemv(kd, port, tmp_path, dtype_name):
    from oracle import oracle as O
    dtype = getattr(kd, dtype_name)
    rows, K = 37, 1024
    packed = kd.ggml_pack.random_payload(dtype, rows, K, 11)
    f = kd.GgufFile(_file(kd, tmp_path, [("pad", [5], 24, np.zeros(5, np.uint8)), ("w", [K, rows], dtype, packed)]))
    w = kd.load_quant_weight(f, f.tensor("w"))
    x = torch.randn(K, generator=torch.Generator().manual_seed(12))
    y = torch.empty(rows, device="cuda")
    scratch = torch.zeros(kd.quant_gemv_int8_scratch_bytes(K), dtype=torch.uint8, device="cuda")
    kd.quant_gemv(x.cuda(), w, y, scratch)
    torch.cuda.synchronize()
    y_ref, _ = port.gemv_int8(dtype, O.aligned_copy(packed), rows, K, x.numpy())
    assert np.abs(y.cpu().numpy() - y_ref).max() <= 1e-3 * max(np.abs(y_ref).max(), 1e-30)


@pytest.mark.gpu
def test_loaded_experts_feed_the_table(kd, port, tmp_path):
    from oracle import oracle as O
    E, rows, K = 4, 24, 512
    packed = kd.ggml_pack.random_payload(kd.Q8_0, E * rows, K, 21)   # 34-byte blocks: slices need the padding
    f = kd.GgufFile(_file(kd, tmp_path, [("ffn_up_exps", [K, rows, E], kd.Q8_0, packed)]))
    ws = kd.load_expert_weights(f, f.tensor("ffn_up_exps"))
    table = kd.make_quant_weight_table(ws, "up")
    assert table.size() == E and table.rows == rows and table.cols == K
    assert all(w.data.data_ptr() % 256 == 0 for w in ws)
    x = torch.randn(K, generator=torch.Generator().manual_seed(22))
    scratch = torch.zeros(kd.quant_gemv_int8_scratch_bytes(K), dtype=torch.uint8, device="cuda")
    per = rows * kd.ggml_row_bytes(kd.Q8_0, K)
    flat = packed.reshape(-1)
    for e in range(E):
        y = torch.empty(rows, device="cuda")
        kd.quant_gemv(x.cuda(), ws[e], y, scratch)
        y_ref, _ = port.gemv_int8(kd.Q8_0, O.aligned_copy(flat[e * per:(e + 1) * per]), rows, K, x.numpy())
        assert np.abs(y.cpu().numpy() - y_ref).max() <= 1e-3 * max(np.abs(y_ref).max(), 1e-30)


def _fixture_tensors(kd):
    import importlib.util
    import os
    here = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
    spec = importlib.util.spec_from_file_location("_make_golden", os.path.join(here, "make_golden.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return os.path.join(here, "ref_written.gguf"), mod.gguf_fixture_tensors(kd.ggml_pack)


def test_reads_the_file_the_reference_wrote(kd):
    """tests/golden/ref_written.gguf came out of the reference's own writer (make_golden.py)."""
    path, tensors = _fixture_tensors(kd)
    f = kd.GgufFile(path)
    assert f.get("general.architecture", str) == "lfm2moe" and f.get("general.name", str) == "fixture"
    assert f.get("lfm2moe.block_count", int) == 2 and f.get("lfm2moe.expert_count", int) == 3
    assert f.get("lfm2moe.attention.layer_norm_rms_epsilon", float) == pytest.approx(1e-5)
    assert [t.name for t in f.tensors] == [t[0] for t in tensors]
    for name, dims, dtype, raw in tensors:
        t = f.tensor(name)
        assert (t.dims, t.dtype) == (list(dims), dtype)
        assert np.array_equal(f.payload(t), np.ascontiguousarray(raw).view(np.uint8).reshape(-1))
    ws = kd.load_expert_weights(f, f.tensor("blk.0.ffn_gate_exps.weight"), device="cpu")
    assert len(ws) == 3 and (ws[0].rows, ws[0].cols) == (5, 256)
    w = kd.load_quant_weight(f, f.tensor("blk.1.ffn_down.weight"), device="cpu")
    assert (w.dtype, w.rows, w.cols) == (kd.Q5_K, 2, 512)


def test_reference_reader_accepts_what_the_writer_wrote(kd, ref, tmp_path):
    """The other direction, where the reference's library was built: its GgufFile parses this writer's file."""
    _, tensors = _fixture_tensors(kd)
    kv = {"general.architecture": "lfm2moe", "lfm2moe.block_count": 7, "lfm2moe.rope.freq_base": 5e5,
          "tokenizer.ggml.tokens": ["x", "yz"], "lfm2moe.flags": np.array([True, False, True])}
    p = _file(kd, tmp_path, tensors, kv)
    mine = kd.GgufFile(p)
    assert ref.gguf_read_kv(p, "general.architecture", "str") == "lfm2moe"
    assert ref.gguf_read_kv(p, "lfm2moe.block_count", "u32") == 7
    assert ref.gguf_read_kv(p, "lfm2moe.rope.freq_base", "f32") == pytest.approx(5e5)
    for name, dims, dtype, raw in tensors:
        rd, rdims, roff, rbytes, rstart, payload = ref.gguf_read_tensor(p, name)
        t = mine.tensor(name)
        assert (rd, rdims, roff, rbytes, rstart) == (dtype, list(dims), t.offset, t.nbytes, mine.data_start)
        assert np.array_equal(payload, np.ascontiguousarray(raw).view(np.uint8).reshape(-1))
    with pytest.raises(RuntimeError, match="tensor not found"):
        ref.gguf_read_tensor(p, "absent")


def test_reference_writer_round_trip(kd, ref, tmp_path):
    """A file from the reference's writer, made on the spot, parses to the same records in both readers."""
    w = kd.ggml_pack.random_payload(kd.Q4_K, 6, 768, 31)
    p = str(tmp_path / "r.gguf")
    ref.gguf_write(p, [("a", [768, 6], kd.Q4_K, w), ("b", [3], 0, np.ones(3, np.float32))],
                   strings={"k": "v"}, u32={"n": 4})
    f = kd.GgufFile(p)
    rd, rdims, roff, rbytes, rstart, payload = ref.gguf_read_tensor(p, "a")
    t = f.tensor("a")
    assert (t.dtype, t.dims, t.offset, t.nbytes, f.data_start) == (rd, rdims, roff, rbytes, rstart)
    assert np.array_equal(f.payload(t), payload) and np.array_equal(payload, w.reshape(-1))
    assert f.kv == {"k": "v", "n": 4}


def test_dense_tensors_widen_exactly(kd, tmp_path):
    g = torch.Generator().manual_seed(5)
    a32 = torch.randn(3, 8, generator=g)
    a16 = torch.randn(2, 16, generator=g).half()
    ab = torch.randn(4, 8, generator=g).bfloat16()
    p = _file(kd, tmp_path, [("a32", [8, 3], 0, a32.numpy()), ("a16", [16, 2], 1, a16.numpy()),
                             ("ab", [8, 4], 30, ab.view(torch.int16).numpy()), ("v", [5], 0, np.ones(5, np.float32)),
                             ("q", [256, 1], kd.Q4_K, kd.ggml_pack.random_payload(kd.Q4_K, 1, 256, 1)),
                             ("i", [4], 26, np.zeros(4, np.int32))])
    f = kd.GgufFile(p)
    assert torch.equal(kd.tensor_to_float(f, f.tensor("a32"), "cpu"), a32)
    assert torch.equal(kd.tensor_to_float(f, f.tensor("a16"), "cpu"), a16.float())
    assert torch.equal(kd.tensor_to_float(f, f.tensor("ab"), "cpu"), ab.float())
    assert tuple(kd.tensor_to_float(f, f.tensor("v"), "cpu").shape) == (1, 5)
    with pytest.raises(RuntimeError, match="CUDA device"):
        kd.tensor_to_float(f, f.tensor("q"), "cpu")
    with pytest.raises(RuntimeError, match="unsupported dtype"):
        kd.tensor_to_float(f, f.tensor("i"), "cpu")


@pytest.mark.gpu
@pytest.mark.parametrize("dtype_name", ["Q4_K", "Q5_K", "Q6_K", "Q8_0"])
def test_packed_tensor_to_float_matches_the_block_formulas(kd, port, tmp_path, dtype_name):
    from oracle import oracle as O
    dtype = getattr(kd, dtype_name)
    rows, K = 9, 512
    packed = kd.ggml_pack.random_payload(dtype, rows, K, 41)
    f = kd.GgufFile(_file(kd, tmp_path, [("w", [K, rows], dtype, packed)]))
    got = kd.tensor_to_float(f, f.tensor("w")).cpu().numpy()
    want = port.dequant_rows(dtype, O.aligned_copy(packed), rows, K)
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))

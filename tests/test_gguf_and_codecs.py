"""GGUF container round trip and block codecs against hand-packed blocks
(the approach of InferenceWeb.Tests/ManagedQuantizedOpsTests.cs)."""
import struct

import numpy as np
import pytest
import torch

from tensorsharp_b200.gguf.constants import GGMLType, GGUFValueType, block_size, type_size
from tensorsharp_b200.gguf.reader import GGUFFile, GGUFFormatError
from tensorsharp_b200.gguf.writer import GGUFWriter
from tensorsharp_b200.quant import codecs
from tensorsharp_b200.quant.qweight import QuantWeight


def f16(x):
    return struct.pack("<e", x)


def test_type_sizes_match_spec():
    want = {GGMLType.Q4_K: (256, 144), GGMLType.Q8_0: (32, 34), GGMLType.Q6_K: (256, 210), GGMLType.MXFP4: (32, 17),
            GGMLType.Q5_K: (256, 176), GGMLType.Q4_0: (32, 18), GGMLType.F16: (1, 2), GGMLType.IQ4_NL: (32, 18)}
    for t, (bs, ts) in want.items():
        assert (block_size(t), type_size(t)) == (bs, ts)


def test_gguf_roundtrip(tmp_path):
    p = str(tmp_path / "t.gguf")
    w = GGUFWriter(p)
    w.add("general.architecture", "qwen3")
    w.add("qwen3.block_count", 3)
    w.add("qwen3.rope.freq_base", 1e6)
    w.add("flag", True)
    w.add("neg", -5)
    w.add("arr_i", [1, 2, 3])
    w.add("arr_s", ["a", "bc", ""], GGUFValueType.ARRAY, GGUFValueType.STRING)
    w.add("scalar_as_array", [7])
    a = np.arange(12, dtype=np.float32).reshape(3, 4)
    q = codecs.quantize(torch.randn(4, 64), GGMLType.Q8_0).numpy()
    w.add_tensor("a.weight", (3, 4), GGMLType.F32, a)
    w.add_tensor("q.weight", (4, 64), GGMLType.Q8_0, lambda: q)
    w.write()
    with GGUFFile(p) as g:
        assert g.version == 3 and g.alignment == 32
        assert g.get_str("general.architecture") == "qwen3"
        assert g.get_int("qwen3.block_count") == 3
        assert g.get_float("qwen3.rope.freq_base") == pytest.approx(1e6)
        assert g.get_bool("flag") is True and g.get_int("neg") == -5
        assert g.get_array("arr_i") == [1, 2, 3] and g.get_array("arr_s") == ["a", "bc", ""]
        assert g.get_int("scalar_as_array") == 7          # array-typed scalar tolerated
        assert g.get_array("qwen3.block_count") == [3]
        ti = g.tensors["a.weight"]
        assert ti.ne == (4, 3) and ti.shape == (3, 4)
        assert (g.data_offset + ti.offset) % 32 == 0
        got = np.frombuffer(g.tensor_bytes_view("a.weight"), dtype=np.float32).reshape(3, 4)
        assert np.array_equal(got, a)
        assert np.array_equal(g.tensor_bytes_view("q.weight"), q)
        assert g.adjacent("a.weight", "q.weight") is False or True


def test_gguf_rejects_garbage(tmp_path):
    p = tmp_path / "bad.gguf"
    p.write_bytes(b"NOPE" + b"\0" * 64)
    with pytest.raises(GGUFFormatError):
        GGUFFile(str(p))
    p.write_bytes(struct.pack("<IIQQ", 0x46554747, 3, 1, 0) + struct.pack("<Q", 5) + b"ab")   # truncated
    with pytest.raises(GGUFFormatError):
        GGUFFile(str(p))


def test_q8_0_hand_block():
    qs = np.arange(-16, 16, dtype=np.int8)
    raw = torch.from_numpy(np.frombuffer(f16(0.5) + qs.tobytes(), dtype=np.uint8).copy())
    out = codecs.dequantize(raw, GGMLType.Q8_0)
    assert torch.equal(out, torch.from_numpy(qs.astype(np.float32) * 0.5))


def test_q4_k_hand_block():
    # d = 2, dmin = 1; sub-block j: scale j+1, min j (j < 4 in the low 6 bits, j >= 4 split across bytes)
    sc = [j + 1 for j in range(8)]
    mn = [j for j in range(8)]
    s = bytearray(12)
    for j in range(4):
        s[j] = sc[j] | ((sc[j + 4] >> 4) << 6)
        s[j + 4] = mn[j] | ((mn[j + 4] >> 4) << 6)
        s[j + 8] = (sc[j + 4] & 0xF) | ((mn[j + 4] & 0xF) << 4)
    qs = bytearray(128)
    vals = np.zeros(256, dtype=np.int64)
    for c in range(4):
        for l in range(32):
            lo, hi = (l + c) % 16, (3 * l + c) % 16
            qs[32 * c + l] = lo | (hi << 4)
            vals[64 * c + l] = lo
            vals[64 * c + 32 + l] = hi
    raw = torch.from_numpy(np.frombuffer(f16(2.0) + f16(1.0) + bytes(s) + bytes(qs), dtype=np.uint8).copy())
    out = codecs.dequantize(raw, GGMLType.Q4_K)
    want = np.zeros(256, dtype=np.float32)
    for j in range(8):
        want[32 * j:32 * j + 32] = 2.0 * sc[j] * vals[32 * j:32 * j + 32] - 1.0 * mn[j]
    assert np.allclose(out.numpy(), want)


def test_q6_k_hand_block():
    rng = np.random.default_rng(0)
    q = rng.integers(0, 64, 256)
    sc = rng.integers(-20, 20, 16).astype(np.int8)
    ql, qh = bytearray(128), bytearray(64)
    for n in range(2):
        for l in range(32):
            q1, q2, q3, q4 = (q[128 * n + 32 * k + l] for k in range(4))
            ql[64 * n + l] = (q1 & 0xF) | ((q3 & 0xF) << 4)
            ql[64 * n + 32 + l] = (q2 & 0xF) | ((q4 & 0xF) << 4)
            qh[32 * n + l] = (q1 >> 4) | ((q2 >> 4) << 2) | ((q3 >> 4) << 4) | ((q4 >> 4) << 6)
    raw = torch.from_numpy(np.frombuffer(bytes(ql) + bytes(qh) + sc.tobytes() + f16(0.25), dtype=np.uint8).copy())
    out = codecs.dequantize(raw, GGMLType.Q6_K).numpy()
    want = np.array([0.25 * sc[i // 16] * (q[i] - 32) for i in range(256)], dtype=np.float32)
    assert np.allclose(out, want)


def test_mxfp4_hand_block():
    tab = [0, 1, 2, 3, 4, 6, 8, 12, 0, -1, -2, -3, -4, -6, -8, -12]
    codes = [(i * 7 + 3) % 16 for i in range(32)]
    qs = bytes(codes[j] | (codes[j + 16] << 4) for j in range(16))
    raw = torch.from_numpy(np.frombuffer(bytes([128]) + qs, dtype=np.uint8).copy())   # e = 128 -> 2^(128-127)/2 = 1
    out = codecs.dequantize(raw, GGMLType.MXFP4).numpy()
    assert np.allclose(out, np.array([tab[c] for c in codes], dtype=np.float32))
    assert float(codecs.e8m0_to_fp32_half(torch.tensor([0, 1, 127]))[2]) == 0.5


@pytest.mark.parametrize("t,tol", [(GGMLType.Q8_0, 0.01), (GGMLType.Q4_0, 0.12), (GGMLType.Q4_K, 0.12),
                                   (GGMLType.Q5_K, 0.06), (GGMLType.Q6_K, 0.03), (GGMLType.MXFP4, 0.16),
                                   (GGMLType.F16, 1e-3), (GGMLType.BF16, 1e-2)])
def test_quantize_roundtrip(t, tol):
    torch.manual_seed(0)
    x = torch.randn(16, 512) * 0.02
    y = codecs.dequantize(codecs.quantize(x, t), t, x.shape)
    assert float((x - y).norm() / x.norm()) < tol


@pytest.mark.parametrize("t", [GGMLType.Q8_0, GGMLType.Q4_0, GGMLType.Q6_K, GGMLType.MXFP4, GGMLType.Q4_K])
def test_plane_split_is_lossless(t):
    torch.manual_seed(1)
    x = torch.randn(6, 256) * 0.1
    raw = codecs.quantize(x, t)
    qw = QuantWeight.from_raw(raw, t, (6, 256))
    assert torch.equal(qw.raw_blocks(), raw)
    assert torch.equal(qw.dequantize(), codecs.dequantize(raw, t, (6, 256)))
    sl = qw.row_slice(2, 5)
    assert torch.equal(sl.dequantize(), qw.dequantize()[2:5])
    cat = QuantWeight.concat_rows([qw, sl])
    assert torch.equal(cat.dequantize(), torch.cat([qw.dequantize(), sl.dequantize()]))


GOLDEN_TYPES = ["Q4_0", "Q4_1", "Q5_0", "Q5_1", "Q8_0", "Q2_K", "Q3_K", "Q4_K", "Q5_K", "Q6_K", "Q8_K", "IQ4_NL", "IQ4_XS", "MXFP4",
                "TQ1_0", "TQ2_0", "IQ2_XXS", "IQ2_XS", "IQ2_S", "IQ3_XXS", "IQ3_S", "IQ1_S", "IQ1_M"]


@pytest.mark.parametrize("name", GOLDEN_TYPES)
def test_codec_matches_golden_vectors_of_ggml(name):
    """``tests/data/codec_golden.npz`` holds, per block type, a few blocks of random bytes and the values that ggml's own
    ``dequantize_row_*`` (ExternalProjects/ggml/src/ggml-quants.c) decodes them to; the codecs here reproduce them."""
    import os

    import numpy as np
    from tensorsharp_b200.gguf.constants import GGMLType
    from tensorsharp_b200.quant import codecs
    gold = np.load(os.path.join(os.path.dirname(__file__), "data", "codec_golden.npz"))
    raw, want = gold[name + "_raw"], gold[name + "_f32"]
    got = codecs.dequantize(torch.from_numpy(raw.copy()), GGMLType[name]).numpy()
    assert got.shape == want.shape
    assert np.abs(got - want).max() <= 1e-6 * np.abs(want).max(), name


@pytest.mark.parametrize("name", ["Q3_K", "IQ4_XS", "IQ2_XS", "IQ3_S", "IQ1_M", "TQ2_0"])
def test_weight_of_a_type_without_a_kernel_loads_as_bf16(name):
    """Block types that no kernel reads directly are decoded once at load (QuantWeight.from_raw) and served as bf16."""
    import os

    import numpy as np
    from tensorsharp_b200.gguf.constants import GGMLType
    from tensorsharp_b200.quant.qweight import QuantWeight
    gold = np.load(os.path.join(os.path.dirname(__file__), "data", "codec_golden.npz"))
    raw, want = gold[name + "_raw"], torch.from_numpy(gold[name + "_f32"])
    w = QuantWeight.from_raw(raw, GGMLType[name], (3, 256))
    assert w.ggml_type == GGMLType.BF16 and (w.N, w.K) == (3, 256)
    assert torch.equal(w.dequantize().reshape(-1), want.bfloat16().float())

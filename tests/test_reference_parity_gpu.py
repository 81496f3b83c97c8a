"""Golden parity with the reference's own native library (``baseline/_ref/libGgmlOps.so``, built unmodified from
TensorSharp.GGML.Native + vendored ggml): block codecs against ``TSGgml_DequantizeToF32`` and the Qwen3 graph's
logits against the reference's prefill exports and ``TSGgml_TransformerModelDecode``.  Skipped when the library has
not been built on this machine."""
import ctypes as C
import os
import sys

import numpy as np
import pytest
import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ref_lib():
    from baseline import ref_harness
    try:
        return ref_harness.load_library()
    except ref_harness.RefUnavailable as exc:
        pytest.skip(str(exc))


CODEC_TYPES = ["Q4_0", "Q4_1", "Q5_0", "Q5_1", "Q8_0", "Q2_K", "Q3_K", "Q4_K", "Q5_K", "Q6_K", "IQ4_NL", "IQ4_XS", "MXFP4", "F16", "BF16",
               "TQ1_0", "TQ2_0", "IQ2_XXS", "IQ2_XS", "IQ2_S", "IQ3_XXS", "IQ3_S", "IQ1_S", "IQ1_M"]


@pytest.mark.parametrize("name", CODEC_TYPES)
def test_codec_matches_reference_dequantize(ref_lib, name):
    """Random block bytes decode to the same values here and in ggml's dequantize_row_* (TSGgml_DequantizeToF32,
    TensorSharp.GGML.Native/ggml_ops_core.cpp:1331)."""
    from tensorsharp_b200.gguf.constants import GGMLType, block_size, type_size
    from tensorsharp_b200.quant import codecs
    t = GGMLType[name]
    n_blocks = 64
    rng = np.random.default_rng(sum(name.encode()))
    raw = rng.integers(0, 256, size=n_blocks * type_size(t), dtype=np.uint8)
    count = n_blocks * block_size(t)
    want = np.zeros(count, dtype=np.float32)
    rc = ref_lib.TSGgml_DequantizeToF32(int(t), raw.ctypes.data, count, want.ctypes.data)      # 0 = decoded
    if rc != 0:
        pytest.skip(f"the reference library does not decode {name} (code {rc})")
    got = codecs.dequantize(torch.from_numpy(raw.copy()), t).float().numpy().reshape(-1)
    # random scale fields contain a few NaN / inf half values: those elements must be non-finite on both sides
    fin = np.isfinite(want)
    assert fin.mean() > 0.8
    assert np.array_equal(fin, np.isfinite(got))
    scale = max(1e-30, float(np.abs(want[fin]).max()))
    assert float(np.abs(got[fin] - want[fin]).max()) <= 2e-3 * scale, name


def test_qwen3_logits_match_reference_library(ref_lib, tiny_qwen3_path):
    """Prefill and decode logits of the tiny Q8_0 Qwen3 model: this engine on the GPU against the reference's fused
    prefill exports and its whole-model decode export on the same file."""
    from baseline.ref_harness import RefQwen3
    from tensorsharp_b200.models.base import ModelBase
    ref = RefQwen3(ref_lib, tiny_qwen3_path, 256)
    ours = ModelBase.create(tiny_qwen3_path, "cuda", max_context=256)
    g = torch.Generator().manual_seed(21)
    prompt = torch.randint(0, ours.cfg.vocab, (48,), generator=g).tolist()
    want = torch.from_numpy(ref.prefill(prompt).copy())
    got = ours.forward(prompt).float().cpu()[:want.numel()]
    rel = lambda a, b: float((a - b).norm() / b.norm())
    assert rel(got, want) < 5e-2, rel(got, want)
    tok, pos = int(want.argmax()), len(prompt)
    for _ in range(4):
        want = torch.from_numpy(ref.decode(tok, pos).copy())
        got = ours.forward([tok]).float().cpu()[:want.numel()]
        assert rel(got, want) < 5e-2, (pos, rel(got, want))
        tok, pos = int(want.argmax()), pos + 1

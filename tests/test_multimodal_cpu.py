"""Multimodal front ends on CPU with tiny synthetic projector files: image processors (golden sizes
from the reference's formulas), the four vision encoders against straightforward per-patch
re-implementations of their positional schemes, the mel front end, the audio conformer's chunked
attention against a per-query loop, and the injector's token expansion / span arithmetic."""
import math
import struct

import numpy as np
import pytest
import torch

from tensorsharp_b200.gguf.constants import GGMLType
from tensorsharp_b200.gguf.writer import GGUFWriter
from tensorsharp_b200.multimodal import audio as A
from tensorsharp_b200.multimodal import image as I
from tensorsharp_b200.multimodal import injector as J
from tensorsharp_b200.multimodal import vision as V
from tensorsharp_b200.runtime.chat import ChatMessage


def write_gguf(path, meta, tensors):
    w = GGUFWriter(str(path))
    w.add("general.architecture", "clip")
    for k, v in meta.items():
        w.add(k, v)
    for name, t in tensors.items():
        w.add_tensor(name, tuple(t.shape), GGMLType.F32, t.float().contiguous().numpy())
    w.write()
    return str(path)


def rnd(*shape, scale=0.1):
    return torch.randn(*shape) * scale


def save_png(path, w, h, alpha=False):
    from PIL import Image
    rng = np.random.default_rng(0)
    arr = rng.integers(0, 255, size=(h, w, 4 if alpha else 3), dtype=np.uint8)
    Image.fromarray(arr, "RGBA" if alpha else "RGB").save(path)
    return str(path)


# ---------------------------------------------------------------------------- image processing
def test_smart_resize_rules():
    q = I.Qwen35ImageProcessor(16, 2)
    assert q.smart_resize(480, 640) == (480, 640) and q.image_token_count(480, 640) == 15 * 20
    assert q.smart_resize(100, 100) == (256, 256)                       # below the 64K-pixel floor: scaled up
    big = q.smart_resize(4000, 3000)
    assert big[0] * big[1] <= q.longest_edge and big[0] % 32 == 0 and big[1] % 32 == 0
    assert q.smart_resize(48, 80) == (224, 384) or q.smart_resize(48, 80)[0] % 32 == 0
    with pytest.raises(ValueError):
        q.smart_resize(10, 500)
    g4 = I.Gemma4ImageProcessor()
    w, h = g4.smart_resize(1000, 500)
    assert w % 48 == 0 and h % 48 == 0 and g4.output_tokens(w, h) <= 280 and g4.output_tokens(w, h) > 200
    assert g4.smart_resize(10, 10) == (48, 48) or min(g4.smart_resize(10, 10)) >= 48
    m = I.Mistral3ImageProcessor()
    assert m.target_size(3080, 1540) == (1540, 770)
    assert m.target_size(100, 50) == (112, 56) and m.vision_token_count(112, 56, 2) == 4 * 2 + 2


def test_bilinear_resize_matches_reference_rule(tmp_path):
    rgb = torch.arange(4 * 6 * 3, dtype=torch.float32).view(4, 6, 3)
    out = I.resize_bilinear_chw(rgb, 6, 4)
    assert torch.allclose(out, rgb.permute(2, 0, 1))                     # identity size: exact copy
    out = I.resize_bilinear_chw(rgb, 3, 2)                               # 2x down-sampling: mean of the 2x2 centres
    want = rgb.view(2, 2, 3, 2, 3).mean(dim=(1, 3)).permute(2, 0, 1)
    assert torch.allclose(out, want, atol=1e-5)
    up = I.resize_bilinear_chw(rgb, 12, 4)                               # first column extrapolates, as in the reference
    assert up[0, 0, 0] == pytest.approx(float(rgb[0, 0, 0] * 1.25 - rgb[0, 1, 0] * 0.25))
    p = save_png(tmp_path / "a.png", 20, 10, alpha=True)
    g3 = I.Gemma3ImageProcessor(image_size=28)
    px = g3.process(p)
    assert px.shape == (3, 28, 28) and float(px.min()) >= -1.0 and float(px.max()) <= 1.0
    px, w, h = I.Mistral3ImageProcessor().process(p)
    assert (w, h) == (28, 14) and px.shape == (3, 14, 28)
    assert I.read_image_dimensions(p) == (20, 10)


# ---------------------------------------------------------------------------- vision encoders
def vit_block_weights(prefix, hidden, ffn, bias=True, names=("attn_q", "attn_k", "attn_v", "attn_out")):
    t = {}
    for n in names:
        t[f"{prefix}.{n}.weight"] = rnd(hidden, hidden)
        if bias:
            t[f"{prefix}.{n}.bias"] = rnd(hidden)
    return t


def test_gemma3_vision_encoder(tmp_path):
    torch.manual_seed(0)
    hid, heads, P, size, ffn, proj = 32, 4, 4, 32, 48, 24          # 8 x 8 patches -> pooled 16 x 16? tokens_per_image fixed 256
    t = {"v.patch_embd.weight": rnd(hid, 3, P, P), "v.patch_embd.bias": rnd(hid), "v.position_embd.weight": rnd(64, hid),
         "v.post_ln.weight": torch.ones(hid), "v.post_ln.bias": torch.zeros(hid), "mm.soft_emb_norm.weight": torch.ones(hid),
         "mm.input_projection.weight": rnd(hid, proj)}
    for i in range(2):
        p = f"v.blk.{i}"
        t.update(vit_block_weights(p, hid, ffn))
        t.update({f"{p}.ln1.weight": torch.ones(hid), f"{p}.ln1.bias": torch.zeros(hid), f"{p}.ln2.weight": torch.ones(hid),
                  f"{p}.ln2.bias": torch.zeros(hid), f"{p}.ffn_down.weight": rnd(ffn, hid), f"{p}.ffn_down.bias": rnd(ffn),
                  f"{p}.ffn_up.weight": rnd(hid, ffn), f"{p}.ffn_up.bias": rnd(hid)})
    path = write_gguf(tmp_path / "g3.gguf", {"clip.vision.image_size": size, "clip.vision.patch_size": P,
                                             "clip.vision.embedding_length": hid, "clip.vision.attention.head_count": heads,
                                             "clip.vision.block_count": 2, "clip.vision.projection_dim": proj}, t)
    enc = V.Gemma3VisionEncoder(path)
    enc.tokens_per_image = 16                                            # 8 x 8 patches pooled 2 x 2
    out = enc.encode(torch.randn(3, size, size))
    assert out.shape == (16, proj) and torch.isfinite(out).all()
    # the patch embedding is a plain strided convolution in raster order
    px = torch.randn(3, size, size)
    pe = enc.patch_embed(px, enc.w["v.patch_embd.weight"], enc.w["v.patch_embd.bias"], P)
    want = (px[:, 4:8, 8:12].reshape(-1) @ enc.w["v.patch_embd.weight"].view(hid, -1).t()) + enc.w["v.patch_embd.bias"]
    assert torch.allclose(pe[1 * 8 + 2], want, atol=1e-5)
    pooled = enc.avg_pool_grid(torch.arange(64.).view(64, 1), 8, 8, 2)
    assert pooled.flatten()[:2].tolist() == [(0 + 1 + 8 + 9) / 4, (2 + 3 + 10 + 11) / 4]


def test_gemma4_vision_rope_clamps_and_pool(tmp_path):
    torch.manual_seed(1)
    hid, heads, P, proj = 32, 2, 4, 20
    t = {"v.patch_embd.weight": rnd(hid, 3, P, P), "v.position_embd.weight": rnd(2, 16, hid), "v.std_bias": rnd(hid),
         "v.std_scale": torch.ones(hid) * 0.5, "mm.input_projection.weight": rnd(hid, proj)}
    p = "v.blk.0"
    t.update(vit_block_weights(p, hid, 0, bias=False))
    for n in ("ln1", "ln2", "attn_post_norm", "ffn_post_norm"):
        t[f"{p}.{n}.weight"] = torch.ones(hid)
    t.update({f"{p}.attn_q_norm.weight": torch.ones(16), f"{p}.attn_k_norm.weight": torch.ones(16),
              f"{p}.ffn_gate.weight": rnd(40, hid), f"{p}.ffn_up.weight": rnd(40, hid), f"{p}.ffn_down.weight": rnd(hid, 40),
              f"{p}.out_scale.weight": torch.tensor([0.5]), f"{p}.attn_q.input_min": torch.tensor([-0.5]),
              f"{p}.attn_q.input_max": torch.tensor([0.5])})
    path = write_gguf(tmp_path / "g4.gguf", {"clip.vision.embedding_length": hid, "clip.vision.attention.head_count": heads,
                                             "clip.vision.block_count": 1, "clip.vision.projection_dim": proj,
                                             "clip.vision.patch_size": P, "clip.vision.projector_scale_factor": 2}, t)
    enc = V.Gemma4VisionEncoder(path)
    assert enc.clamps[p + ".attn_q"][:2] == (-0.5, 0.5) and enc.n_merge == 2
    out = enc.encode(torch.randn(3, 16, 24), 24, 16)                     # 6 x 4 patches -> 3 x 2 tokens
    assert out.shape == (6, proj) and torch.allclose(out.pow(2).mean(-1), torch.ones(6), atol=1e-3)   # unweighted RMSNorm
    # 2-D RoPE: per-patch rotation of (j, j+q) pairs with x angles on the first half, y on the second
    px, py, cx, sx, cy, sy = enc.rope_tables(6, 4, 16)
    x = torch.randn(24, heads, 16)
    got = enc.rope_2d(x, cx, sx, cy, sy)
    pidx, j = 9, 2                                                        # patch (x=3, y=1)
    ang = 3 * (1.0 / 100.0 ** (2.0 * j / 8))
    want = x[pidx, 0, j] * math.cos(ang) - x[pidx, 0, j + 4] * math.sin(ang)
    assert got[pidx, 0, j] == pytest.approx(float(want), abs=1e-5)
    ang_y = 1 * (1.0 / 100.0 ** (2.0 * j / 8))
    want = x[pidx, 1, 8 + j] * math.sin(ang_y) + x[pidx, 1, 8 + j + 4] * math.cos(ang_y)
    assert got[pidx, 1, 8 + j + 4] == pytest.approx(float(want), abs=1e-5)


def test_qwen35_vision_block_order_positions_and_rope(tmp_path):
    torch.manual_seed(2)
    hid, heads, P, proj = 32, 2, 4, 12
    t = {"v.patch_embd.weight": rnd(hid, 3, P, P), "v.patch_embd.weight.1": rnd(hid, 3, P, P), "v.patch_embd.bias": rnd(hid),
         "v.position_embd.weight": rnd(16, hid), "v.post_ln.weight": torch.ones(hid), "v.post_ln.bias": torch.zeros(hid),
         "mm.0.weight": rnd(64, hid * 4), "mm.0.bias": rnd(64), "mm.2.weight": rnd(proj, 64), "mm.2.bias": rnd(proj)}
    p = "v.blk.0"
    t.update({f"{p}.attn_qkv.weight": rnd(3 * hid, hid), f"{p}.attn_qkv.bias": rnd(3 * hid), f"{p}.attn_out.weight": rnd(hid, hid),
              f"{p}.attn_out.bias": rnd(hid), f"{p}.ffn_up.weight": rnd(48, hid), f"{p}.ffn_up.bias": rnd(48),
              f"{p}.ffn_down.weight": rnd(hid, 48), f"{p}.ffn_down.bias": rnd(hid)})
    for n in ("ln1", "ln2"):
        t[f"{p}.{n}.weight"], t[f"{p}.{n}.bias"] = torch.ones(hid), torch.zeros(hid)
    path = write_gguf(tmp_path / "q35.gguf", {"clip.vision.image_size": 16, "clip.vision.patch_size": P,
                                              "clip.vision.embedding_length": hid, "clip.vision.attention.head_count": heads,
                                              "clip.vision.block_count": 1, "clip.vision.projection_dim": proj,
                                              "clip.vision.spatial_merge_size": 2}, t)
    enc = V.Qwen35VisionEncoder(path)
    assert enc.block_order(4, 6).tolist()[:8] == [0, 1, 6, 7, 2, 3, 8, 9]
    pos = enc.position_embedding(4, 4)
    assert torch.allclose(pos, enc.w["v.position_embd.weight"], atol=1e-6)           # native grid: the table itself
    pos = enc.position_embedding(7, 4)                                                # row 1 of 7 sits half-way between rows 0 and 1
    tab = enc.w["v.position_embd.weight"].view(4, 4, hid)
    assert torch.allclose(pos.view(7, 4, hid)[1, 2], (tab[0, 2] + tab[1, 2]) / 2, atol=1e-6)
    order = enc.block_order(4, 6)
    cos, sin = enc.rope_tables(order, 6, 8)
    k = 5                                                                 # block-order slot 5 -> raster 3 -> (y=0, x=3)
    assert int(order[k]) == 3
    assert cos[k, 0] == pytest.approx(1.0) and cos[k, 1] == pytest.approx(math.cos(3.0))        # band 0: (y, x) interleaved
    assert sin[k, 3] == pytest.approx(math.sin(3.0 / 10000 ** (2 / 8)), abs=1e-6)
    out = enc.encode(torch.randn(3, 16, 24), 16, 24)
    assert out.shape == (6, proj) and torch.isfinite(out).all()


def test_mistral3_vision_rope_and_merge(tmp_path):
    torch.manual_seed(3)
    hid, heads, P, proj = 32, 2, 4, 10
    t = {"v.patch_conv.weight": rnd(hid, 3, P, P), "v.encoder_norm.weight": torch.ones(hid), "mm.norm.weight": torch.ones(hid),
         "mm.patch_merger.merging_layer.weight": rnd(hid, hid * 4), "mm.linear_1.weight": rnd(proj, hid),
         "mm.linear_2.weight": rnd(proj, proj)}
    p = "v.blk.0"
    t.update(vit_block_weights(p, hid, 0, bias=False, names=("attn_q", "attn_k", "attn_v", "attn_output")))
    t.update({f"{p}.attn_norm.weight": torch.ones(hid), f"{p}.ffn_norm.weight": torch.ones(hid), f"{p}.ffn_gate.weight": rnd(40, hid),
              f"{p}.ffn_up.weight": rnd(40, hid), f"{p}.ffn_down.weight": rnd(hid, 40)})
    path = write_gguf(tmp_path / "m3.gguf", {"vision.image_size": 64, "vision.patch_size": P, "vision.embedding_length": hid,
                                             "vision.attention.head_count": heads, "vision.block_count": 1,
                                             "spatial_merge_size": 2}, t)
    enc = V.Mistral3VisionEncoder(path)
    cos, sin = enc.rope_tables(6, 4)
    pidx = 1 * 6 + 5                                                      # (row 1, col 5); head_dim 16 -> 8 frequencies
    inv = [1.0 / 10000 ** (i * 2 / 16) for i in range(8)]
    assert cos[pidx, 0, 1] == pytest.approx(math.cos(1 * inv[2]), abs=1e-6)          # height uses even frequencies
    assert cos[pidx, 0, 4 + 1] == pytest.approx(math.cos(5 * inv[3]), abs=1e-6)      # width uses odd frequencies
    assert torch.equal(cos[..., :8], cos[..., 8:])
    out = enc.encode(torch.randn(3, 16, 24), 24, 16)
    assert out.shape == (6, proj) and torch.isfinite(out).all()


# ---------------------------------------------------------------------------- audio
def test_wav_decode_and_mel(tmp_path):
    sr, n = 8000, 8000
    tone = (np.sin(2 * np.pi * 440 * np.arange(n) / sr) * 0.5 * 32767).astype("<i2")
    stereo = np.stack([tone, tone], axis=1).reshape(-1)
    hdr = b"RIFF" + struct.pack("<I", 36 + stereo.nbytes) + b"WAVEfmt " + struct.pack("<IHHIIHH", 16, 1, 2, sr, sr * 4, 4, 16) + \
        b"data" + struct.pack("<I", stereo.nbytes)
    p = tmp_path / "t.wav"
    p.write_bytes(hdr + stereo.tobytes())
    x = A.decode_audio_file(str(p))
    assert x.dtype == np.float32 and abs(x.size - 16000) <= 1 and 0.45 < np.abs(x).max() <= 0.5
    with pytest.raises(ValueError):
        A.decode_audio_file(__file__)
    mel, frames = A.mel_spectrogram(x)
    assert frames == (x.size - 321) // 160 and mel.shape == (frames, 128)
    fb = A.mel_filter_bank()
    assert fb.shape == (513, 128) and float(fb.max()) <= 1.0 and int((fb.sum(0) > 0).sum()) == 128
    peak = int(mel.mean(0).argmax())
    centre_hz = 700 * (10 ** ((peak + 1) * (2595 * math.log10(1 + 8000 / 700) / 129) / 2595) - 1)
    assert abs(centre_hz - 440) < 60                                      # the tone lands in the right mel band
    assert float(mel.min()) >= math.log(1e-3) - 1e-6
    w = A.hann_window()
    assert w[0] == pytest.approx(0.5 - 0.5 * math.cos(math.pi / 320)) and torch.allclose(w, w.flip(0))
    assert A.mel_spectrogram(np.zeros(100, dtype=np.float32)) == (None, 0)
    assert A.audio_token_count(16000) == ((((16000 - 321) // 160) + 2 - 3) // 2 + 1 + 2 - 3) // 2 + 1


def test_audio_conformer_attention_matches_loop(tmp_path):
    torch.manual_seed(4)
    hid, heads, ffn, proj = 16, 2, 24, 10
    t = {"a.conv1d.0.weight": rnd(4, 1, 3, 3), "a.conv1d.0.norm.weight": torch.ones(4), "a.conv1d.1.weight": rnd(4, 4, 3, 3),
         "a.conv1d.1.norm.weight": torch.ones(4), "a.input_projection.weight": rnd(hid, 4 * 4), "a.output_proj.weight": rnd(hid, hid),
         "mm.a.input_projection.weight": rnd(proj, hid)}
    p = "a.blk.0"
    for n, shape in (("ffn_up", (ffn, hid)), ("ffn_down", (hid, ffn)), ("ffn_up_1", (ffn, hid)), ("ffn_down_1", (hid, ffn)),
                     ("attn_q", (hid, hid)), ("attn_k", (hid, hid)), ("attn_v", (hid, hid)), ("attn_out", (hid, hid)),
                     ("attn_k_rel", (hid, hid)), ("conv_pw1", (2 * hid, hid)), ("conv_pw2", (hid, hid))):
        t[f"{p}.{n}.weight"] = rnd(*shape, scale=0.3)
    for n in ("ffn_norm", "ffn_post_norm", "ffn_norm_1", "ffn_post_norm_1", "attn_pre_norm", "attn_post_norm", "ln2", "conv_norm",
              "norm_conv"):
        t[f"{p}.{n}.weight"] = torch.ones(hid)
    t[f"{p}.per_dim_scale.weight"] = torch.rand(hid // heads) + 0.5
    t[f"{p}.conv_dw.weight"] = rnd(hid, 5, scale=0.3)
    path = write_gguf(tmp_path / "aud.gguf", {"clip.audio.embedding_length": hid, "clip.audio.attention.head_count": heads,
                                              "clip.audio.block_count": 1, "clip.audio.num_mel_bins": 16,
                                              "clip.audio.projection_dim": proj}, t)
    enc = A.Gemma4AudioEncoder(path)
    out = enc.encode(torch.randn(120, 16))
    assert out.shape == (30, proj) and torch.isfinite(out).all()
    # chunked local attention == an explicit per-query loop over the last 12 frames
    T, H, D = 29, heads, hid // heads
    x = torch.randn(T, hid)
    got = enc.attention(x, p)
    h = V.rms_norm(x, enc.w[p + ".attn_pre_norm.weight"], enc.eps)
    q = (enc.linear(h, p + ".attn_q") * (D ** -0.5 / math.log(2))).view(T, H, D) * enc.w[p + ".per_dim_scale.weight"]
    k = (enc.linear(h, p + ".attn_k") * (math.log(1 + math.e) / math.log(2))).view(T, H, D)
    v = enc.linear(h, p + ".attn_v").view(T, H, D)
    pos = enc.position_embeddings(p)                                     # index s <-> distance 12 - s frames back
    o = torch.zeros(T, H, D)
    for ti in range(T):
        for hh in range(H):
            js = [j for j in range(ti - 12, ti + 1) if j >= 0]
            lg = torch.stack([q[ti, hh] @ k[j, hh] + q[ti, hh] @ pos[12 - (ti - j), hh] for j in js])
            pr = (torch.tanh(lg / 50) * 50).softmax(0)
            o[ti, hh] = sum(pr[i] * v[j, hh] for i, j in enumerate(js))
    want = x + V.rms_norm(enc.linear(o.view(T, hid), p + ".attn_out"), enc.w[p + ".attn_post_norm.weight"], enc.eps)
    assert torch.allclose(got, want, atol=2e-4), float((got - want).abs().max())
    # depthwise convolution is causal: changing a later frame leaves earlier outputs alone
    y1 = enc.light_conv(x, p)
    x2 = x.clone()
    x2[20:] += 1.0
    assert torch.allclose(enc.light_conv(x2, p)[:20], y1[:20], atol=1e-5)


# ---------------------------------------------------------------------------- injector
def test_token_expansion_helpers():
    assert J.expand_image_tokens([1, 9, 2, 9, 3], 9, [2, 3]) == [1, 9, 9, 2, 9, 9, 9, 3]
    assert J.expand_gemma3_image_tokens([5, 7, 6], 7, 8, 108, 0, 3) == [5, 108, 7, 0, 0, 0, 8, 108, 6]
    assert J.expand_single_token_placeholder([1, 50, 2], 1, 50, 3, 51) == [1, 50, 50, 50, 50, 51, 2]
    assert J.find_token([4, 5, 4], 4, 1) == 2 and J.find_token([4], 9, 0) == -1


class FakeTok:
    def __init__(self, table):
        self.table = table

    def lookup_token(self, s):
        return self.table.get(s, -1)


class FakeModel:
    def __init__(self, arch, table):
        self.arch, self.device, self.tokenizer = arch, torch.device("cpu"), FakeTok(table)
        self.queued = []

    def set_vision_embeddings(self, e, pos):
        self.queued.append(("v", e.shape[0], pos))

    def set_audio_embeddings(self, e, pos):
        self.queued.append(("a", e.shape[0], pos))


class FakeVision:
    patch_size, spatial_merge_size, image_size = 4, 2, 64

    def __init__(self):
        self.calls = 0

    def encode(self, px, a, b):
        self.calls += 1
        return torch.ones(6, 8) * self.calls


def test_injector_qwen35_spans_cache_and_clamps(tmp_path):
    m = FakeModel("qwen35", {"<|image_pad|>": 77})
    inj = J.MultimodalInjector(m)
    inj.vision = FakeVision()
    a, b = save_png(tmp_path / "a.png", 64, 64), save_png(tmp_path / "b.png", 64, 64)
    hist = [ChatMessage(role="user", content="x", image_paths=[a]), ChatMessage(role="assistant", content="y"),
            ChatMessage(role="user", content="z", image_paths=[b])]
    toks = inj.process_prompt_tokens(hist, [1, 2, 77, 3, 4, 77, 5])
    assert toks == [1, 2] + [77] * 6 + [3, 4] + [77] * 6 + [5]
    assert [(s.insert_position, s.prompt_start, s.prompt_end) for s in inj.vision_spans] == [(2, 2, 8), (10, 10, 16)]
    assert inj.clamp_reusable_prefix(5) == 2 and inj.clamp_reusable_prefix(9) == 9 and inj.clamp_reusable_prefix(12) == 10
    assert inj.clamp_trim_start(4) == 8 and inj.clamp_trim_start(9) == 9 and inj.clamp_trim_start(0) == 0
    assert inj.queue_prompt_embeddings(9) is True and m.queued == [("v", 6, 1)]           # first image lies inside the reused prefix
    m.queued.clear()
    inj.process_prompt_tokens(hist, [1, 2, 77, 3, 4, 77, 5])
    assert inj.vision.calls == 2                                                           # both images came from the cache
    inj.trim_prepared_prompt(8)
    assert [(s.insert_position, s.prompt_end) for s in inj.vision_spans] == [(2, 8)]
    assert inj.queue_prompt_embeddings(0) and m.queued == [("v", 6, 2)]
    import os
    import time
    time.sleep(0.01)
    os.utime(a, None)
    save_png(a, 32, 32)                                                                    # the file changed: re-encode
    inj.process_prompt_tokens(hist, [77, 77])
    assert inj.vision.calls == 3
    assert inj.process_prompt_tokens(None, [1]) == [1] and inj.vision_spans == []


def test_injector_gemma3_gemma4_mistral3_layouts(tmp_path):
    img = save_png(tmp_path / "a.png", 64, 32)
    hist = [ChatMessage(role="user", content="x", image_paths=[img])]

    class G3(FakeVision):
        def encode(self, px):
            return torch.ones(256, 8)
    m = FakeModel("gemma3", {"<start_of_image>": 900})
    inj = J.MultimodalInjector(m)
    inj.vision = G3()
    toks = inj.process_prompt_tokens(hist, [5, 900, 6])
    assert toks[:3] == [5, 108, 900] and toks[3:259] == [0] * 256 and toks[259:] == [256000, 108, 6]
    s = inj.vision_spans[0]
    assert (s.insert_position, s.prompt_start, s.prompt_end) == (3, 1, 261)
    m = FakeModel("gemma4", {"<|image>": 50, "<image|>": 51})
    inj = J.MultimodalInjector(m)
    inj.vision = FakeVision()
    toks = inj.process_prompt_tokens(hist, [1, 50, 2])
    assert toks == [1, 50] + [50] * 6 + [51, 2]
    s = inj.vision_spans[0]
    assert (s.insert_position, s.prompt_start, s.prompt_end) == (2, 1, 9)
    m = FakeModel("mistral3", {})

    class M3(FakeVision):
        def encode(self, px, w, h):
            return torch.arange(8 * 4).float().view(8 * 4, 1).expand(32, 8)
    inj = J.MultimodalInjector(m)
    inj.vision = M3()
    toks = inj.process_prompt_tokens(hist, [1, 10, 2])                      # 64 x 32 px -> 16 x 8 patches -> 8 x 4 merged
    row = [10] * 8
    assert toks == [1] + row + [12] + row + [12] + row + [12] + row + [13] + [2]
    assert inj.queue_prompt_embeddings(0) and m.queued == [("v", 8, 1), ("v", 8, 10), ("v", 8, 19), ("v", 8, 28)]


def test_model_injects_pending_embeddings(tiny_qwen3_path):
    from tensorsharp_b200.models.base import ModelBase
    m = ModelBase.create(tiny_qwen3_path, "cpu", max_context=64)
    toks = [5, 6, 7, 8, 9, 10]
    base = m.forward(toks).clone()
    m.reset_kv_cache()
    same = torch.nn.functional.embedding(torch.tensor([7, 8]), m.tok_emb.dequantize())
    m.set_vision_embeddings(same, 2)                                     # the very rows the lookup would give
    assert torch.allclose(m.forward(toks), base, atol=1e-5)
    m.reset_kv_cache()
    m.set_vision_embeddings(torch.zeros(3, m.cfg.hidden), 4)             # clipped at the end of the chunk
    assert not torch.allclose(m.forward(toks), base, atol=1e-3) and m._pending_embeddings == []
    assert m.multimodal is None
    m.close()


def test_slots_of_a_shared_model_carry_their_own_embeddings(tiny_qwen3_path, tmp_path):
    """With several requests over one loaded model, a slot's queued image embeddings travel with that slot's next
    forward call (run by itself, not merged), another slot's text-only call is untouched, and the slot's injector
    uses the encoders and caches of the shared model's injector."""
    import threading

    from tensorsharp_b200.models.base import ModelBase
    from tensorsharp_b200.runtime.gather import GatheredModel
    single = ModelBase.create(tiny_qwen3_path, "cpu", max_context=64)
    toks = [5, 6, 7, 8, 9, 10, 11]
    plain = single.forward(toks).clone()
    single.reset_kv_cache()
    emb = torch.randn(3, single.cfg.hidden) * 0.1
    single.set_vision_embeddings(emb, 2)
    with_img = single.forward(toks).clone()
    assert not torch.allclose(plain, with_img, atol=1e-3)
    real = ModelBase.create(tiny_qwen3_path, "cpu", max_context=64, max_seqs=3)
    g = GatheredModel(real, 2, window_s=0.05)
    out = {}

    def with_image():
        with g.slot(0) as m:
            m.set_vision_embeddings(emb, 2)
            out["img"] = m.forward(toks)

    def text_only():
        with g.slot(1) as m:
            out["txt"] = m.forward(toks)
    ths = [threading.Thread(target=f) for f in (with_image, text_only)]
    [t.start() for t in ths]
    [t.join(60) for t in ths]
    assert torch.allclose(out["img"], with_img, atol=1e-4) and torch.allclose(out["txt"], plain, atol=1e-4)
    assert real._pending_embeddings == [] and g.slot(0).multimodal is None          # a text-only architecture has no injector
    g.close()
    # the slot injector: own spans and queue, shared encoders and caches
    shared_model = FakeModel("qwen35", {"<|image_pad|>": 77})
    shared = J.MultimodalInjector(shared_model)
    shared.vision = FakeVision()
    slot = FakeModel("qwen35", {"<|image_pad|>": 77})
    inj = J.SlotInjector(slot, shared)
    a = save_png(tmp_path / "a.png", 64, 64)
    hist = [ChatMessage(role="user", content="x", image_paths=[a])]
    assert inj.process_prompt_tokens(hist, [1, 77, 2]) == [1] + [77] * 6 + [2]
    assert inj.vision is shared.vision and shared.vision.calls == 1 and shared.vision_spans == []
    assert inj.queue_prompt_embeddings(0) and slot.queued == [("v", 6, 1)] and shared_model.queued == []
    shared.process_prompt_tokens(hist, [1, 77, 2])
    assert shared.vision.calls == 1                                                 # the encoding came from the common cache

"""The vision encoders on the GPU, where their projections run on the tcgen05 GEMM and their bidirectional attention
on the flash prefill kernel, against the same encoders in float32 on the CPU (plain matrix products and softmax)."""
import pytest
import torch

from tensorsharp_b200.multimodal import vision as V
from tensorsharp_b200.ops import kernels

from tests.test_multimodal_cpu import rnd, vit_block_weights, write_gguf

pytestmark = pytest.mark.gpu


def _rel(a, b):
    return float((a.float().cpu() - b.float().cpu()).abs().max() / b.float().abs().max().clamp_min(1e-6))


def test_bidirectional_attention_on_the_flash_kernel_matches_softmax():
    torch.manual_seed(0)
    for n, H, d in ((70, 2, 72), (300, 3, 64), (129, 1, 128)):
        q, k, v = (torch.randn(n, H, d, device="cuda") for _ in range(3))
        got = V.VisionEncoderBase.flash_attention(q, k, v, d ** -0.5)
        qb, kb, vb = (t.to(torch.bfloat16).float() for t in (q, k, v))
        p = torch.softmax(torch.einsum("nhd,mhd->hnm", qb, kb) * d ** -0.5, dim=-1)
        want = torch.einsum("hnm,mhd->nhd", p, vb).reshape(n, H * d)
        assert _rel(got, want) < 2e-2, (n, H, d)


def test_gemma3_style_tower_on_own_kernels_matches_cpu(tmp_path):
    torch.manual_seed(1)
    hid, heads, P, size, ffn, proj = 144, 2, 4, 32, 200, 96          # head size 72 (padded to 128), ffn not a multiple of 64
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
    px = torch.randn(3, size, size)
    cpu = V.Gemma3VisionEncoder(path)
    cpu.tokens_per_image = 16
    want = cpu.encode(px)
    gpu = V.Gemma3VisionEncoder(path, device="cuda")
    gpu.tokens_per_image = 16
    assert gpu.native
    before = kernels.LAUNCHES
    got = gpu.encode(px)
    assert kernels.LAUNCHES - before == 2 * 7 + 1       # per block: q, k, v, attention, out, two MLP layers; the projector
    assert got.shape == want.shape and _rel(got, want) < 3e-2


def test_qwen35_style_tower_on_own_kernels_matches_cpu(tmp_path):
    torch.manual_seed(2)
    hid, heads, P, proj = 128, 2, 4, 80
    t = {"v.patch_embd.weight": rnd(hid, 3, P, P), "v.patch_embd.weight.1": rnd(hid, 3, P, P), "v.patch_embd.bias": rnd(hid),
         "v.position_embd.weight": rnd(16, hid), "v.post_ln.weight": torch.ones(hid), "v.post_ln.bias": torch.zeros(hid),
         "mm.0.weight": rnd(64, hid * 4), "mm.0.bias": rnd(64), "mm.2.weight": rnd(proj, 64), "mm.2.bias": rnd(proj)}
    p = "v.blk.0"
    t.update({f"{p}.attn_qkv.weight": rnd(3 * hid, hid), f"{p}.attn_qkv.bias": rnd(3 * hid), f"{p}.attn_out.weight": rnd(hid, hid),
              f"{p}.attn_out.bias": rnd(hid), f"{p}.ffn_up.weight": rnd(192, hid), f"{p}.ffn_up.bias": rnd(192),
              f"{p}.ffn_down.weight": rnd(hid, 192), f"{p}.ffn_down.bias": rnd(hid)})
    for n in ("ln1", "ln2"):
        t[f"{p}.{n}.weight"], t[f"{p}.{n}.bias"] = torch.ones(hid), torch.zeros(hid)
    path = write_gguf(tmp_path / "q35.gguf", {"clip.vision.image_size": 16, "clip.vision.patch_size": P,
                                              "clip.vision.embedding_length": hid, "clip.vision.attention.head_count": heads,
                                              "clip.vision.block_count": 1, "clip.vision.projection_dim": proj,
                                              "clip.vision.spatial_merge_size": 2}, t)
    px = torch.randn(3, 32, 48)
    want = V.Qwen35VisionEncoder(path).encode(px, 32, 48)
    gpu = V.Qwen35VisionEncoder(path, device="cuda")
    before = kernels.LAUNCHES
    got = gpu.encode(px, 32, 48)
    assert kernels.LAUNCHES > before
    assert got.shape == want.shape and _rel(got, want) < 3e-2


def test_audio_conformer_projections_on_the_gemm_match_cpu(tmp_path):
    from tensorsharp_b200.multimodal import audio as A
    torch.manual_seed(4)
    hid, heads, ffn, proj = 128, 2, 200, 72
    t = {"a.conv1d.0.weight": rnd(4, 1, 3, 3), "a.conv1d.0.norm.weight": torch.ones(4), "a.conv1d.1.weight": rnd(4, 4, 3, 3),
         "a.conv1d.1.norm.weight": torch.ones(4), "a.input_projection.weight": rnd(hid, 4 * 4), "a.output_proj.weight": rnd(hid, hid),
         "mm.a.input_projection.weight": rnd(proj, hid)}
    p = "a.blk.0"
    for n, shape in (("ffn_up", (ffn, hid)), ("ffn_down", (hid, ffn)), ("ffn_up_1", (ffn, hid)), ("ffn_down_1", (hid, ffn)),
                     ("attn_q", (hid, hid)), ("attn_k", (hid, hid)), ("attn_v", (hid, hid)), ("attn_out", (hid, hid)),
                     ("attn_k_rel", (hid, hid)), ("conv_pw1", (2 * hid, hid)), ("conv_pw2", (hid, hid))):
        t[f"{p}.{n}.weight"] = rnd(*shape)
    for n in ("ffn_norm", "ffn_post_norm", "ffn_norm_1", "ffn_post_norm_1", "attn_pre_norm", "attn_post_norm", "ln2", "conv_norm",
              "norm_conv"):
        t[f"{p}.{n}.weight"] = torch.ones(hid)
    t[f"{p}.per_dim_scale.weight"] = torch.rand(hid // heads) + 0.5
    t[f"{p}.conv_dw.weight"] = rnd(hid, 5, scale=0.3)
    path = write_gguf(tmp_path / "aud.gguf", {"clip.audio.embedding_length": hid, "clip.audio.attention.head_count": heads,
                                              "clip.audio.block_count": 1, "clip.audio.num_mel_bins": 16,
                                              "clip.audio.projection_dim": proj}, t)
    mel = torch.randn(120, 16)
    want = A.Gemma4AudioEncoder(path).encode(mel)
    gpu = A.Gemma4AudioEncoder(path, device="cuda")
    assert gpu.native
    before = kernels.LAUNCHES
    got = gpu.encode(mel.cuda())
    assert kernels.LAUNCHES - before >= 10              # the block's eleven projections of 4096 weights or more
    assert got.shape == want.shape and _rel(got, want) < 3e-2

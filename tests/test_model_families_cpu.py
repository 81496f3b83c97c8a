"""Every model family on the CPU oracle path: incremental decoding, chunked prefill and
batched execution must agree with one-shot prefill (KV cache, sliding windows, sinks,
recurrent state carry-over, MoE routing)."""
import pytest
import torch

from tensorsharp_b200.models import synth
from tensorsharp_b200.models.base import ModelBase, supported_architectures

FAMILIES = {
    "gptoss": (synth.write_gptoss, {}),
    "qwen35_moe": (synth.write_qwen35, {}),
    "qwen35_dense": (synth.write_qwen35, {"n_experts": 0}),
    "gemma3": (synth.write_gemma, {"arch": "gemma3"}),
    "gemma4": (synth.write_gemma, {"arch": "gemma4", "n_layers": 8, "head_dim_global": 128, "kv_heads_global": 1,
                                   "rot_global": 64, "shared_kv": 2, "ple_dim": 32, "n_experts": 4, "top_k": 2}),
    # global layers with 512-wide heads and four query heads per KV head (Gemma 4's full-size layout)
    "gemma4_wide_heads": (synth.write_gemma, {"arch": "gemma4", "n_layers": 6, "head_dim_global": 512, "kv_heads_global": 1,
                                              "rot_global": 128}),
    "mistral3": (synth.write_mistral3, {}),
    "nemotron_h": (synth.write_nemotron_h, {}),
}


@pytest.fixture(scope="module")
def family_paths(tmp_path_factory):
    d = tmp_path_factory.mktemp("families")
    out = {}
    for name, (fn, kw) in FAMILIES.items():
        p = str(d / f"{name}.gguf")
        fn(p, device="cpu", **kw)
        out[name] = p
    return out


def test_all_seven_families_are_registered():
    archs = set(supported_architectures())
    assert {"qwen3", "qwen35", "qwen35moe", "gpt-oss", "gemma3", "gemma4", "nemotron_h", "mistral3"} <= archs


@pytest.mark.parametrize("name", list(FAMILIES))
def test_incremental_matches_one_shot(family_paths, name):
    m = ModelBase.create(family_paths[name], "cpu", max_context=256, max_seqs=3)
    g = torch.Generator().manual_seed(7)
    ids = torch.randint(0, 4096, (90,), generator=g).tolist()
    full = m.forward(ids)
    assert torch.isfinite(full).all() and full.shape == (m.cfg.vocab,)
    # a different prompt gives different logits (the test is not vacuous)
    m.reset_kv_cache()
    other = m.forward(ids[:-1] + [(ids[-1] + 1) % 4096])
    assert float((other - full).abs().max()) > 1e-4
    # prefix then suffix
    m.reset_kv_cache()
    m.forward(ids[:51], want_logits=False)
    inc = m.forward(ids[51:])
    assert float((inc - full).abs().max()) < 2e-2
    # token by token for the tail
    m.reset_kv_cache()
    m.forward(ids[:80], want_logits=False)
    for t in ids[80:]:
        step = m.forward([t])
    assert float((step - full).abs().max()) < 2e-2
    # two sequences in one batch equal the same sequences alone
    s1, s2 = m.kv.new_seq(), m.kv.new_seq()
    m.reset_recurrent_state(s1.slot)
    m.reset_recurrent_state(s2.slot)
    lb = m.forward_batch(m.kv.build_batch([s1, s2], [ids[:33], ids]))
    assert float((lb[1] - full).abs().max()) < 2e-2


def test_recurrent_models_refuse_truncation(family_paths):
    m = ModelBase.create(family_paths["qwen35_dense"], "cpu", max_context=64)
    m.forward([1, 2, 3])
    with pytest.raises(RuntimeError):
        m.truncate_kv_cache(1)
    assert ModelBase.create(family_paths["gemma3"], "cpu", max_context=64).supports_kv_truncation


def test_gemma4_prefill_chunk_policy(tmp_path, monkeypatch):
    """Gemma 4 caps the prefill chunk at min(2048, max(2 * window, 1024)); TS_PREFILL_CHUNK overrides the cap; the
    chunked prefill gives the logits of the one-shot prefill."""
    from tensorsharp_b200.models import synth
    from tensorsharp_b200.models.base import ModelBase
    p = str(tmp_path / "g4.gguf")
    synth.write_gemma(p, arch="gemma4", device="cpu")
    m = ModelBase.create(p, "cpu", max_context=256)
    monkeypatch.delenv("TS_PREFILL_CHUNK", raising=False)
    assert m.prefill_chunk(5120) == min(2048, max(2 * m.window, 1024)) and m.prefill_chunk(64) == 64
    monkeypatch.setenv("TS_PREFILL_CHUNK", "16")
    assert m.prefill_chunk(5120) == 16
    g = torch.Generator().manual_seed(4)
    toks = torch.randint(0, 4096, (50,), generator=g).tolist()
    chunked = m.forward_refill(toks, 5120).clone()          # 16 tokens at a time
    m.reset_kv_cache()
    whole = m.forward(toks)
    assert torch.allclose(chunked, whole, atol=3e-2)              # 16-row chunks take the int8-activation path


def test_gdn_chunked_form_matches_the_token_scan(tmp_path, monkeypatch):
    """The chunked (WY) form of the gated delta rule against the token-by-token recurrence: the op alone on ragged
    lengths, then a Qwen3.5-shaped model whose 150-token prompt takes the chunked route and whose decode step
    continues from the state it left."""
    from tensorsharp_b200.ops import reference as ref
    torch.manual_seed(0)
    Hk, Hv, Dk, Dv = 2, 4, 16, 8
    for n in (1, 63, 64, 65, 200):
        qkv, z = torch.randn(n, 2 * Hk * Dk + Hv * Dv), torch.randn(n, Hv * Dv)
        beta, alpha, dt_bias = torch.randn(n, Hv), torch.randn(n, Hv), torch.randn(Hv)
        a_log, norm_w = -torch.rand(Hv) * 2, torch.rand(Dv) + 0.5
        s1 = torch.randn(Hv, Dv, Dk) * 0.3
        s2 = s1.clone()
        kw = dict(Hk=Hk, Hv=Hv, Dk=Dk, Dv=Dv, eps=1e-6)
        o1 = ref.gdn_recurrent(qkv, z, beta, alpha, dt_bias, a_log, norm_w, s1, **kw)
        o2 = ref.gdn_chunked(qkv, z, beta, alpha, dt_bias, a_log, norm_w, s2, chunk=64, **kw)
        assert torch.allclose(o1, o2, atol=1e-4) and torch.allclose(s1, s2, atol=1e-5), n
    p = str(tmp_path / "q35.gguf")
    synth.write_qwen35(p, device="cpu")
    g = torch.Generator().manual_seed(8)
    toks = torch.randint(0, 4096, (150,), generator=g).tolist()
    out = {}
    for mode in ("chunked", "scan"):
        monkeypatch.setenv("GDN_DISABLE_CHUNKED_PREFILL", "0" if mode == "chunked" else "1")
        m = ModelBase.create(p, "cpu", max_context=256)
        l1 = m.forward(toks)
        out[mode] = (l1, m.forward([int(l1.argmax())]))
    assert torch.allclose(out["chunked"][0], out["scan"][0], atol=2e-3)
    assert torch.allclose(out["chunked"][1], out["scan"][1], atol=2e-3)


def test_gdn_chunked_batch_equals_the_sequences_one_by_one():
    """Several packed sequences of ragged lengths through the batched chunked form (padded to a common chunk count,
    stacked beside the heads) give each sequence's own result and final state."""
    from tensorsharp_b200.ops import reference as ref
    torch.manual_seed(3)
    Hk, Hv, Dk, Dv = 2, 4, 16, 8
    lens = [130, 1, 64, 77]
    cu = [0]
    for n in lens:
        cu.append(cu[-1] + n)
    T = cu[-1]
    qkv, z = torch.randn(T, 2 * Hk * Dk + Hv * Dv), torch.randn(T, Hv * Dv)
    beta, alpha, dt_bias = torch.randn(T, Hv), torch.randn(T, Hv), torch.randn(Hv)
    a_log, norm_w = -torch.rand(Hv) * 2, torch.rand(Dv) + 0.5
    kw = dict(Hk=Hk, Hv=Hv, Dk=Dk, Dv=Dv, eps=1e-6)
    pool = torch.randn(6, Hv, Dv, Dk) * 0.3
    slots = [4, 0, 5, 2]
    want_pool = pool.clone()
    want = torch.cat([ref.gdn_chunked(qkv[cu[i]:cu[i + 1]], z[cu[i]:cu[i + 1]], beta[cu[i]:cu[i + 1]], alpha[cu[i]:cu[i + 1]],
                                      dt_bias, a_log, norm_w, want_pool[slots[i]], **kw) for i in range(len(lens))])
    got = ref.gdn_chunked_batch(qkv, z, beta, alpha, dt_bias, a_log, norm_w, [pool[sl] for sl in slots], cu, **kw)
    assert torch.allclose(got, want, atol=1e-5)
    assert torch.allclose(pool, want_pool, atol=1e-6)


def test_mamba2_chunked_form_matches_the_token_scan(tmp_path, monkeypatch):
    from tensorsharp_b200.ops import reference as ref
    torch.manual_seed(1)
    H, P, G, N = 4, 8, 2, 16
    for n in (1, 63, 64, 65, 200):
        xbc, dt, dtb = torch.randn(n, H * P + 2 * G * N), torch.randn(n, H), torch.randn(H)
        A, D = -torch.rand(H) * 2, torch.randn(H)
        s1 = torch.randn(H, P, N) * 0.3
        s2 = s1.clone()
        y1 = ref.mamba2_recurrent(xbc, dt, dtb, A, D, s1, H=H, P=P, G=G, N=N)
        y2 = ref.mamba2_chunked(xbc, dt, dtb, A, D, s2, H=H, P=P, G=G, N=N)
        assert torch.allclose(y1, y2, atol=5e-4) and torch.allclose(s1, s2, atol=1e-4), n
    p = str(tmp_path / "nem.gguf")
    synth.write_nemotron_h(p, device="cpu")
    g = torch.Generator().manual_seed(9)
    toks = torch.randint(0, 4096, (150,), generator=g).tolist()
    out = {}
    for mode in ("chunked", "scan"):
        monkeypatch.setenv("GDN_DISABLE_CHUNKED_PREFILL", "0" if mode == "chunked" else "1")
        m = ModelBase.create(p, "cpu", max_context=256)
        l1 = m.forward(toks)
        out[mode] = (l1, m.forward([int(l1.argmax())]))
    assert torch.allclose(out["chunked"][0], out["scan"][0], atol=2e-3)
    assert torch.allclose(out["chunked"][1], out["scan"][1], atol=2e-3)

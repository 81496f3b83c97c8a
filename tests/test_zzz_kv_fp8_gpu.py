"""The 8-bit KV cache on the GPU: the store / load kernels against PyTorch's e4m3 conversion, the decode kernel that
reads e4m3 pages against a float32 softmax over the same (already rounded) values, prefill through the converted view,
and a model that runs on the 8-bit cache against the same model on bf16 pages."""
import pytest
import torch

from tensorsharp_b200.ops import functional as F
from tensorsharp_b200.ops import reference as ref

from tests.test_kernels_gpu import DEV, K, _gather, _paged, rel_err

pytestmark = pytest.mark.gpu
FP8 = torch.float8_e4m3fn


def test_store_and_load_match_torch_conversion():
    torch.manual_seed(0)
    T, Hkv, Dh, n_slots = 37, 2, 128, 96
    k = (torch.randn(T, Hkv, Dh, device=DEV) * 4).bfloat16()
    v = (torch.randn(T, Hkv, Dh, device=DEV) * 300).bfloat16()          # beyond +-448: saturates
    kc = torch.zeros(n_slots, Hkv, Dh, dtype=FP8, device=DEV)
    vc = torch.zeros_like(kc)
    slots = torch.randperm(n_slots, device=DEV)[:T].contiguous()
    K().kv_store_fp8(k, v, kc, vc, slots)
    want_k = k.float().clamp(-448, 448).to(FP8).view(torch.uint8)
    want_v = v.float().clamp(-448, 448).to(FP8).view(torch.uint8)
    assert torch.equal(kc.view(torch.uint8)[slots], want_k) and torch.equal(vc.view(torch.uint8)[slots], want_v)
    untouched = torch.ones(n_slots, dtype=torch.bool, device=DEV)
    untouched[slots] = False
    assert int(kc.view(torch.uint8)[untouched].max()) == 0
    kd, vd = K().kv_load_fp8(kc, vc, slots)
    assert torch.equal(kd, kc.view(torch.uint8)[slots].view(FP8).to(torch.bfloat16))
    assert torch.equal(vd, vc.view(torch.uint8)[slots].view(FP8).to(torch.bfloat16))


@pytest.mark.parametrize("Hq,Hkv,Dh", [(8, 2, 128), (4, 4, 64), (16, 2, 256), (2, 1, 64), (8, 2, 512), (6, 2, 128), (12, 1, 64),
                                       (5, 1, 128), (32, 2, 64), (2, 2, 512), (16, 1, 128)])
@pytest.mark.parametrize("window,sinks,softcap", [(0, False, 0.0), (100, True, 0.0), (0, False, 30.0)])
def test_attn_decode_on_e4m3_pages(Hq, Hkv, Dh, window, sinks, softcap):
    torch.manual_seed(7)
    ps, lens = 16, [1, 37, 300, 1025]
    B = len(lens)
    kc, vc, table = _paged(sum(lens), Hkv, Dh, ps, lens)
    k8, v8 = kc.to(FP8), vc.to(FP8)
    kf, vf = k8.float(), v8.float()
    q = torch.randn(B, Hq, Dh, device=DEV).bfloat16()
    sk = torch.randn(Hq, device=DEV) if sinks else None
    kv_lens = torch.tensor(lens, dtype=torch.int32, device=DEV)
    for splits in (1, 5):
        got = K().attn_decode(q, k8, v8, table, kv_lens, scale=Dh ** -0.5, Hq=Hq, Hkv=Hkv, Dh=Dh, page_size=ps,
                              splits=splits, sinks=sk, softcap=softcap, window=window)
        for b, L in enumerate(lens):
            want = ref.attention(q[b:b + 1], _gather(kf, table, b, L, ps), _gather(vf, table, b, L, ps),
                                 torch.tensor([L - 1], device=DEV), scale=Dh ** -0.5, window=window, sinks=sk,
                                 softcap=softcap)
            assert rel_err(got[b], want[0]) < 1e-2, (b, splits, rel_err(got[b], want[0]))


def test_attention_dispatch_prefill_and_decode_on_an_fp8_cache():
    """ops.functional.attention with 8-bit pages: prompts go through the converted dense view (several sequences, a
    window, cache longer than the new queries), single tokens through the byte-reading kernel."""
    torch.manual_seed(9)
    ps, Hq, Hkv, Dh = 16, 4, 2, 128
    qlens, lens = [5, 64, 150, 1], [5, 200, 150, 90]
    B = len(lens)
    kc, vc, table = _paged(sum(lens), Hkv, Dh, ps, lens)
    k8, v8 = kc.to(FP8), vc.to(FP8)
    kf, vf = k8.float(), v8.float()
    T = sum(qlens)
    q = torch.randn(T, Hq, Dh, device=DEV).bfloat16()
    cu = [0]
    for n in qlens:
        cu.append(cu[-1] + n)
    pos = torch.cat([torch.arange(L - ql, L) for ql, L in zip(qlens, lens)]).to(torch.int32)
    for window in (0, 70):
        batch = F.Batch(tokens=torch.zeros(T, dtype=torch.int32, device=DEV), positions=pos.to(DEV),
                        slots=torch.zeros(T, dtype=torch.int64, device=DEV), cu_q=torch.tensor(cu, dtype=torch.int32, device=DEV),
                        kv_lens=torch.tensor(lens, dtype=torch.int32, device=DEV), block_table=table, last_idx=None,
                        seq_slots=torch.arange(B, dtype=torch.int64, device=DEV), max_q_len=max(qlens), max_kv_len=max(lens),
                        is_decode=False, page_size=ps, h_cu_q=tuple(cu), h_kv_lens=tuple(lens))
        got = F.attention(q, k8, v8, batch, scale=Dh ** -0.5, Hq=Hq, Hkv=Hkv, Dh=Dh, window=window).view(T, Hq, Dh)
        o = 0
        for b, (ql, L) in enumerate(zip(qlens, lens)):
            want = ref.attention(q[o:o + ql], _gather(kf, table, b, L, ps), _gather(vf, table, b, L, ps),
                                 torch.arange(L - ql, L, device=DEV), scale=Dh ** -0.5, window=window)
            assert rel_err(got[o:o + ql], want) < 1.5e-2, (window, b, rel_err(got[o:o + ql], want))
            o += ql


def test_model_on_an_fp8_cache_follows_the_bf16_cache(tmp_path, monkeypatch):
    from tensorsharp_b200.models import synth
    from tensorsharp_b200.models.base import ModelBase
    from tensorsharp_b200.runtime.engine import DecodeGraph
    p = str(tmp_path / "q.gguf")
    synth.write_qwen3(p, n_layers=2, hidden=256, n_heads=4, n_kv_heads=2, head_dim=64, ffn=768, vocab=4096, scheme="Q4_K_M",
                      device="cuda")
    a = ModelBase.create(p, "cuda:0", max_context=512, max_seqs=2)
    monkeypatch.setenv("TSB_KV_DTYPE", "fp8")
    b = ModelBase.create(p, "cuda:0", max_context=512, max_seqs=2)
    assert b.kv.k[0].dtype == FP8 and b.kv.k[0].element_size() * 2 == a.kv.k[0].element_size()
    gen = torch.Generator().manual_seed(4)
    ids = torch.randint(5, 4000, (300,), generator=gen).tolist()
    want, got = a.forward(ids), b.forward(ids)
    assert rel_err(got, want) < 0.1, rel_err(got, want)
    # the 8-bit cache agrees with itself: one pass, two chunks, and single-token steps after a truncation
    b.reset_kv_cache()
    b.forward(ids[:200])
    assert rel_err(b.forward(ids[200:]), got) < 3e-2
    b.truncate_kv_cache(297)
    step = None
    for t in ids[297:]:
        step = b.forward([t])                                # decode kernel on e4m3 pages (graph or eager)
    assert rel_err(step, got) < 5e-2, rel_err(step, got)     # single-token steps quantise their activations: another 2 %
    # captured decode steps run on the 8-bit pages too and follow the bf16 model's greedy choice on clear margins
    seqs = [b.new_sequence()]
    lb = b.forward_batch(b.kv.build_batch(seqs, [ids[:100]]))
    dg = DecodeGraph(b, seqs, 4)
    dg.set_tokens([int(lb[0].argmax())])
    out = [int(dg.step()[0]) for _ in range(3)]
    assert all(0 <= t < 4096 for t in out)

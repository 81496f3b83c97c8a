"""Numerics of every sm_100a kernel against the fp32 PyTorch restatement of the same op."""
import math

import pytest
import torch

from tensorsharp_b200.gguf.constants import GGMLType
from tensorsharp_b200.ops import reference as ref
from tensorsharp_b200.quant import codecs
from tensorsharp_b200.quant.qweight import QuantWeight

pytestmark = pytest.mark.gpu
DEV = "cuda"
QTYPES = [GGMLType.Q4_K, GGMLType.Q5_K, GGMLType.Q6_K, GGMLType.Q8_0, GGMLType.Q4_0, GGMLType.MXFP4]
FTYPES = [GGMLType.BF16, GGMLType.F16, GGMLType.F32]


def K():
    from tensorsharp_b200.ops import kernels
    return kernels


def expected_gemv(qw, x_bf16):
    """What the GEMV computes: int8-rounded activations against the scaled quants, and - for
    the K-quants that carry a per-sub-block minimum - the *unrounded* activation sums against
    the minimum term (the same contract as ggml's q8_1 activations)."""
    xr = ref.quantize_q8_dequant(x_bf16.float())
    W = qw.dequantize()
    if qw.ggml_type in (GGMLType.Q4_K, GGMLType.Q5_K):
        raw = qw.raw_blocks().clone().view(-1, 144 if qw.ggml_type == GGMLType.Q4_K else 176)
        raw[:, 16:] = 0
        Z = codecs.dequantize(raw.view(-1), qw.ggml_type, W.shape)      # the "- dmin * m" part alone
        return xr @ (W - Z).t() + x_bf16.float() @ Z.t()
    return xr @ W.t()


def rel_err(a, b):
    a, b = a.float(), b.float()
    return float((a - b).norm() / b.norm().clamp_min(1e-12))


@pytest.mark.parametrize("t", QTYPES + FTYPES)
def test_gather_rows_matches_codec(t):
    torch.manual_seed(0)
    w = torch.randn(70, 512, device=DEV) * 0.05
    qw = QuantWeight.from_float(w, t)
    want = qw.dequantize()
    got = K().gather_rows(qw, None, 1.0, torch.float32)
    assert torch.allclose(got, want, atol=1e-6, rtol=1e-6)
    ids = torch.tensor([3, 69, 0, 3], dtype=torch.int32, device=DEV)
    got = K().gather_rows(qw, ids, 2.0, torch.bfloat16)
    assert torch.allclose(got.float(), (want[ids.long()] * 2.0).bfloat16().float(), atol=1e-6)


@pytest.mark.parametrize("t", QTYPES)
@pytest.mark.parametrize("M", [1, 3, 8, 13])
def test_gemv_quant(t, M):
    torch.manual_seed(1)
    N, Kd = 203, 768
    w = torch.randn(N, Kd, device=DEV) * 0.05
    x = torch.randn(M, Kd, device=DEV)
    qw = QuantWeight.from_float(w, t)
    xq, xds = K().quantize_q8(x.bfloat16())
    want = expected_gemv(qw, x.bfloat16())
    got = K().gemv(qw, xq=xq, xds=xds, M=M)
    assert rel_err(got, want) < 1e-3, rel_err(got, want)
    # bias + residual, bf16 output
    bias = torch.randn(N, device=DEV)
    res = torch.randn(M, N, device=DEV)
    got = K().gemv(qw, xq=xq, xds=xds, M=M, bias=bias, residual=res)
    assert rel_err(got, want + bias + res) < 2e-3


@pytest.mark.parametrize("t", FTYPES)
def test_gemv_float(t):
    torch.manual_seed(2)
    N, Kd, M = 130, 256, 5
    w = torch.randn(N, Kd, device=DEV) * 0.05
    x = torch.randn(M, Kd, device=DEV).bfloat16()
    qw = QuantWeight.from_float(w, t)
    want = x.float() @ qw.dequantize().t()
    got = K().gemv(qw, xb=x, M=M)
    assert rel_err(got, want) < 1e-3


@pytest.mark.parametrize("act", ["swiglu", "geglu", "geglu_erf", "swiglu_oai"])
def test_gemv_glu(act):
    torch.manual_seed(3)
    F, Kd, M = 96, 512, 2
    w = torch.randn(2 * F, Kd, device=DEV) * 0.1
    x = torch.randn(M, Kd, device=DEV)
    qw = QuantWeight.from_float(w, GGMLType.Q4_K)
    xq, xds = K().quantize_q8(x.bfloat16())
    y = expected_gemv(qw, x.bfloat16())
    want = ref.glu(act, y[:, :F], y[:, F:])
    got = K().gemv(qw, xq=xq, xds=xds, M=M, act=act)
    assert got.shape == (M, F)
    assert rel_err(got, want) < 3e-3


def test_gemv_moe_ids():
    torch.manual_seed(4)
    E, N, Kd, T, topk = 6, 64, 256, 3, 2
    w = torch.randn(E, N, Kd, device=DEV) * 0.1
    qw = QuantWeight.from_float(w, GGMLType.MXFP4)
    x = torch.randn(T, Kd, device=DEV)
    ids = torch.tensor([0, 5, 2, 2, 4, 1], dtype=torch.int32, device=DEV)
    scale = torch.rand(T * topk, device=DEV)
    xq, xds = K().quantize_q8(x.bfloat16())
    xr = ref.quantize_q8_dequant(x.bfloat16().float())
    wd = qw.dequantize().view(E, N, Kd)
    want = torch.stack([wd[int(ids[p])] @ xr[p // topk] * scale[p] for p in range(T * topk)])
    got = K().gemv(qw, xq=xq, xds=xds, M=1, ids=ids, x_div=topk, row_scale=scale)
    assert rel_err(got, want) < 2e-3


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_rmsnorm(dtype):
    torch.manual_seed(5)
    rows, D = 7, 2560
    x = torch.randn(rows, D, device=DEV).to(dtype)
    w = torch.rand(D, device=DEV) + 0.5
    want = ref.rmsnorm(x, w, 1e-6)
    yb, yf, yq, yds = K().rmsnorm(x.clone(), w, 1e-6, want_q8=True, want_f32=True)
    assert rel_err(yf, want) < 1e-5
    assert rel_err(yb, want) < 5e-3
    deq = (yq.float().view(rows, D // 32, 32) * yds[..., 0:1]).view(rows, D)
    assert rel_err(deq, want) < 1e-2
    assert torch.allclose(yds[..., 1], want.view(rows, D // 32, 32).sum(-1), atol=1e-3)
    # delta add writes the stream back
    delta = torch.randn(rows, D, device=DEV).bfloat16()
    xs = x.clone()
    yb, *_ = K().rmsnorm(xs, w, 1e-6, delta=delta)
    assert rel_err(xs, x.float() + delta.float()) < 5e-3
    assert rel_err(yb, ref.rmsnorm(x.float() + delta.float(), w, 1e-6)) < 6e-3
    # sandwich add and L2
    h = torch.randn(rows, D, device=DEV)
    _, yf, _, _ = K().rmsnorm(x.clone(), w, 1e-6, want_bf16=False, add=h)
    assert rel_err(yf, h + want) < 1e-5
    _, yf, _, _ = K().rmsnorm(x.clone(), None, 1e-6, want_bf16=False, want_f32=True, l2=True)
    assert rel_err(yf, ref.l2norm(x, 1e-6)) < 1e-5


@pytest.mark.parametrize("mode,rot,Dh,yarn", [(0, 128, 128, False), (0, 64, 128, True), (1, 64, 64, False),
                                              (0, 256, 256, False), (1, 32, 96, True)])
def test_qkv_rope_cache(mode, rot, Dh, yarn):
    from tensorsharp_b200.ops import functional as F
    torch.manual_seed(6)
    T, Hq, Hkv = 9, 4, 2
    qkv = torch.randn(T, (Hq + 2 * Hkv) * Dh, device=DEV)
    pos = torch.tensor([0, 1, 2, 3, 100, 4000, 31999, 7, 8], dtype=torch.int32, device=DEV)
    slots = torch.arange(T, dtype=torch.int64, device=DEV) + 5
    qn, kn = torch.rand(Dh, device=DEV) + 0.5, torch.rand(Dh, device=DEV) + 0.5
    spec = F.RopeSpec(rot_dim=rot, theta_base=150000.0, mode=mode)
    if yarn:
        lo, hi = K().yarn_corr_dims(rot, 4096, 150000.0, 32.0, 1.0)
        spec = F.RopeSpec(rot_dim=rot, theta_base=150000.0, mode=mode, freq_scale=1 / 32.0, ext_factor=1.0,
                          attn_factor=1.0, corr_lo=lo, corr_hi=hi)
    outs = {}
    for dev in ("cuda", "cpu"):
        x = qkv.to(dev)
        q = x[:, :Hq * Dh].view(T, Hq, Dh)
        k = x[:, Hq * Dh:(Hq + Hkv) * Dh].view(T, Hkv, Dh)
        v = x[:, (Hq + Hkv) * Dh:].view(T, Hkv, Dh)
        kc = torch.zeros(32, Hkv, Dh, dtype=torch.bfloat16 if dev == "cuda" else torch.float32, device=dev)
        vc = torch.zeros_like(kc)
        batch = F.Batch(tokens=pos.to(dev), positions=pos.to(dev), slots=slots.to(dev), cu_q=None, kv_lens=None,
                        block_table=None, last_idx=None, seq_slots=None, max_q_len=T, max_kv_len=T, is_decode=False,
                        page_size=16)
        qo = F.qkv_rope_cache(q, k, v, Hq=Hq, Hkv=Hkv, Dh=Dh, batch=batch, k_cache=kc, v_cache=vc, rope=spec,
                              qn=qn.to(dev), kn=kn.to(dev), v_norm=True, q_scale=0.5)
        outs[dev] = (qo.float().cpu(), kc.float().cpu(), vc.float().cpu())
    for a, b in zip(outs["cuda"], outs["cpu"]):
        assert rel_err(a, b) < 6e-3, rel_err(a, b)


def _paged(T_total, Hkv, Dh, page_size, lens):
    """Random cache with a shuffled page table for sequences of the given lengths."""
    n_pages = sum((l + page_size - 1) // page_size for l in lens) + 3
    kc = torch.randn(n_pages * page_size, Hkv, Dh, device=DEV).bfloat16()
    vc = torch.randn(n_pages * page_size, Hkv, Dh, device=DEV).bfloat16()
    perm = torch.randperm(n_pages).tolist()
    width = max((l + page_size - 1) // page_size for l in lens)
    table = torch.zeros(len(lens), width, dtype=torch.int32)
    for b, l in enumerate(lens):
        for i in range((l + page_size - 1) // page_size):
            table[b, i] = perm.pop()
    return kc, vc, table.to(DEV)


def _gather(kc, table, b, L, ps):
    pages = table[b, :(L + ps - 1) // ps].long()
    idx = (pages.unsqueeze(1) * ps + torch.arange(ps, device=kc.device)).reshape(-1)[:L]
    return kc[idx]


@pytest.mark.parametrize("Hq,Hkv,Dh", [(8, 2, 128), (4, 4, 64), (16, 2, 256), (2, 1, 64), (8, 2, 512), (6, 2, 128), (12, 1, 64),
                                       (5, 1, 128), (32, 2, 64), (2, 2, 512)])
@pytest.mark.parametrize("window,sinks,softcap", [(0, False, 0.0), (100, True, 0.0), (0, False, 30.0)])
def test_attn_decode(Hq, Hkv, Dh, window, sinks, softcap):
    torch.manual_seed(7)
    ps, lens = 16, [1, 37, 300, 1025]
    B = len(lens)
    kc, vc, table = _paged(sum(lens), Hkv, Dh, ps, lens)
    q = torch.randn(B, Hq, Dh, device=DEV).bfloat16()
    sk = torch.randn(Hq, device=DEV) if sinks else None
    kv_lens = torch.tensor(lens, dtype=torch.int32, device=DEV)
    for splits in (1, 5):
        got = K().attn_decode(q, kc, vc, table, kv_lens, scale=Dh ** -0.5, Hq=Hq, Hkv=Hkv, Dh=Dh, page_size=ps,
                              splits=splits, sinks=sk, softcap=softcap, window=window)
        for b, L in enumerate(lens):
            want = ref.attention(q[b:b + 1], _gather(kc, table, b, L, ps), _gather(vc, table, b, L, ps),
                                 torch.tensor([L - 1], device=DEV), scale=Dh ** -0.5, window=window, sinks=sk,
                                 softcap=softcap)
            assert rel_err(got[b], want[0]) < 1e-2, (b, splits, rel_err(got[b], want[0]))


@pytest.mark.parametrize("Hq,Hkv,Dh,B,splits", [(32, 8, 128, 16, 9), (64, 8, 64, 12, 7), (16, 8, 128, 20, 4), (8, 8, 64, 20, 4),
                                                (48, 4, 128, 40, 4), (64, 4, 64, 40, 5), (12, 4, 128, 50, 3),
                                                # 8 or 16 splits: merged inside the kernel by a thread-block cluster
                                                (32, 8, 128, 1, 16), (32, 8, 128, 3, 8), (64, 8, 64, 2, 16), (16, 2, 128, 5, 8),
                                                (32, 2, 64, 4, 16), (8, 8, 64, 3, 16)])
@pytest.mark.parametrize("window,sinks,softcap", [(0, False, 0.0), (100, True, 0.0), (0, False, 30.0)])
def test_attn_decode_batches_on_the_tensor_cores(Hq, Hkv, Dh, B, splits, window, sinks, softcap, monkeypatch):
    """Grids of more than four CTAs per SM take the tensor-core split kernel (csrc/attention_decode_mma.cu): groups of
    1 to 16 query heads per KV head, ragged lengths (one key, a partial last chunk, splits left empty), window, sinks,
    soft-cap, against the float32 softmax.  With 8 or 16 splits the cluster form of the kernel (off by default) runs."""
    monkeypatch.setenv("TSB_ATTN_CLUSTER", "1")
    torch.manual_seed(17)
    ps = 16
    lens = [1 + (37 * i * i + 11 * i + 600) % 700 for i in range(B)]
    if B > 2:
        lens[1], lens[2] = 1, 32
    kc, vc, table = _paged(sum(lens), Hkv, Dh, ps, lens)
    q = torch.randn(B, Hq, Dh, device=DEV).bfloat16()
    sk = torch.randn(Hq, device=DEV) if sinks else None
    kv_lens = torch.tensor(lens, dtype=torch.int32, device=DEV)
    got = K().attn_decode(q, kc, vc, table, kv_lens, scale=Dh ** -0.5, Hq=Hq, Hkv=Hkv, Dh=Dh, page_size=ps,
                          splits=splits, sinks=sk, softcap=softcap, window=window)
    assert torch.isfinite(got.float()).all()
    for b, L in enumerate(lens):
        want = ref.attention(q[b:b + 1], _gather(kc, table, b, L, ps), _gather(vc, table, b, L, ps),
                             torch.tensor([L - 1], device=DEV), scale=Dh ** -0.5, window=window, sinks=sk, softcap=softcap)
        assert rel_err(got[b], want[0]) < 1.5e-2, (b, L, rel_err(got[b], want[0]))
    # a split length fixed by the caller (what the model path passes) gives the same result
    sl = ((max(lens) + splits - 1) // splits + 31) & ~31
    if not window:
        fixed = K().attn_decode(q, kc, vc, table, kv_lens, scale=Dh ** -0.5, Hq=Hq, Hkv=Hkv, Dh=Dh, page_size=ps,
                                splits=splits, sinks=sk, softcap=softcap, window=window, split_len=sl)
        assert rel_err(fixed, got) < 1e-2
    # the int8 form for the following projection equals a separate quantise of the bf16 output
    out, oq, ods = K().attn_decode(q, kc, vc, table, kv_lens, scale=Dh ** -0.5, Hq=Hq, Hkv=Hkv, Dh=Dh, page_size=ps,
                                   splits=splits, sinks=sk, softcap=softcap, window=window, want_q8=True)
    wq, wds = K().quantize_q8(out.view(B, Hq * Dh))
    assert torch.equal(out, got) and torch.equal(oq, wq) and torch.equal(ods, wds)


@pytest.mark.parametrize("Hq,Hkv,Dh", [(4, 2, 128), (2, 2, 64), (4, 1, 256), (4, 2, 512), (3, 1, 128)])
@pytest.mark.parametrize("window,sinks,softcap", [(0, False, 0.0), (70, True, 0.0), (0, False, 50.0)])
def test_attn_prefill(Hq, Hkv, Dh, window, sinks, softcap):
    torch.manual_seed(8)
    ps = 16
    qlens, lens = [5, 64, 150, 1], [5, 200, 150, 90]     # (new queries, total cache length)
    B = len(lens)
    kc, vc, table = _paged(sum(lens), Hkv, Dh, ps, lens)
    T = sum(qlens)
    q = torch.randn(T, Hq, Dh, device=DEV).bfloat16()
    sk = torch.randn(Hq, device=DEV) if sinks else None
    cu = torch.tensor([0] + list(torch.tensor(qlens).cumsum(0)), dtype=torch.int32, device=DEV)
    kv_lens = torch.tensor(lens, dtype=torch.int32, device=DEV)
    got = K().attn_prefill(q, kc, vc, table, kv_lens, cu, max(qlens), scale=Dh ** -0.5, Hq=Hq, Hkv=Hkv, Dh=Dh,
                           page_size=ps, sinks=sk, softcap=softcap, window=window)
    o = 0
    for b, (ql, L) in enumerate(zip(qlens, lens)):
        qpos = torch.arange(L - ql, L, device=DEV)
        want = ref.attention(q[o:o + ql], _gather(kc, table, b, L, ps), _gather(vc, table, b, L, ps), qpos,
                             scale=Dh ** -0.5, window=window, sinks=sk, softcap=softcap)
        assert rel_err(got[o:o + ql], want) < 1.5e-2, (b, rel_err(got[o:o + ql], want))
        o += ql


# the last four shapes have more tiles than SMs and take the persistent kernel (two accumulators in tensor memory, the
# epilogue of a tile under the next tile's main loop): 256- and 128-token tiles, ragged edges, a single k-block
@pytest.mark.parametrize("T,N,Kd", [(5, 128, 64), (33, 200, 320), (100, 384, 2560), (300, 1000, 512), (2048, 256, 1024),
                                    (3900, 7744, 320), (4096, 7680, 64), (100, 20480, 256), (520, 19400, 192),
                                    (16, 2560, 9728), (33, 640, 4096), (9, 256, 8192)])     # the last three: split-K
def test_gemm_bf16_tcgen05(T, N, Kd):
    torch.manual_seed(9)
    W = (torch.randn(N, Kd, device=DEV) * 0.05).bfloat16()
    X = torch.randn(T, Kd, device=DEV).bfloat16()
    want = X.float() @ W.float().t()
    got = K().gemm_bf16(W, X, out_dtype=torch.float32)
    torch.cuda.synchronize()
    assert int(K().gemm_status(DEV).item()) == 0
    assert rel_err(got, want) < 1e-3, rel_err(got, want)
    bias = torch.randn(N, device=DEV)
    res = torch.randn(T, N, device=DEV).bfloat16()
    got = K().gemm_bf16(W, X, out_dtype=torch.bfloat16, bias=bias, residual=res)
    assert rel_err(got, want + bias + res.float()) < 6e-3


@pytest.mark.parametrize("act", ["swiglu", "geglu", "swiglu_oai", "relu2", "sigmoid_mul"])
def test_glu(act):
    torch.manual_seed(10)
    T, F = 6, 160
    y = torch.randn(T, 2 * F, device=DEV)
    g, u = y[:, :F], y[:, F:]
    want = ref.glu(act, g, u if act != "relu2" else None)
    out, yq, yds = K().glu(g, None if act == "relu2" else u, act, F, 2 * F, 2 * F, T, want_q8=True)
    assert rel_err(out, want) < 5e-3
    deq = (yq.float().view(T, F // 32, 32) * yds[..., 0:1]).view(T, F)
    assert rel_err(deq, want) < 1.2e-2


def test_argmax():
    torch.manual_seed(11)
    x = torch.randn(5, 151936, device=DEV)
    x[2, 77] = 100.0
    x[3, 5] = x[3, 9000] = 50.0
    got = K().argmax(x)
    assert got.tolist() == x.argmax(-1).tolist()
    assert got[3].item() == 5
    for V in (151937, 20001, 4097 * 4):              # odd lengths: unaligned rows, ragged last chunk; repeated calls reuse the tickets
        y = torch.randn(3, V, device=DEV)
        y[1, V - 1] = 99.0
        for _ in range(2):
            assert K().argmax(y).tolist() == y.argmax(-1).tolist()


@pytest.mark.parametrize("t", QTYPES + FTYPES)
@pytest.mark.parametrize("M", [1, 2, 3, 4])
def test_fused_gemv_norm_prologue(t, M):
    """In-kernel RMSNorm + quantise prologue against the separate norm and GEMV kernels and
    against the fp32 reference."""
    torch.manual_seed(21)
    N, Kd = 205, 2560
    w = torch.randn(N, Kd, device=DEV) * 0.05
    h = torch.randn(M, Kd, device=DEV) * 3
    g = torch.rand(Kd, device=DEV) + 0.5
    qw = QuantWeight.from_float(w, t)
    bias = torch.randn(N, device=DEV)
    res = torch.randn(M, N, device=DEV)
    yb, _, yq, yds = K().rmsnorm(h.clone(), g, 1e-6, want_q8=True)
    if qw.uses_q8_activations:
        sep = K().gemv(qw, xq=yq, xds=yds, M=M, bias=bias, residual=res)
    else:
        sep = K().gemv(qw, xb=yb, M=M, bias=bias, residual=res)
    got = K().fused_gemv(qw, x_f32=h, norm_w=g, eps=1e-6, do_norm=True, bias=bias, residual=res)
    assert rel_err(got, sep) < 2e-3, rel_err(got, sep)
    want = ref.rmsnorm(h, g, 1e-6) @ qw.dequantize().t() + bias + res
    assert rel_err(got, want) < 1.5e-2
    # in place on the residual stream, as the model uses it
    stream = res.clone()
    K().fused_gemv(qw, x_f32=h, norm_w=g, eps=1e-6, do_norm=True, bias=bias, residual=stream, out=stream)
    assert torch.equal(stream, got)


@pytest.mark.parametrize("Kd", [4096, 9728, 1024 + 32])
def test_fused_gemv_cast_prologue_and_glu(Kd):
    torch.manual_seed(22)
    F_, M = 120, 2
    w = torch.randn(2 * F_, Kd, device=DEV) * 0.05
    x = torch.randn(M, Kd, device=DEV).bfloat16()
    t = GGMLType.Q4_K if Kd % 256 == 0 else GGMLType.Q8_0
    qw = QuantWeight.from_float(w, t)
    y = expected_gemv(qw, x)
    got = K().fused_gemv(qw, x_bf16=x)
    assert rel_err(got, y) < 2e-3
    got = K().fused_gemv(qw, x_bf16=x, act="swiglu", out_dtype=torch.bfloat16)
    assert got.shape == (M, F_) and got.dtype == torch.bfloat16
    assert rel_err(got, ref.glu("swiglu", y[:, :F_], y[:, F_:])) < 8e-3
    # unweighted norm of an f32 input
    xf = torch.randn(M, Kd, device=DEV)
    got = K().fused_gemv(qw, x_f32=xf, eps=1e-5, do_norm=True)
    assert rel_err(got, ref.rmsnorm(xf, None, 1e-5) @ qw.dequantize().t()) < 3e-2


@pytest.mark.parametrize("t", [GGMLType.Q4_K, GGMLType.Q6_K, GGMLType.Q8_0, GGMLType.MXFP4, GGMLType.BF16])
@pytest.mark.parametrize("M", [1, 2, 3, 4])
def test_gemv_split_rows(t, M):
    """Long rows, few of them: the four warps of a CTA share one row."""
    torch.manual_seed(31)
    N, Kd = 130, 4096
    w = torch.randn(N, Kd, device=DEV) * 0.05
    x = torch.randn(M, Kd, device=DEV).bfloat16()
    qw = QuantWeight.from_float(w, t)
    bias = torch.randn(N, device=DEV)
    res = torch.randn(M, N, device=DEV)
    if qw.uses_q8_activations:
        xq, xds = K().quantize_q8(x)
        want = expected_gemv(qw, x)
        got = K().gemv(qw, xq=xq, xds=xds, M=M, bias=bias, residual=res)
    else:
        want = x.float() @ qw.dequantize().t()
        got = K().gemv(qw, xb=x, M=M, bias=bias, residual=res)
    assert rel_err(got, want + bias + res) < 2e-3


# ---------------------------------------------------------------- device-side MoE routing / grouping
@pytest.mark.parametrize("E,k", [(32, 4), (128, 8), (256, 8), (6, 2), (512, 10)])
def test_moe_route_softmax_matches_topk(E, k):
    torch.manual_seed(20)
    T = 37
    logits = torch.randn(T, E, device=DEV)
    ids, w = K().moe_route(logits, k, mode=0)
    vals, want_ids = torch.topk(logits, k, dim=-1)
    assert torch.equal(ids.long(), want_ids)
    assert torch.allclose(w, torch.softmax(vals, -1), atol=1e-6, rtol=1e-5)


def test_moe_route_sigmoid_bias_normalise():
    torch.manual_seed(21)
    T, E, k = 19, 64, 6
    logits = torch.randn(T, E, device=DEV)
    bias = torch.randn(E, device=DEV) * 0.3
    ids, w = K().moe_route(logits, k, mode=1, sel_bias=bias, normalize=True, scale=2.5)
    p = torch.sigmoid(logits)
    _, want_ids = torch.topk(p + bias, k, dim=-1)
    ww = p.gather(-1, want_ids)
    ww = ww / ww.sum(-1, keepdim=True).clamp_min(6.103515625e-5) * 2.5
    assert torch.equal(ids.long(), want_ids)
    assert torch.allclose(w, ww, atol=1e-6, rtol=1e-5)


@pytest.mark.parametrize("t,act", [(GGMLType.MXFP4, "swiglu_oai"), (GGMLType.Q4_K, "swiglu"), (GGMLType.BF16, "relu2")])
@pytest.mark.parametrize("e0,E_local,Kd,Fd", [(0, 8, 256, 512), (4, 4, 256, 512), (0, 8, 288, 160)])
def test_moe_grouped_matches_per_slot_reference(t, act, e0, E_local, Kd, Fd):
    if t == GGMLType.Q4_K and (Kd % 256 or Fd % 256):
        pytest.skip("K-quants need rows of whole 256-value blocks")
    torch.manual_seed(22)
    E, T, k = 8, 45, 3
    glu = act != "relu2"
    gu_rows = 2 * Fd if glu else Fd
    wg = torch.randn(E, gu_rows, Kd, device=DEV) * 0.08
    wd = torch.randn(E, Kd, Fd, device=DEV) * 0.08
    gate_up = QuantWeight.from_float(wg[e0:e0 + E_local].contiguous(), t)
    down = QuantWeight.from_float(wd[e0:e0 + E_local].contiguous(), t)
    gb = torch.randn(E_local, gu_rows, device=DEV) * 0.1
    db = torch.randn(E_local, Kd, device=DEV) * 0.1
    x = torch.randn(T, Kd, device=DEV).bfloat16()
    ids = torch.stack([torch.randperm(E, device=DEV)[:k] for _ in range(T)]).to(torch.int32)
    w = torch.rand(T, k, device=DEV)
    kw = dict(ids=ids, weights=w, gate_up=gate_up, down=down, act=act, gate_up_bias=gb, down_bias=db, expert_offset=e0)
    if gate_up.uses_q8_activations:
        xq, xds = K().quantize_q8(x)
        got = K().moe_grouped(xq=xq, xds=xds, **kw)
    else:
        got = K().moe_grouped(xb=x, **kw)

    def proj(qw, v):                           # the GEMV's arithmetic contract for one expert
        if qw.uses_q8_activations:
            return expected_gemv(qw, v)
        return v.float() @ qw.dequantize().t()
    want = torch.zeros(T, Kd, device=DEV)
    for tk in range(T):
        for j in range(k):
            e = int(ids[tk, j]) - e0
            if not 0 <= e < E_local:
                continue
            y = proj(gate_up.expert(e), x[tk:tk + 1])[0] + gb[e]
            y = ref.glu(act, y[None, :Fd], y[None, Fd:])[0] if glu else torch.relu(y) ** 2
            want[tk] += (proj(down.expert(e), y.bfloat16()[None])[0] + db[e]) * w[tk, j]
    assert rel_err(got, want) < 1e-2


@pytest.mark.parametrize("t,act", [(GGMLType.MXFP4, "swiglu_oai"), (GGMLType.Q4_K, "swiglu"), (GGMLType.BF16, "relu2")])
@pytest.mark.parametrize("e0,E_local,T,k", [(0, 8, 700, 2), (4, 4, 900, 3), (0, 8, 40, 2), (0, 8, 2000, 3)])   # the last: persistent kernel
def test_moe_prefill_grouped_gemm_matches_per_expert_route(monkeypatch, t, act, e0, E_local, T, k):
    """Large batches: both expert projections as one grouped tensor-core GEMM each over a device-built tile list
    (F.moe_experts above MOE_TILE_MAX_PAIRS) against the route that sorts on the host and runs expert after expert;
    experts with no rows, experts held elsewhere, uneven group sizes."""
    from tensorsharp_b200.ops import functional as F
    torch.manual_seed(24)
    E, Kd, Fd = 8, 256, 512
    glu = act != "relu2"
    gu_rows = 2 * Fd if glu else Fd
    gate_up = QuantWeight.from_float(torch.randn(E_local, gu_rows, Kd, device=DEV) * 0.08, t)
    down = QuantWeight.from_float(torch.randn(E_local, Kd, Fd, device=DEV) * 0.08, t)
    gb = torch.randn(E_local, gu_rows, device=DEV) * 0.1
    db = torch.randn(E_local, Kd, device=DEV) * 0.1
    x = torch.randn(T, Kd, device=DEV).bfloat16()
    ids = torch.stack([torch.randperm(E - 1, device=DEV)[:k] for _ in range(T)]).to(torch.int32)     # expert 7 gets no rows
    w = torch.rand(T, k, device=DEV)
    monkeypatch.setattr(F, "MOE_TILE_MAX_PAIRS", 0)
    monkeypatch.setattr(F, "GEMV_MAX_M", 0)
    monkeypatch.setattr(F, "DENSE_GEMV_MAX_M", 0)         # the per-expert route multiplies in bf16 too, whatever the group size
    outs = {}
    for mode in ("1", "0"):
        monkeypatch.setenv("TSB_MOE_GROUPED_GEMM", mode)
        outs[mode] = F.moe_experts(F.Act(x), ids, w, gate_up, down, act=act, gate_up_bias=gb, down_bias=db, expert_offset=e0)
    assert rel_err(outs["1"], outs["0"]) < 1e-2, rel_err(outs["1"], outs["0"])
    assert int(K().gemm_status(x.device).item()) == 0


def test_moe_grouped_is_graph_capturable_and_follows_new_routing():
    torch.manual_seed(23)
    E, T, k, Kd, Fd = 16, 64, 4, 256, 256
    gate_up = QuantWeight.from_float(torch.randn(E, 2 * Fd, Kd, device=DEV) * 0.08, GGMLType.MXFP4)
    down = QuantWeight.from_float(torch.randn(E, Kd, Fd, device=DEV) * 0.08, GGMLType.MXFP4)
    x = torch.randn(T, Kd, device=DEV).bfloat16()
    xq, xds = K().quantize_q8(x)
    logits = torch.randn(T, E, device=DEV)
    out = torch.zeros(T, Kd, device=DEV)

    def step():
        ids, w = K().moe_route(logits, k, mode=0)
        out.copy_(K().moe_grouped(xq=xq, xds=xds, ids=ids, weights=w, gate_up=gate_up, down=down, act="swiglu"))
    step()
    torch.cuda.synchronize()
    s = torch.cuda.Stream()
    s.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(s):
        step()
    torch.cuda.current_stream().wait_stream(s)
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        step()
    logits.copy_(torch.randn(T, E, device=DEV))          # a different routing, same graph
    g.replay()
    torch.cuda.synchronize()
    got = out.clone()
    step()
    torch.cuda.synchronize()
    assert torch.equal(got, out)


# ---------------------------------------------------------------- device sampler
def _philox(seed, c0, c1):
    M = 0xFFFFFFFF
    k0, k1 = seed & M, (seed >> 32) & M
    x = [c0, c1, 0x243F6A88, 0x85A308D3]
    for _ in range(10):
        p0, p1 = 0xD2511F53 * x[0], 0xCD9E8D57 * x[2]
        x = [((p1 >> 32) ^ x[1] ^ k0) & M, p1 & M, ((p0 >> 32) ^ x[3] ^ k1) & M, p0 & M]
        k0, k1 = (k0 + 0x9E3779B9) & M, (k1 + 0xBB67AE85) & M
    return x


def _host_sample(logits, counts, u, temperature, top_k, top_p, min_p, rep, pres, freq):
    s = logits.double().clone()
    if counts is not None:
        seen = counts > 0
        if rep != 1.0:
            s = torch.where(seen, torch.where(s > 0, s / rep, s * rep), s)
        s = torch.where(seen, s - pres - freq * counts.double(), s)
    if temperature <= 0:
        return int(s.argmax())
    probs = torch.softmax(s / temperature, -1)
    if min_p > 0:
        probs = torch.where(probs < min_p * probs.max(), torch.zeros_like(probs), probs)
    if top_k > 0:
        cp, ci = torch.topk(probs, min(top_k, probs.numel()))
        if top_p < 1.0:
            cum = torch.cumsum(cp, 0)
            hit = torch.nonzero(cum >= top_p)
            cut = int(hit[0]) + 1 if hit.numel() else cp.numel()
            cp, ci = cp[:cut], ci[:cut]
    else:
        cp, ci = probs, torch.arange(probs.numel(), device=probs.device)
    cum = torch.cumsum(cp, 0)
    r = u * float(cum[-1])
    nz = torch.nonzero((cum >= r) & (cp > 0))
    return int(ci[int(nz[0])]) if nz.numel() else int(ci[-1])


@pytest.mark.parametrize("cfg", [
    dict(temperature=0.8, top_k=40, top_p=0.9, min_p=0.0, rep=1.1, pres=0.0, freq=0.0),
    dict(temperature=1.3, top_k=500, top_p=1.0, min_p=0.02, rep=1.0, pres=0.5, freq=0.2),
    dict(temperature=0.7, top_k=0, top_p=1.0, min_p=0.05, rep=1.0, pres=0.0, freq=0.0),
    dict(temperature=0.0, top_k=0, top_p=1.0, min_p=0.0, rep=1.3, pres=0.0, freq=0.0),
])
def test_device_sampler_matches_host_order(cfg):
    torch.manual_seed(30)
    B, V, seed = 48, 5003, 1234
    logits = (torch.randn(B, V, device=DEV) * 3).contiguous()
    counts = torch.zeros(B, V, dtype=torch.int32, device=DEV)
    counts[:, ::7] = 2
    counts[:, 5] = 1
    before = counts.clone()
    ngen = torch.full((B,), 3, dtype=torch.int32, device=DEV)
    got = K().sample(logits, ngen, temperature=cfg["temperature"], top_k=cfg["top_k"], top_p=cfg["top_p"], min_p=cfg["min_p"],
                     repetition_penalty=cfg["rep"], presence_penalty=cfg["pres"], frequency_penalty=cfg["freq"], seed=seed,
                     counts=counts)
    torch.cuda.synchronize()
    same = 0
    for b in range(B):
        u = (_philox(seed, b, 3)[0] >> 8) / 16777216.0
        want = _host_sample(logits[b], before[b], u, cfg["temperature"], cfg["top_k"], cfg["top_p"], cfg["min_p"],
                            cfg["rep"], cfg["pres"], cfg["freq"])
        same += int(got[b]) == want
    assert same >= B - 1                       # float32 vs float64 cumulative sums may move one boundary draw
    assert torch.equal(ngen, torch.full_like(ngen, 4))
    bump = counts - before
    assert int(bump.sum()) == B and all(int(bump[b, int(got[b])]) == 1 for b in range(B))


def test_device_sampler_distribution_and_seed():
    torch.manual_seed(31)
    V, B = 64, 4096
    row = torch.randn(V, device=DEV) * 2
    logits = row.repeat(B, 1).contiguous()
    ngen = torch.zeros(B, dtype=torch.int32, device=DEV)
    a = K().sample(logits, ngen, temperature=1.0, top_k=8, top_p=1.0, min_p=0.0, seed=7)
    ngen.zero_()
    b = K().sample(logits, ngen, temperature=1.0, top_k=8, top_p=1.0, min_p=0.0, seed=7)
    assert torch.equal(a, b)                   # same seed, same counters: same draws
    top = torch.topk(row, 8)
    p = torch.softmax(top.values, -1)
    freq = torch.bincount(a.long(), minlength=V).float() / B
    assert float(freq.sum() - freq[top.indices].sum()) == 0.0
    assert torch.allclose(freq[top.indices], p, atol=0.03)


def test_gemv_multi_matches_separate_launches():
    torch.manual_seed(40)
    Kd = 512
    ws = [QuantWeight.from_float(torch.randn(n, Kd, device=DEV) * 0.05, t)
          for n, t in ((96, GGMLType.Q4_K), (32, GGMLType.Q4_K), (40, GGMLType.Q6_K))]
    for M in (1, 3, 8, 11):
        x = torch.randn(M, Kd, device=DEV).bfloat16()
        xq, xds = K().quantize_q8(x)
        got = K().gemv_multi(ws, xq=xq, xds=xds, M=M)
        want = torch.cat([K().gemv(w, xq=xq, xds=xds, M=M) for w in ws], 1)
        assert torch.allclose(got, want, atol=2e-4, rtol=1e-4)    # single-token Q4_K takes another kernel: same sums, other order
    wf = [QuantWeight.from_float(torch.randn(n, Kd, device=DEV) * 0.05, GGMLType.BF16) for n in (24, 8)]
    x = torch.randn(2, Kd, device=DEV).bfloat16()
    got = K().gemv_multi(wf, xb=x, M=2, out_dtype=torch.bfloat16)
    want = torch.cat([K().gemv(w, xb=x, M=2, out_dtype=torch.bfloat16) for w in wf], 1)
    assert torch.equal(got, want)


def test_attn_decode_q8_output_equals_separate_quantise():
    torch.manual_seed(41)
    B, Hq, Hkv, Dh, ps, ctx = 3, 8, 2, 128, 64, 200
    n_pages = B * 4
    kc = torch.randn(n_pages * ps, Hkv, Dh, device=DEV).bfloat16()
    vc = torch.randn(n_pages * ps, Hkv, Dh, device=DEV).bfloat16()
    table = torch.arange(n_pages, dtype=torch.int32, device=DEV).view(B, 4)
    lens = torch.tensor([ctx, 77, 130], dtype=torch.int32, device=DEV)
    q = torch.randn(B, Hq, Dh, device=DEV).bfloat16()
    kw = dict(scale=Dh ** -0.5, Hq=Hq, Hkv=Hkv, Dh=Dh, page_size=ps, splits=3)
    plain = K().attn_decode(q, kc, vc, table, lens, **kw)
    out, oq, ods = K().attn_decode(q, kc, vc, table, lens, want_q8=True, **kw)
    assert torch.equal(out, plain)
    wq, wds = K().quantize_q8(plain.view(B, Hq * Dh))
    assert torch.equal(oq, wq) and torch.equal(ods, wds)


@pytest.mark.parametrize("t", [GGMLType.Q4_K, GGMLType.Q5_K, GGMLType.Q6_K])
@pytest.mark.parametrize("N,Kd,act", [(2048, 2560, "swiglu"), (2560, 9728, None), (1021, 4096, None), (66, 256, "swiglu"),
                                      (4099, 2560, None), (300, 512, None)])
@pytest.mark.parametrize("M", [1, 2, 4])
def test_gemv_row_pipeline_shapes(t, N, Kd, act, M):
    """Decode shapes that take the shared-memory row pipeline: long and short rows, odd row counts,
    gated pairs, bias, residual and both output types."""
    torch.manual_seed(50)
    qw = QuantWeight.from_float(torch.randn(N, Kd, device=DEV) * 0.05, t)
    x = torch.randn(M, Kd, device=DEV).bfloat16()
    xq, xds = K().quantize_q8(x)
    bias = torch.randn(N, device=DEV) * 0.1
    y = expected_gemv(qw, x) + bias
    if act:
        F = N // 2
        want = ref.glu(act, y[:, :F], y[:, F:])
        got = K().gemv(qw, xq=xq, xds=xds, M=M, act=act, bias=bias, out_dtype=torch.bfloat16)
        assert got.shape == (M, F)
        assert rel_err(got, want) < 6e-3
    else:
        res = torch.randn(M, N, device=DEV)
        got = K().gemv(qw, xq=xq, xds=xds, M=M, bias=bias, residual=res)
        assert rel_err(got, y + res) < 3e-3


@pytest.mark.parametrize("N,Kd,act", [(2048, 2560, "swiglu"), (2560, 4096, None), (1000, 1024, None), (40, 256, "swiglu")])
@pytest.mark.parametrize("M", [5, 8, 11, 16])
def test_gemv_tensor_core_batches_q4k(N, Kd, act, M):
    """Batches of 5 to 16 rows over Q4_K weights run on the int8 tensor-core path: ragged row counts,
    gated pairs, bias, residual, row scale."""
    torch.manual_seed(60)
    qw = QuantWeight.from_float(torch.randn(N, Kd, device=DEV) * 0.05, GGMLType.Q4_K)
    x = torch.randn(M, Kd, device=DEV).bfloat16()
    xq, xds = K().quantize_q8(x)
    bias = torch.randn(N, device=DEV) * 0.1
    y = expected_gemv(qw, x) + bias
    if act:
        F = N // 2
        want = ref.glu(act, y[:, :F], y[:, F:])
        got = K().gemv(qw, xq=xq, xds=xds, M=M, act=act, bias=bias, out_dtype=torch.bfloat16)
        assert got.shape == (M, F)
        assert rel_err(got, want) < 6e-3
    else:
        res = torch.randn(M, N, device=DEV)
        scale = torch.rand(M, device=DEV) + 0.5
        got = K().gemv(qw, xq=xq, xds=xds, M=M, bias=bias, residual=res, row_scale=scale)
        assert rel_err(got, y * scale[:, None] + res) < 3e-3


def test_index_check_mode_names_the_bad_index_before_the_launch(monkeypatch):
    """TSB_CHECK_INDICES=1: an index that would take a kernel out of bounds (a token id past the embedding, a block-table
    page past the pool) raises IndexError on the host; nothing is launched with it."""
    from tensorsharp_b200.ops import kernels as kmod
    monkeypatch.setattr(kmod, "CHECK_INDICES", True)
    w = QuantWeight.from_float(torch.randn(64, 256, device=DEV) * 0.1, GGMLType.Q8_0)
    ok = K().gather_rows(w, torch.tensor([0, 63], dtype=torch.int32, device=DEV))
    assert ok.shape == (2, 256)
    with pytest.raises(IndexError, match="gather_rows: row id"):
        K().gather_rows(w, torch.tensor([0, 64], dtype=torch.int32, device=DEV))
    ps, lens = 16, [20]
    kc, vc, table = _paged(sum(lens), 2, 64, ps, lens)
    q = torch.randn(1, 4, 64, device=DEV).bfloat16()
    kv_lens = torch.tensor(lens, dtype=torch.int32, device=DEV)
    bad = table.clone()
    bad[0, 1] = kc.shape[0] // ps                         # first page past the pool
    with pytest.raises(IndexError, match="block-table page"):
        K().attn_decode(q, kc, vc, bad, kv_lens, scale=0.125, Hq=4, Hkv=2, Dh=64, page_size=ps, splits=1)
    K().attn_decode(q, kc, vc, table, kv_lens, scale=0.125, Hq=4, Hkv=2, Dh=64, page_size=ps, splits=1)

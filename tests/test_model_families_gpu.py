"""Every model family: the CUDA kernels against the CPU oracle path on tiny random models,
for prefill (tensor-core GEMM + flash attention), decode (GEMV + paged attention) and the
recurrent kernels (conv1d, GatedDeltaNet, Mamba2)."""
import pytest
import torch

from tensorsharp_b200.models.base import ModelBase
from tensorsharp_b200.ops import functional as F
from tensorsharp_b200.ops import reference as ref
from tests.test_model_families_cpu import FAMILIES, family_paths  # noqa: F401

pytestmark = pytest.mark.gpu


def _rel(a, b):
    return float((a.float() - b.float()).norm() / b.float().norm().clamp_min(1e-9))


# Tolerance on the relative error of the logits.  The CUDA path quantises activations to int8 groups of 32
# in front of every quantised projection (the reference's q8_1 contract) where the oracle keeps fp32; the
# eight MoE layers of the tiny Gemma 4 (hidden 256, 4 experts) accumulate the most of that noise.
TOL = {"gemma4": 0.1}


@pytest.mark.parametrize("name", list(FAMILIES))
def test_cuda_matches_cpu_oracle(family_paths, name):
    cpu = ModelBase.create(family_paths[name], "cpu", max_context=256)
    gpu = ModelBase.create(family_paths[name], "cuda", max_context=256)
    g = torch.Generator().manual_seed(11)
    ids = torch.randint(0, 4096, (70,), generator=g).tolist()
    lc, lg = cpu.forward(ids), gpu.forward(ids).cpu()
    tol = TOL.get(name, 6e-2)
    assert torch.isfinite(lg).all()
    assert _rel(lg, lc) < tol, _rel(lg, lc)
    t = int(lc.argmax())
    for _ in range(4):
        lc, lg = cpu.forward([t]), gpu.forward([t]).cpu()
        assert _rel(lg, lc) < tol, _rel(lg, lc)
        t = int(lc.argmax())


@pytest.mark.parametrize("name", list(FAMILIES))
def test_captured_decode_graph_follows_eager_steps(family_paths, name):
    """Greedy decode through DecodeGraph (one replay per token) gives the eager tokens in every family; for the families
    with recurrent layers this also checks that the capture's warm-up step leaves their state where it was."""
    from tensorsharp_b200.runtime.engine import DecodeGraph
    g = torch.Generator().manual_seed(12)
    prompt = torch.randint(0, 4096, (40,), generator=g).tolist()
    eager = ModelBase.create(family_paths[name], "cuda", max_context=256)
    t = int(eager.forward(prompt).argmax())
    want = [t]
    for _ in range(6):
        t = int(eager.forward([t]).argmax())
        want.append(t)
    m = ModelBase.create(family_paths[name], "cuda", max_context=256)
    seq = m.new_sequence()
    first = int(F.argmax(m.forward_batch(m.kv.build_batch([seq], [prompt])))[0])
    dg = DecodeGraph(m, [seq], 8)
    dg.set_tokens([first])
    dg.capture()
    got = [first] + [int(dg.step()[0]) for _ in range(6)]
    assert got == want


def _batch(lens, dev):
    cu = [0]
    for n in lens:
        cu.append(cu[-1] + n)
    T = cu[-1]
    z = torch.zeros(T, dtype=torch.int32)
    return F.Batch(tokens=z.to(dev), positions=z.to(dev), slots=torch.zeros(T, dtype=torch.int64, device=dev),
                   cu_q=torch.tensor(cu, dtype=torch.int32, device=dev),
                   kv_lens=torch.tensor(lens, dtype=torch.int32, device=dev), block_table=None, last_idx=None,
                   seq_slots=torch.tensor([2, 0, 1][:len(lens)], dtype=torch.int64, device=dev), max_q_len=max(lens),
                   max_kv_len=max(lens), is_decode=False, page_size=16, h_cu_q=tuple(cu), h_kv_lens=tuple(lens))


def test_conv1d_gdn_mamba_kernels():
    torch.manual_seed(0)
    lens = [5, 1, 37]
    T = sum(lens)
    # conv1d with carried tail, two consecutive calls
    C, K = 96, 4
    w, bias = torch.randn(C, K) * 0.3, torch.randn(C) * 0.1
    st_c, st_g = torch.randn(3, K - 1, C), None
    st_g = st_c.clone().cuda()
    for _ in range(2):
        x = torch.randn(T, C + 8)[:, :C]          # row-strided view
        oc = F.causal_conv1d(x, w, bias, st_c, _batch(lens, "cpu"))
        og = F.causal_conv1d(x.cuda(), w.cuda(), bias.cuda(), st_g, _batch(lens, "cuda"))
        assert _rel(og.cpu(), oc) < 1e-5 and _rel(st_g.cpu(), st_c) < 1e-6
    # GatedDeltaNet
    Hk, Hv, Dk, Dv = 2, 4, 64, 64
    qkv = torch.randn(T, 2 * Hk * Dk + Hv * Dv)
    z, beta, alpha = torch.randn(T, Hv * Dv), torch.randn(T, Hv), torch.randn(T, Hv)
    dtb, a_log, nw = torch.randn(Hv) * 0.5, -torch.rand(Hv), torch.rand(Dv) + 0.5
    s_c = torch.randn(3, Hv, Dv, Dk) * 0.1
    s_g = s_c.clone().cuda()
    oc = F.gdn(qkv, z, beta, alpha, dtb, a_log, nw, s_c, _batch(lens, "cpu"), Hk=Hk, Hv=Hv, Dk=Dk, Dv=Dv, eps=1e-6)
    og = F.gdn(qkv.cuda(), z.cuda(), beta.cuda(), alpha.cuda(), dtb.cuda(), a_log.cuda(), nw.cuda(), s_g,
               _batch(lens, "cuda"), Hk=Hk, Hv=Hv, Dk=Dk, Dv=Dv, eps=1e-6)
    assert _rel(og.cpu(), oc) < 1e-2 and _rel(s_g.cpu(), s_c) < 1e-4
    # Mamba2
    H, P, G, N = 4, 64, 2, 64
    xbc, dt = torch.randn(T, H * P + 2 * G * N), torch.randn(T, H)
    A, D, dtb = -torch.rand(H), torch.randn(H), torch.randn(H) * 0.5
    s_c = torch.randn(3, H, P, N) * 0.1
    s_g = s_c.clone().cuda()
    yc = F.mamba2(xbc, dt, dtb, A, D, s_c, _batch(lens, "cpu"), H=H, P=P, G=G, N=N)
    yg = F.mamba2(xbc.cuda(), dt.cuda(), dtb.cuda(), A.cuda(), D.cuda(), s_g, _batch(lens, "cuda"), H=H, P=P, G=G, N=N)
    assert _rel(yg.cpu(), yc) < 1e-4 and _rel(s_g.cpu(), s_c) < 1e-4


@pytest.mark.parametrize("family", ["gemma3", "gptoss"])
def test_window_ring_pool_on_cuda(tmp_path, monkeypatch, family):
    """TSB_KV_WINDOW_RING=1 on the GPU: sliding-window layers on a ring of pages give the logits of the pool that keeps
    every page (same prefill chunks), through eager steps and through a captured decode graph that wraps the ring."""
    from tensorsharp_b200.models import synth
    from tensorsharp_b200.runtime.engine import DecodeGraph
    p = str(tmp_path / "m.gguf")
    if family == "gemma3":
        synth.write_gemma(p, arch="gemma3", window=16, device="cpu")
    else:
        synth.write_gptoss(p, n_layers=2, window=16, device="cpu")
    monkeypatch.setenv("TSB_KV_RING_CHUNK", "32")
    monkeypatch.setenv("TSB_GRAPH_FORWARD", "0")
    g = torch.Generator().manual_seed(13)
    toks = torch.randint(0, 4096, (200,), generator=g).tolist()
    logits, tokens = [], []
    for ring in ("0", "1"):
        monkeypatch.setenv("TSB_KV_WINDOW_RING", ring)
        m = ModelBase.create(p, "cuda", max_context=512, page_size=16)
        assert m.kv.ring == (ring == "1")
        for i in range(0, 192, 32):
            m.forward(toks[i:i + 32], want_logits=False)
        lg = m.forward(toks[192:]).float().cpu()
        logits.append(lg)
        seq = m._seq()
        dg = DecodeGraph(m, [seq], 100)
        dg.set_tokens([int(lg.argmax())])
        dg.capture()
        tokens.append([int(dg.step()[0]) for _ in range(90)])
    assert _rel(logits[1], logits[0]) < 1e-5, _rel(logits[1], logits[0])
    assert tokens[0] == tokens[1]

"""The chunked forms of the GatedDeltaNet and Mamba2 recurrences on the GPU (tensor ops, opt-in by environment)
against the token-by-token kernels."""
import pytest
import torch

from tensorsharp_b200.ops import functional as F

pytestmark = pytest.mark.gpu


def _batch(lens, dev):
    cu = [0]
    for n in lens:
        cu.append(cu[-1] + n)
    T = cu[-1]
    z = torch.zeros(T, dtype=torch.int32)
    return F.Batch(tokens=z.to(dev), positions=z.to(dev), slots=torch.zeros(T, dtype=torch.int64, device=dev),
                   cu_q=torch.tensor(cu, dtype=torch.int32, device=dev),
                   kv_lens=torch.tensor(lens, dtype=torch.int32, device=dev), block_table=None, last_idx=None,
                   seq_slots=torch.tensor([1, 0][:len(lens)], dtype=torch.int64, device=dev), max_q_len=max(lens),
                   max_kv_len=max(lens), is_decode=False, page_size=16, h_cu_q=tuple(cu), h_kv_lens=tuple(lens))


def _rel(a, b):
    return float((a.float() - b.float()).abs().max() / b.float().abs().max().clamp_min(1e-6))


def test_chunked_routes_match_the_scan_kernels(monkeypatch):
    torch.manual_seed(0)
    lens = [200, 70]
    T = sum(lens)
    dev = "cuda"
    Hk, Hv, Dk, Dv = 2, 4, 64, 64
    qkv = torch.randn(T, 2 * Hk * Dk + Hv * Dv, device=dev)
    z, beta, alpha = torch.randn(T, Hv * Dv, device=dev), torch.randn(T, Hv, device=dev), torch.randn(T, Hv, device=dev)
    dtb, a_log, nw = torch.randn(Hv, device=dev) * 0.5, -torch.rand(Hv, device=dev), torch.rand(Dv, device=dev) + 0.5
    s0 = torch.randn(2, Hv, Dv, Dk, device=dev) * 0.1
    outs, states = {}, {}
    for mode in ("0", "1"):
        monkeypatch.setenv("TSB_GDN_CHUNKED", mode)
        st = s0.clone()
        outs[mode] = F.gdn(qkv, z, beta, alpha, dtb, a_log, nw, st, _batch(lens, dev), Hk=Hk, Hv=Hv, Dk=Dk, Dv=Dv, eps=1e-6)
        states[mode] = st
    assert outs["1"].dtype == outs["0"].dtype
    assert _rel(outs["1"], outs["0"]) < 2e-2 and _rel(states["1"], states["0"]) < 1e-3
    H, P, G, N = 4, 64, 2, 64
    xbc, dt = torch.randn(T, H * P + 2 * G * N, device=dev), torch.randn(T, H, device=dev)
    A, D, dtb = -torch.rand(H, device=dev), torch.randn(H, device=dev), torch.randn(H, device=dev) * 0.5
    s0 = torch.randn(2, H, P, N, device=dev) * 0.1
    for mode in ("0", "1"):
        monkeypatch.setenv("TSB_MAMBA_CHUNKED", mode)
        st = s0.clone()
        outs[mode] = F.mamba2(xbc, dt, dtb, A, D, st, _batch(lens, dev), H=H, P=P, G=G, N=N)
        states[mode] = st
    # the chunk loop runs in the chunk-carry kernel (tf32 operands, f32 accumulation and state)
    assert _rel(outs["1"], outs["0"]) < 5e-3 and _rel(states["1"], states["0"]) < 5e-3, (_rel(outs["1"], outs["0"]), _rel(states["1"], states["0"]))
    monkeypatch.setenv("TSB_MAMBA_CARRY_KERNEL", "0")
    st = s0.clone()
    plain = F.mamba2(xbc, dt, dtb, A, D, st, _batch(lens, dev), H=H, P=P, G=G, N=N)
    assert _rel(plain, outs["0"]) < 1e-3 and _rel(st, states["0"]) < 1e-3


@pytest.mark.parametrize("Hk,Hv,Dk,Dv", [(2, 4, 128, 128), (1, 2, 64, 96)])
def test_chunk_carry_kernel_matches_the_scan_across_chunk_and_call_boundaries(monkeypatch, Hk, Hv, Dk, Dv):
    """csrc/gdn_chunk.cu (state carried chunk after chunk on the tensor cores, tf32 operands) against the token-by-token
    scan kernel and against the same chunked algebra as tensor ops: odd lengths, a state that is not zero, and a second
    call that continues from the state the first one left."""
    torch.manual_seed(1)
    dev = "cuda"
    dtb, a_log, nw = torch.randn(Hv, device=dev) * 0.5, -torch.rand(Hv, device=dev), torch.rand(Dv, device=dev) + 0.5
    s0 = torch.randn(2, Hv, Dv, Dk, device=dev) * 0.1
    results = {}
    # scan kernel; chunked tensor ops; tensor ops + carry kernel; the three chunk kernels (prep, carry, finish)
    for mode, carry, kernels in (("0", "1", "0"), ("1", "0", "0"), ("1", "1", "0"), ("1", "1", "1")):
        monkeypatch.setenv("TSB_GDN_CHUNKED", mode)
        monkeypatch.setenv("TSB_GDN_CARRY_KERNEL", carry)
        monkeypatch.setenv("TSB_GDN_CHUNK_KERNELS", kernels)
        torch.manual_seed(2)
        st = s0.clone()
        outs = []
        for lens in ([333], [129, 64], [70]):                       # the first sequence slot continues over three calls
            T = sum(lens)
            qkv = torch.randn(T, 2 * Hk * Dk + Hv * Dv, device=dev)
            z, beta, alpha = torch.randn(T, Hv * Dv, device=dev), torch.randn(T, Hv, device=dev), torch.randn(T, Hv, device=dev)
            b = _batch(lens, dev)
            outs.append(F.gdn(qkv, z, beta, alpha, dtb, a_log, nw, st, b, Hk=Hk, Hv=Hv, Dk=Dk, Dv=Dv, eps=1e-6).float())
        results[(mode, carry, kernels)] = (torch.cat(outs), st)
    scan, loop, kern, full = results[("0", "1", "0")], results[("1", "0", "0")], results[("1", "1", "0")], results[("1", "1", "1")]
    assert _rel(full[0], loop[0]) < 1e-2 and _rel(full[1], loop[1]) < 3e-3, (_rel(full[0], loop[0]), _rel(full[1], loop[1]))
    assert _rel(full[0], scan[0]) < 2e-2 and _rel(full[1], scan[1]) < 3e-3, (_rel(full[0], scan[0]), _rel(full[1], scan[1]))
    assert _rel(kern[0], loop[0]) < 1e-2 and _rel(kern[1], loop[1]) < 3e-3, (_rel(kern[0], loop[0]), _rel(kern[1], loop[1]))
    assert _rel(kern[0], scan[0]) < 2e-2 and _rel(kern[1], scan[1]) < 3e-3, (_rel(kern[0], scan[0]), _rel(kern[1], scan[1]))


@pytest.mark.parametrize("H,P,G,N", [(4, 64, 2, 128), (6, 32, 1, 64), (8, 64, 8, 128)])
def test_mamba2_chunk_kernels_match_the_scan_across_chunk_and_call_boundaries(monkeypatch, H, P, G, N):
    """csrc/gdn_chunk.cu: mamba2_chunk_prep_kernel + the chunk-carry kernel against the token-by-token scan kernel and
    against the chunked algebra as tensor ops: odd lengths, two sequences in a call, a state that is not zero, and calls
    that continue from the state the previous one left."""
    torch.manual_seed(3)
    dev = "cuda"
    A, D, dtb = -torch.rand(H, device=dev), torch.randn(H, device=dev), torch.randn(H, device=dev) * 0.5
    s0 = torch.randn(2, H, P, N, device=dev) * 0.1
    results = {}
    # scan kernel; chunked tensor ops; tensor ops + carry kernel; prep kernel + carry kernel
    for mode, carry, kernels in (("0", "1", "1"), ("1", "0", "0"), ("1", "1", "0"), ("1", "1", "1")):
        monkeypatch.setenv("TSB_MAMBA_CHUNKED", mode)
        monkeypatch.setenv("TSB_MAMBA_CARRY_KERNEL", carry)
        monkeypatch.setenv("TSB_MAMBA_CHUNK_KERNELS", kernels)
        torch.manual_seed(4)
        st = s0.clone()
        outs = []
        for lens in ([333], [129, 64], [70]):
            T = sum(lens)
            xbc, dt = torch.randn(T, H * P + 2 * G * N, device=dev), torch.randn(T, H, device=dev)
            outs.append(F.mamba2(xbc, dt, dtb, A, D, st, _batch(lens, dev), H=H, P=P, G=G, N=N).float())
        results[(mode, carry, kernels)] = (torch.cat(outs), st)
    scan, loop, kern, full = results[("0", "1", "1")], results[("1", "0", "0")], results[("1", "1", "0")], results[("1", "1", "1")]
    assert _rel(loop[0], scan[0]) < 1e-3 and _rel(loop[1], scan[1]) < 1e-3
    assert _rel(kern[0], scan[0]) < 5e-3 and _rel(kern[1], scan[1]) < 5e-3, (_rel(kern[0], scan[0]), _rel(kern[1], scan[1]))
    assert _rel(full[0], scan[0]) < 5e-3 and _rel(full[1], scan[1]) < 5e-3, (_rel(full[0], scan[0]), _rel(full[1], scan[1]))
    assert _rel(full[0], loop[0]) < 5e-3 and _rel(full[1], loop[1]) < 5e-3, (_rel(full[0], loop[0]), _rel(full[1], loop[1]))

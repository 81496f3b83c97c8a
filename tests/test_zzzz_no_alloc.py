"""The allocation-free decode-attention entry point against the regular one.

Some hosts of this library cannot allocate device memory when they call it (a server that
has given the whole GPU to its own arena, a decode loop that must not touch the allocator,
a binding that can only pass tensors it already holds).  ``tsb_attn_decode_noalloc`` keeps
its split-KV scratch in a static device array inside the library, so such a caller passes
only inputs and outputs.  This test calls it through its exported C symbol, twice in a row
with different inputs (the shared scratch keeps the first call's contents), and checks each
result against ``tsb_attn_decode`` run with caller-provided scratch.  It also checks that a
request larger than the built-in scratch is refused with a clear message.

The file name sorts last on purpose: a run that stops at the first failure has already run
every other test.  It passes alone in a fresh process and after the other tests.
"""
import ctypes as C

import pytest
import torch

pytestmark = pytest.mark.gpu


def _problem(seed, B, Hq, Hkv, Dh, ps, lens):
    g = torch.Generator(device="cuda").manual_seed(seed)
    n_pages = sum((l + ps - 1) // ps for l in lens) + 2
    kc = torch.randn(n_pages * ps, Hkv, Dh, device="cuda", generator=g).bfloat16()
    vc = torch.randn(n_pages * ps, Hkv, Dh, device="cuda", generator=g).bfloat16()
    width = max((l + ps - 1) // ps for l in lens)
    table = torch.zeros(B, width, dtype=torch.int32)
    perm = torch.randperm(n_pages).tolist()
    for b, l in enumerate(lens):
        for i in range((l + ps - 1) // ps):
            table[b, i] = perm.pop()
    q = torch.randn(B, Hq, Dh, device="cuda", generator=g).bfloat16()
    return q, kc, vc, table.cuda(), torch.tensor(lens, dtype=torch.int32, device="cuda")


def test_noalloc_matches_regular_twice_in_a_row():
    from tensorsharp_b200.ops import kernels, native
    lib = native.lib()
    fn = lib.tsb_attn_decode_noalloc            # the exported C symbol
    fn.restype = C.c_int
    lib.tsb_attn_decode_noalloc_capacity.restype = C.c_long
    cap = lib.tsb_attn_decode_noalloc_capacity()
    assert cap == 4 * 1024 * 1024
    Hq, Hkv, Dh, ps, splits = 8, 2, 128, 16, 6
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    for seed, lens in ((1, [9, 130, 700]), (2, [513, 64, 1])):
        B = len(lens)
        q, kc, vc, table, kv_lens = _problem(seed, B, Hq, Hkv, Dh, ps, lens)
        want = kernels.attn_decode(q, kc, vc, table, kv_lens, scale=Dh ** -0.5, Hq=Hq, Hkv=Hkv, Dh=Dh,
                                   page_size=ps, splits=splits, window=0)
        got = torch.empty_like(q)
        a = kernels._attn_args(q, kc, vc, got, table, kv_lens, None, None, Dh ** -0.5, 0.0, 0, Hq, Hkv, Dh, ps, B)
        a.splits = splits
        rc = fn(C.byref(a), stream)
        assert rc == 0, lib.tsb_last_error().decode()
        torch.cuda.synchronize()
        err = float((got.float() - want.float()).norm() / want.float().norm())
        assert err < 1e-2, err
        assert torch.equal(got, want)            # same kernels, same split: bit-identical in practice

    # a request beyond the built-in scratch is rejected, nothing is launched
    a.B, a.splits = 4096, 64
    rc = fn(C.byref(a), stream)
    assert rc != 0
    assert b"exceeds the built-in scratch" in lib.tsb_last_error()
    torch.cuda.synchronize()

"""Merged single-token steps through captured graphs (BatchGraphStepper) against the eager batched step on the GPU."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_graph_replays_follow_changing_membership(tmp_path):
    from tensorsharp_b200.models import synth
    from tensorsharp_b200.models.base import ModelBase
    from tensorsharp_b200.runtime.engine import BatchGraphStepper
    p = str(tmp_path / "q.gguf")
    synth.write_qwen3(p, n_layers=2, hidden=256, n_heads=4, n_kv_heads=2, head_dim=64, ffn=768, vocab=4096, scheme="Q4_K_M",
                      device="cuda")
    a = ModelBase.create(p, "cuda:0", max_context=512, max_seqs=4)
    b = ModelBase.create(p, "cuda:0", max_context=512, max_seqs=4)
    st = BatchGraphStepper(a, 3)
    gen = torch.Generator().manual_seed(2)
    prompts = [torch.randint(5, 4000, (n,), generator=gen).tolist() for n in (60, 30, 7)]
    sa, sb = [a.new_sequence() for _ in prompts], [b.new_sequence() for _ in prompts]
    for m, seqs in ((a, sa), (b, sb)):
        for s, pr in zip(seqs, prompts):
            m.forward_batch(m.kv.build_batch([s], [pr]), False)
    members = [[0, 1, 2], [0, 1, 2], [0, 2], [2], [1, 2, 0], [1, 0]] + [[0, 1, 2]] * 6          # sequence 0 crosses a page boundary
    for step, idx in enumerate(members):
        toks = [100 + step + i for i in idx]
        got = st.step([sa[i] for i in idx], toks)
        want = b.forward_batch(b.kv.build_batch([sb[i] for i in idx], [[t] for t in toks]), True)
        torch.cuda.synchronize()
        assert got is not None
        err = float((got.float() - want.float()).abs().max() / want.float().abs().max())
        assert err < 2e-2, (step, err)
    assert st.captures == 3 and st.replays == len(members)               # one graph per batch size, reused afterwards

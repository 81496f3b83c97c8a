"""The arithmetic of the expert-parallel dispatch / combine, played through on the CPU with every rank's buffers as
plain tensors: which ranks a token's row is sent to, which partial sums come back, and which accumulator slots the owner
adds.  The GPU kernels (csrc/tp_fused.cu: tp_seq_dispatch_kernel, tp_seq_push_rows_kernel with k > 0,
tp_seq_norm_gather_kernel with acc_k > 0) follow the same rules; stale data in the slots that are skipped must not
reach the result, so the model fills every buffer with NaN first."""
import torch

from tensorsharp_b200.ops import functional as F


def _dests(ids_row, epr):
    m = 0
    for e in ids_row.tolist():
        if e >= 0:
            m |= 1 << (e // epr)
    return m


def test_routed_dispatch_and_combine_equal_the_dense_mixture():
    torch.manual_seed(0)
    size, shard, D, Fd, E, k = 4, 8, 32, 48, 8, 2
    epr = E // size
    T = size * shard - 3                                    # the last shard has padding rows
    x = torch.randn(size * shard, D)
    logits = torch.randn(size * shard, E)
    ids, w = F.route_topk_softmax(logits, k)
    gate_up = torch.randn(E, 2 * Fd, D) * 0.2
    down = torch.randn(E, D, Fd) * 0.2

    def expert(e, rows):
        y = rows @ gate_up[e].t()
        return (torch.nn.functional.silu(y[:, :Fd]) * y[:, Fd:]) @ down[e].t()
    want = torch.zeros(T, D)
    for t in range(T):
        for j in range(k):
            want[t] += w[t, j] * expert(int(ids[t, j]), x[t:t + 1])[0]

    nan = float("nan")
    xfull = [torch.full((size * shard, D), nan) for _ in range(size)]
    route_ids = [torch.full((size * shard, k), -7, dtype=torch.int32) for _ in range(size)]
    route_w = [torch.full((size * shard, k), nan) for _ in range(size)]
    acc = [torch.full((size, shard, D), nan) for _ in range(size)]          # [owner][source][row]
    sent_rows = 0
    # dispatch (one "CTA" per local row of every rank)
    for rank in range(size):
        for r in range(shard):
            g = rank * shard + r
            live = g < T
            m = _dests(ids[g], epr) if live else 0
            for p in range(size):
                route_ids[p][g] = ids[g] if live else -1
                route_w[p][g] = w[g] if live else 0.0
            xfull[rank][g] = x[g]                            # the local normalised row
            for p in range(size):
                if p != rank and (m >> p) & 1:
                    xfull[p][g] = x[g]
                    sent_rows += 1
    # experts of every rank on what it received, then the masked push into the owners' accumulators
    for rank in range(size):
        e0, e1 = rank * epr, (rank + 1) * epr
        rid, rw = route_ids[rank][:T], route_w[rank][:T]
        y = torch.zeros(T, D)
        for t in range(T):
            for j in range(k):
                e = int(rid[t, j])
                if e0 <= e < e1:
                    assert torch.isfinite(xfull[rank][t]).all()         # every row it needs has arrived
                    y[t] += rw[t, j] * expert(e, xfull[rank][t:t + 1])[0]
        for t in range(size * shard):
            mine = any(e0 <= int(e) < e1 for e in route_ids[rank][t])
            if mine:
                acc[t // shard][rank][t % shard] = y[t] if t < T else 0.0
    # combine in the owner: only the slots named by the row's own routing record
    got = torch.zeros(size * shard, D)
    for rank in range(size):
        for r in range(shard):
            g = rank * shard + r
            m = _dests(route_ids[rank][g], epr)
            for src in range(size):
                if (m >> src) & 1:
                    got[g] += acc[rank][src][r]
    assert torch.isfinite(got).all()
    assert torch.allclose(got[:T], want, atol=1e-5)
    assert float(got[T:].abs().max()) == 0.0
    # and rows really stayed home: with two experts of eight over four ranks a row goes to at most two ranks
    assert sent_rows < T * (size - 1) and sent_rows <= 2 * T

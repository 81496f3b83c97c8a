"""Plain PyTorch fp32 restatements of every fused op.

These are the numerical oracle for the CUDA kernels and the execution path of the CPU
backend (tiny-model tests, golden parity).  They mirror the reference's semantics:
RMSNorm (TensorApplyCPU.cs:2206), RoPE NeoX / adjacent-pair with YaRN
(TensorApplyCPU.cs:1658-1806), softmax attention with sinks
(Models/GptOss/GptOssModel.cs:591-623), sliding-window masks (:575), gated activations
(GptOssModel.cs:901-934 for the clamp variant).
"""
from __future__ import annotations

import math
from typing import Optional

import torch


def rmsnorm(x: torch.Tensor, w: Optional[torch.Tensor], eps: float) -> torch.Tensor:
    x = x.float()
    y = x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps)
    return y * w.float() if w is not None else y


def l2norm(x: torch.Tensor, eps: float) -> torch.Tensor:
    x = x.float()
    return x / x.norm(dim=-1, keepdim=True).clamp_min(eps)


def layernorm(x, w, b, eps):
    return torch.nn.functional.layer_norm(x.float(), (x.shape[-1],), w, b, eps)


def rope_cos_sin(pos: torch.Tensor, rot_dim: int, theta_base: float, freq_scale: float = 1.0,
                 ext_factor: float = 0.0, attn_factor: float = 1.0, corr_lo: float = 0.0, corr_hi: float = 0.0,
                 freq_factors: Optional[torch.Tensor] = None):
    """cos / sin tables [T, rot_dim/2] following ggml's rope_yarn."""
    pair = torch.arange(rot_dim // 2, dtype=torch.float32, device=pos.device)
    theta = pos.float().unsqueeze(1) * torch.pow(torch.tensor(theta_base, dtype=torch.float32, device=pos.device),
                                                 -2.0 * pair / rot_dim)
    if freq_factors is not None:
        theta = theta / freq_factors.float()
    th = freq_scale * theta
    ms = attn_factor
    if ext_factor != 0.0:
        y = (pair - corr_lo) / max(0.001, corr_hi - corr_lo)
        ramp = (1.0 - y.clamp(0, 1)) * ext_factor
        th = th * (1 - ramp) + theta * ramp
        ms = ms * (1.0 + 0.1 * math.log(1.0 / freq_scale))
    return torch.cos(th) * ms, torch.sin(th) * ms


def apply_rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, rot_dim: int, mode: int) -> torch.Tensor:
    """x [T, H, Dh]; mode 0 = NeoX (i, i + rot/2), 1 = adjacent pairs (2i, 2i+1)."""
    x = x.float()
    if rot_dim == 0:
        return x
    xr, xp = x[..., :rot_dim], x[..., rot_dim:]
    c, s = cos.unsqueeze(1), sin.unsqueeze(1)
    if mode == 0:
        h = rot_dim // 2
        x0, x1 = xr[..., :h], xr[..., h:]
        out = torch.cat([x0 * c - x1 * s, x0 * s + x1 * c], -1)
    else:
        x0, x1 = xr[..., 0::2], xr[..., 1::2]
        out = torch.stack([x0 * c - x1 * s, x0 * s + x1 * c], -1).flatten(-2)
    return torch.cat([out, xp], -1)


def glu(act: str, g: torch.Tensor, u: Optional[torch.Tensor]) -> torch.Tensor:
    g = g.float()
    u = u.float() if u is not None else None
    if act == "swiglu":
        return torch.nn.functional.silu(g) * u
    if act in ("geglu", "geglu_tanh"):
        return torch.nn.functional.gelu(g, approximate="tanh") * u
    if act == "geglu_erf":
        return torch.nn.functional.gelu(g) * u
    if act == "swiglu_oai":
        x = g.clamp(max=7.0)
        y = u.clamp(-7.0, 7.0)
        return x * torch.sigmoid(1.702 * x) * (y + 1.0)
    if act == "relu2":
        return torch.relu(g) ** 2
    if act == "silu":
        return torch.nn.functional.silu(g)
    if act == "sigmoid_mul":
        return torch.sigmoid(g) * u
    return g * u


def attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, q_pos: torch.Tensor, *, scale: float,
              window: int = 0, sinks: Optional[torch.Tensor] = None, softcap: float = 0.0) -> torch.Tensor:
    """Naive attention for one sequence.  q [Tq, Hq, Dh]; k, v [Tk, Hkv, Dh] hold cache
    positions 0..Tk-1; q_pos [Tq] are the queries' positions.  Returns [Tq, Hq, Dh] f32."""
    Tq, Hq, Dh = q.shape
    Tk, Hkv, _ = k.shape
    g = Hq // Hkv
    qf = q.float().permute(1, 0, 2)                                  # [Hq, Tq, Dh]
    kf = k.float().permute(1, 0, 2).repeat_interleave(g, 0)          # [Hq, Tk, Dh]
    vf = v.float().permute(1, 0, 2).repeat_interleave(g, 0)
    s = torch.matmul(qf, kf.transpose(1, 2)) * scale                  # [Hq, Tq, Tk]
    if softcap and softcap > 0:
        s = softcap * torch.tanh(s / softcap)
    j = torch.arange(Tk, device=q.device).view(1, 1, Tk)
    p = q_pos.view(1, Tq, 1)
    ok = j <= p
    if window and window > 0:
        ok = ok & (j > p - window)
    s = s.masked_fill(~ok, float("-inf"))
    if sinks is not None:
        s = torch.cat([s, sinks.float().view(Hq, 1, 1).expand(Hq, Tq, 1)], -1)
        pr = torch.softmax(s, -1)[..., :Tk]
    else:
        pr = torch.softmax(s, -1)
    pr = torch.nan_to_num(pr, nan=0.0)
    return torch.matmul(pr, vf).permute(1, 0, 2).contiguous()


def quantize_q8_dequant(x: torch.Tensor) -> torch.Tensor:
    """What the GEMV kernels see: x rounded to int8 in groups of 32 (scale amax/127)."""
    xf = x.float()
    g = xf.reshape(-1, 32)
    d = g.abs().amax(1, keepdim=True) / 127.0
    q = torch.where(d > 0, torch.round(g / d), torch.zeros_like(g))
    return (q * d).reshape(xf.shape)


def causal_conv1d(x: torch.Tensor, w: torch.Tensor, bias, tail: torch.Tensor, act_silu: bool = True):
    """One sequence.  x [n, C]; w [C, K]; tail [K-1, C] (oldest first).  Returns (out [n, C],
    new tail).  out[t] = act(bias + sum_k w[:, k] * in[t - (K-1) + k])."""
    K = w.shape[1]
    ext = torch.cat([tail.float(), x.float()], 0)                     # [K-1+n, C]
    n = x.shape[0]
    out = torch.zeros(n, x.shape[1])
    for k in range(K):
        out = out + ext[k:k + n] * w[:, k].float()
    if bias is not None:
        out = out + bias.float()
    if act_silu:
        out = torch.nn.functional.silu(out)
    return out, ext[ext.shape[0] - (K - 1):].clone()


def gdn_recurrent(qkv, z, beta, alpha, dt_bias, a_log, norm_w, state, *, Hk, Hv, Dk, Dv, eps):
    """One sequence, token by token.  state [Hv, Dv, Dk] is updated in place.  Returns [n, Hv*Dv]."""
    n = qkv.shape[0]
    out = torch.zeros(n, Hv * Dv)
    hk = torch.arange(Hv) % Hk
    for t in range(n):
        q = qkv[t, :Hk * Dk].float().view(Hk, Dk)[hk]
        k = qkv[t, Hk * Dk:2 * Hk * Dk].float().view(Hk, Dk)[hk]
        v = qkv[t, 2 * Hk * Dk:].float().view(Hv, Dv)
        q = q * torch.rsqrt(q.pow(2).sum(-1, keepdim=True) + eps) * (Dv ** -0.5)
        k = k * torch.rsqrt(k.pow(2).sum(-1, keepdim=True) + eps)
        g = torch.nn.functional.softplus(alpha[t].float() + dt_bias.float()) * a_log.float()
        state.mul_(torch.exp(g).view(Hv, 1, 1))
        b = torch.sigmoid(beta[t].float())
        kv = torch.einsum("hvk,hk->hv", state, k)
        delta = (v - kv) * b.view(Hv, 1)
        state.add_(torch.einsum("hv,hk->hvk", delta, k))
        core = torch.einsum("hvk,hk->hv", state, q)
        core = core * torch.rsqrt(core.pow(2).mean(-1, keepdim=True) + eps) * norm_w.float()
        out[t] = (core * torch.nn.functional.silu(z[t].float().view(Hv, Dv))).reshape(-1)
    return out


def gdn_chunked(qkv, z, beta, alpha, dt_bias, a_log, norm_w, state, *, Hk, Hv, Dk, Dv, eps, chunk: int = 64, carry=None):
    """The recurrence of :func:`gdn_recurrent` in chunked form (Qwen35Model.cs:888-1192 does its prefill the same way):
    inside a chunk of ``chunk`` tokens the delta-rule updates are solved at once as a unit lower-triangular system
    (the WY form), so the work is matrix products over (heads x chunks) and only three small products per chunk run
    in sequence to carry the state.  One sequence; ``state`` [Hv, Dv, Dk] is updated in place; plain tensor ops, so it
    runs on whichever device the inputs live on.  ``carry`` replaces the loop over the chunks (a kernel on CUDA).
    Returns [n, Hv*Dv]."""
    n = qkv.shape[0]
    return gdn_chunked_batch(qkv, z, beta, alpha, dt_bias, a_log, norm_w, [state], [0, n], Hk=Hk, Hv=Hv, Dk=Dk, Dv=Dv, eps=eps,
                             chunk=chunk, carry=carry)


def gdn_chunked_batch(qkv, z, beta, alpha, dt_bias, a_log, norm_w, states, cu, *, Hk, Hv, Dk, Dv, eps, chunk: int = 64, carry=None):
    """:func:`gdn_chunked` for several sequences packed along the token axis (``cu``: host list of the B + 1 row offsets):
    the sequences are padded to a common number of chunks and stacked beside the heads, so that every tensor op and the
    chunk loop (or the ``carry`` kernel) runs once for the whole batch.  ``states``: one ``[Hv, Dv, Dk]`` tensor per
    sequence, each updated in place.  Returns [T, Hv*Dv]."""
    T = qkv.shape[0]
    dev = qkv.device
    C = chunk
    B = len(cu) - 1
    lens = [cu[i + 1] - cu[i] for i in range(B)]
    nc = (max(lens) + C - 1) // C
    L = nc * C
    hk = torch.arange(Hv, device=dev) % Hk
    q = qkv[:, :Hk * Dk].float().view(T, Hk, Dk)
    k = qkv[:, Hk * Dk:2 * Hk * Dk].float().view(T, Hk, Dk)
    v = qkv[:, 2 * Hk * Dk:].float().view(T, Hv, Dv)
    q = q * torch.rsqrt(q.pow(2).sum(-1, keepdim=True) + eps) * (Dv ** -0.5)
    k = k * torch.rsqrt(k.pow(2).sum(-1, keepdim=True) + eps)
    g = torch.nn.functional.softplus(alpha.float() + dt_bias.float()) * a_log.float()      # [T, Hv], log of the decay
    b = torch.sigmoid(beta.float())                                                         # [T, Hv]
    # row index of every (sequence, padded position); padding points at one appended row of zeros: a padded token has
    # zero k, v, beta and log-decay, so it changes neither the state nor any real token's output
    if B == 1 and lens[0] == L:
        idx = None
    else:
        pos = torch.arange(L, device=dev).unsqueeze(0)
        start = torch.tensor(cu[:-1], device=dev).unsqueeze(1)
        ln = torch.tensor(lens, device=dev).unsqueeze(1)
        idx = torch.where(pos < ln, start + pos, torch.full((), T, device=dev))            # [B, L]

    def chunks(t, per_kv_head=False):   # [T, H, ...] -> [B * Hv, nc, C, ...]
        if idx is not None:
            t = torch.cat([t, t.new_zeros((1,) + tuple(t.shape[1:]))], 0)[idx]              # [B, L, H, ...]
        else:
            t = t.unsqueeze(0)
        if per_kv_head:
            t = t[:, :, hk]
        t = t.reshape(B, nc, C, *t.shape[2:]).movedim(3, 1)                                  # [B, Hv, nc, C, ...]
        return t.reshape(B * Hv, nc, C, *t.shape[4:])
    Q, K, V = chunks(q, True), chunks(k, True), chunks(v)
    G, Bt = chunks(g), chunks(b)                                             # [B * Hv, nc, C]
    cum = G.cumsum(-1)
    tril = torch.ones(C, C, dtype=torch.bool, device=dev).tril()
    M = torch.where(tril, torch.exp((cum.unsqueeze(-1) - cum.unsqueeze(-2)).clamp(max=0.0)), torch.zeros((), device=dev))
    KT = K.transpose(-1, -2)
    A = (Bt.unsqueeze(-1) * (K @ KT) * M).tril(-1)                           # strictly lower: token i sees tokens j < i
    lhs = A + torch.eye(C, device=dev)
    decay = torch.exp(cum).unsqueeze(-1)                                     # decay from the chunk's start to each token
    rhs = torch.cat([Bt.unsqueeze(-1) * V, Bt.unsqueeze(-1) * decay * K], -1)
    sol = torch.linalg.solve_triangular(lhs, rhs, upper=False, unitriangular=True)          # [.., C, Dv + Dk]
    U0, W = sol[..., :Dv], sol[..., Dv:]
    P = (Q @ KT) * M
    Qd = Q * decay
    Kd = K * torch.exp(cum[..., -1:] - cum).unsqueeze(-1)
    gamma = torch.exp(cum[..., -1])                                          # [B * Hv, nc]
    S = states[0].float() if B == 1 else torch.cat([st.float() for st in states], 0)        # [B * Hv, Dv, Dk]
    if carry is not None:                # the chunk-after-chunk part as one kernel (csrc/gdn_chunk.cu)
        S = S.contiguous()
        core = carry(U0, W, Qd, Kd, P, gamma, S)                             # [B * Hv, nc, C, Dv]; S updated in place
    else:
        outs = []
        for c in range(nc):
            St = S.transpose(-1, -2)                                         # [.., Dk, Dv]
            U = U0[:, c] - W[:, c] @ St
            outs.append(Qd[:, c] @ St + P[:, c] @ U)                         # [.., C, Dv]
            S = gamma[:, c].view(-1, 1, 1) * S + U.transpose(-1, -2) @ Kd[:, c]
        core = torch.stack(outs, 1)
    for i, st in enumerate(states):
        if st.data_ptr() != S.data_ptr():
            st.copy_(S[i * Hv:(i + 1) * Hv])
    core = core.reshape(B, Hv, L, Dv).transpose(1, 2)                        # [B, L, Hv, Dv]
    if idx is None:
        core = core.reshape(T, Hv, Dv)
    else:
        core = torch.cat([core[i, :lens[i]] for i in range(B)], 0)           # back to packed rows
    core = core * torch.rsqrt(core.pow(2).mean(-1, keepdim=True) + eps) * norm_w.float()
    return (core * torch.nn.functional.silu(z.float().view(T, Hv, Dv))).reshape(T, Hv * Dv)


def mamba2_recurrent(xbc, dt, dt_bias, A, D, state, *, H, P, G, N):
    """One sequence.  state [H, P, N] updated in place.  Returns y [n, H*P] (before gating)."""
    n = xbc.shape[0]
    y = torch.zeros(n, H * P)
    grp = torch.arange(H) // (H // G)
    for t in range(n):
        x = xbc[t, :H * P].float().view(H, P)
        Bm = xbc[t, H * P:H * P + G * N].float().view(G, N)[grp]
        Cm = xbc[t, H * P + G * N:].float().view(G, N)[grp]
        d = torch.nn.functional.softplus(dt[t].float() + (dt_bias.float() if dt_bias is not None else 0.0))
        dA = torch.exp(d * A.float())
        state.mul_(dA.view(H, 1, 1)).add_(torch.einsum("hp,hn->hpn", x * d.view(H, 1), Bm))
        yy = torch.einsum("hpn,hn->hp", state, Cm)
        if D is not None:
            yy = yy + D.float().view(H, 1) * x
        y[t] = yy.reshape(-1)
    return y


def mamba2_chunked(xbc, dt, dt_bias, A, D, state, *, H, P, G, N, chunk: int = 64, carry=None):
    """:func:`mamba2_recurrent` in chunked (state-space duality) form: inside a chunk the outputs are one masked
    matrix product ``(decay * C B^T) (dt * x)``, the state is carried from chunk to chunk by two small products.
    One sequence; ``state`` [H, P, N] is updated in place; runs on the inputs' device.  ``carry`` replaces the loop
    over the chunks (a kernel on CUDA).  Returns y [n, H*P]."""
    n = xbc.shape[0]
    dev = xbc.device
    Cn = chunk
    nc = (n + Cn - 1) // Cn
    pad = nc * Cn - n
    grp = torch.arange(H, device=dev) // (H // G)
    x = xbc[:, :H * P].float().view(n, H, P)
    Bm = xbc[:, H * P:H * P + G * N].float().view(n, G, N)[:, grp]           # [n, H, N]
    Cm = xbc[:, H * P + G * N:].float().view(n, G, N)[:, grp]
    d = torch.nn.functional.softplus(dt.float() + (dt_bias.float() if dt_bias is not None else 0.0))    # [n, H]
    la = d * A.float()                                                        # log of the per-token decay

    def chunks(t):                      # [n, H, ...] -> [H, nc, Cn, ...]; padded tokens: zero input, decay 1
        if pad:
            t = torch.cat([t, t.new_zeros((pad,) + tuple(t.shape[1:]))], 0)
        return t.view(nc, Cn, *t.shape[1:]).movedim(2, 0)
    X, Bc, Cc = chunks(x * d.unsqueeze(-1)), chunks(Bm), chunks(Cm)
    cum = chunks(la).cumsum(-1)                                               # [H, nc, Cn]
    tril = torch.ones(Cn, Cn, dtype=torch.bool, device=dev).tril()
    M = torch.where(tril, torch.exp((cum.unsqueeze(-1) - cum.unsqueeze(-2)).clamp(max=0.0)), torch.zeros((), device=dev))
    Y_in = ((Cc @ Bc.transpose(-1, -2)) * M) @ X                              # contributions from inside the chunk
    Cd = Cc * torch.exp(cum).unsqueeze(-1)                                    # reads of the incoming state
    Xd = X * torch.exp(cum[..., -1:] - cum).unsqueeze(-1)                     # writes that survive to the chunk's end
    gamma = torch.exp(cum[..., -1])
    if carry is not None:
        # the chunk-carry kernel of the delta rule (csrc/gdn_chunk.cu) with nothing to correct (W = 0) and no intra-chunk
        # term of its own (P = 0): out = Cd S^T, S <- gamma S + Xd^T B; ``state`` [H, P, N] is updated in place
        zw = torch.zeros((H, nc, Cn, N), dtype=torch.float32, device=dev)
        zp = torch.zeros((H, nc, Cn, Cn), dtype=torch.float32, device=dev)
        y = Y_in + carry(Xd, zw, Cd, Bc, zp, gamma, state)
    else:
        S = state.float()                                                     # [H, P, N]
        outs = []
        for c in range(nc):
            outs.append(Y_in[:, c] + Cd[:, c] @ S.transpose(-1, -2))          # [H, Cn, P]
            S = gamma[:, c].view(H, 1, 1) * S + Xd[:, c].transpose(-1, -2) @ Bc[:, c]
        state.copy_(S)
        y = torch.stack(outs, 1)
    y = y.reshape(H, nc * Cn, P)[:, :n].transpose(0, 1)                        # [n, H, P]
    if D is not None:
        y = y + D.float().view(1, H, 1) * x
    return y.reshape(n, H * P)


"""The state-matrix recurrence kernel against a float64 walk: both forms, every row padding, CTAs of 8, 16 and 32
columns and columns over 8 or 16 lanes (the launcher picks by the step's size), column counts that fill no CTA, sequences whose lengths sit on and
around the borders of the staged chunks, states that come from an earlier step, slots in any order."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def walk(q, k, g, beta, v, S, delta):
    """One head, float64: q, k, g [n, rows], v [n, cols], beta [n] or None, S [rows, cols] (updated in place)."""
    out = torch.zeros(q.shape[0], S.shape[1], dtype=torch.float64)
    for t in range(q.shape[0]):
        if delta:
            S *= g[t][:, None]
            u = beta[t] * (v[t] - S.T @ k[t])
            S += torch.outer(k[t], u)
        else:
            S *= g[t][:, None]
            S += torch.outer(k[t], v[t])
        out[t] = S.T @ q[t]
    return out


CASES = [
    # rows, columns, heads, group, sequence lengths
    (128, 128, 2, 2, [1, 15, 16, 17, 33]),              # 8-column CTAs
    (20, 36, 3, 1, [31, 32, 1, 2]),                     # rows padded to 32, a last CTA with 4 live columns
    (64, 1, 1, 1, [40]),                                # one column
    (256, 24, 2, 1, [7, 8, 9, 17]),                     # 32 rows a lane: chunks of 8 tokens
    (32, 64, 4, 2, [3] * 38 + [19, 1]),                 # 40 x 4 x 2 CTAs of 32 columns
    (64, 64, 4, 4, [5] * 20 + [18]),                    # 21 x 4 x 4: CTAs of 16 columns
    (128, 40, 2, 1, [17, 5]),                           # a small step: a column over 16 lanes, 8 rows a lane
]


@pytest.mark.parametrize("delta", [False, True], ids=["gated_write", "delta_rule"])
@pytest.mark.parametrize("case", CASES, ids=lambda c: "r{}c{}h{}g{}n{}".format(c[0], c[1], c[2], c[3], len(c[4])))
def test_recurrence(case, delta):
    from rustingstrata_b200.kernels import ops
    rows, cols, heads, group, lens = case
    if not delta:
        group = 1
    gen = torch.Generator().manual_seed(rows + cols + heads + len(lens) + int(delta))
    rp = ops.state_rows_pad(rows)
    T, n = sum(lens), len(lens)
    qk_heads = heads // group
    pad = lambda x, hn: torch.nn.functional.pad(x.view(T, hn, rows), (0, rp - rows)).reshape(T, hn * rp).contiguous()     # noqa: E731
    q = torch.randn(T, qk_heads * rows, generator=gen)
    k = torch.randn(T, qk_heads * rows, generator=gen) / rows ** 0.5 if delta else torch.rand(T, heads * rows, generator=gen)
    g = torch.rand(T, heads * rows, generator=gen) * 0.5 + 0.5
    beta = torch.rand(T, heads, generator=gen) if delta else None
    v = torch.randn(T, heads * cols, generator=gen)
    slots = torch.randperm(n + 3, generator=gen)[:n].to(torch.int32)
    state0 = torch.randn(n + 3, heads, cols, rp, generator=gen) * 0.3
    state0[..., rows:] = 0.0                                                   # padded rows stay zero
    q_start = np.concatenate([[0], np.cumsum(lens)]).astype(np.int32)
    ref_out = torch.zeros(T, heads, cols, dtype=torch.float64)
    ref_state = state0.double().clone()
    for s in range(n):
        a, b = int(q_start[s]), int(q_start[s + 1])
        for h in range(heads):
            hq = h // group
            S = ref_state[slots[s], h, :, :rows].T.contiguous()                # [rows, cols]
            ref_out[a:b, h] = walk(q[a:b].view(-1, qk_heads, rows)[:, hq].double(),
                                   k[a:b].view(-1, qk_heads if delta else heads, rows)[:, hq if delta else h].double(),
                                   g[a:b].view(-1, heads, rows)[:, h].double(), beta[a:b, h].double() if delta else None,
                                   v[a:b].view(-1, heads, cols)[:, h].double(), S, delta)
            ref_state[slots[s], h, :, :rows] = S.T
    dev = torch.device("cuda")
    state = state0.view(n + 3, -1).contiguous().to(dev)
    out = torch.full((T, heads * cols), float("nan"), device=dev)
    ops.state_recurrence(pad(q, qk_heads).to(dev), pad(k, qk_heads if delta else heads).to(dev), pad(g, heads).to(dev),
                         beta.to(dev) if delta else None, v.to(dev), out, state, torch.from_numpy(q_start).to(dev), slots.to(dev), n,
                         heads, group, rp, cols, delta)
    torch.cuda.synchronize()
    scale = ref_out.abs().max().item()
    assert (out.cpu().double().view(T, heads, cols) - ref_out).abs().max().item() <= 2e-5 * scale
    got = state.cpu().double().view(n + 3, heads, cols, rp)
    assert (got - ref_state).abs().max().item() <= 2e-5 * ref_state.abs().max().item()
    assert (got[..., rows:] == 0).all()

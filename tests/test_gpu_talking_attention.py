"""The tensor-core form of talking-heads attention against a plain float64 computation over the same bfloat16 cache, and
against the CUDA-core form: head counts with and without grouping, head sizes up to 128, windows, unequal sequences on
shuffled pages, every query tile size, and key tiles dealt out over several CTAs (with parts that get no tile at all)."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def plain(q, k, v, talk, sink, gate, scale, window, first_pos):
    """q [n, H, dk] float64 at positions first_pos.., k [L, G, dk], v [L, G, dv]: out [n, H, dv]."""
    n, H, _ = q.shape
    L, G, dv = v.shape
    r = H // G
    raw = torch.stack([(q[:, h] @ k[:, h // r].T) * scale for h in range(H)])            # [H, n, L]
    mixed = torch.einsum("hg,gij->hij", talk, raw) if talk is not None else raw
    out = torch.zeros(n, H, dv, dtype=torch.float64)
    for i in range(n):
        pos = first_pos + i
        lo = max(0, pos - window + 1) if window else 0
        for h in range(H):
            s = mixed[h, i, lo:pos + 1]
            top = s.max() if sink is None else torch.maximum(s.max(), sink[h])
            e = torch.exp(s - top)
            den = e.sum() + (torch.exp(sink[h] - top) if sink is not None else 0.0)
            out[i, h] = (e / den) @ v[lo:pos + 1, h // r]
    return out * gate[:, :, None] if gate is not None else out


CASES = [
    # H, G, dk, dv, window, talk, sink, gate
    (16, 4, 64, 64, 0, True, True, True),
    (8, 8, 32, 16, 0, True, True, False),
    (32, 4, 16, 64, 0, True, True, True),
    (4, 1, 128, 128, 0, True, False, True),
    (6, 3, 48, 32, 37, True, True, True),
    (2, 2, 16, 16, 0, False, True, True),
    (12, 2, 32, 80, 70, True, False, False),
]


@pytest.mark.parametrize("case", CASES, ids=lambda c: "h{}g{}k{}v{}w{}".format(*c[:5]))
@pytest.mark.parametrize("qt,parts", [(16, 1), (8, 3), (4, 1), (4, 7), (16, 2)])
def test_tensor_core_form(case, qt, parts):
    from rustingstrata_b200.kernels import ops
    H, G, dk, dv, window, has_talk, has_sink, has_gate = case
    most = ops.talking_attention_mma_q_per_cta(H, G, dk, dv)
    assert most >= 4, "a shape the tensor-core form is meant to take"
    qt = min(qt, most)
    dev = torch.device("cuda")
    gen = torch.Generator().manual_seed(H * 1000 + dk + qt + parts)
    page, hdp = 16, (max(dk, dv) + 7) // 8 * 8
    # sequences: (keys after the step, queries in the step): a portion from the start, a portion after 150 keys, a
    # single token far in, a single token that is the sequence's first
    seqs = [(77, 77), (150 + 41, 41), (333, 1), (1, 1)]
    n_pages = sum((kv + page - 1) // page for kv, _ in seqs) + 3
    order = torch.randperm(n_pages, generator=gen).tolist()
    cache = torch.zeros(n_pages, 2, G, page, hdp, dtype=torch.bfloat16)
    table = torch.full((len(seqs), max((kv + page - 1) // page for kv, _ in seqs)), -1, dtype=torch.int32)
    ks, vs = [], []
    for s, (kv, _) in enumerate(seqs):
        k = torch.randn(kv, G, dk, generator=gen).to(torch.bfloat16)
        v = torch.randn(kv, G, dv, generator=gen).to(torch.bfloat16)
        ks.append(k), vs.append(v)
        for b in range((kv + page - 1) // page):
            pg = order.pop()
            table[s, b] = pg
            n = min(page, kv - b * page)
            cache[pg, 0, :, :n, :dk] = k[b * page:b * page + n].transpose(0, 1)
            cache[pg, 1, :, :n, :dv] = v[b * page:b * page + n].transpose(0, 1)
    T = sum(n for _, n in seqs)
    q = torch.randn(T, H * dk, generator=gen) * 1.5
    gate = torch.rand(T, H, generator=gen) if has_gate else None
    talk = (torch.eye(H) * 0.7 + torch.randn(H, H, generator=gen) * 0.3) if has_talk else None
    sink = torch.randn(H, generator=gen) * 2 if has_sink else None
    scale = dk ** -0.5
    q_start = np.concatenate([[0], np.cumsum([n for _, n in seqs])]).astype(np.int32)
    kv_len = np.array([kv for kv, _ in seqs], dtype=np.int32)
    ref = torch.cat([plain(q[q_start[s]:q_start[s + 1]].double().view(-1, H, dk), ks[s].double(), vs[s].double(),
                           None if talk is None else talk.double(), None if sink is None else sink.double(),
                           None if gate is None else gate[q_start[s]:q_start[s + 1]].double(), scale, window, kv - n)
                     for s, (kv, n) in enumerate(seqs)]).view(T, H * dv)
    work, rows = [], 0
    for s, (kv, n) in enumerate(seqs):
        for q0 in range(0, n, qt):
            nq = min(qt, n - q0)
            for p in range(parts):
                work.append((s, q0, p, parts, rows))
            rows += parts * nq if parts > 1 else 0
    work = torch.tensor(work, dtype=torch.int32).flatten()
    d = lambda t: None if t is None else t.to(dev)                                  # noqa: E731
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    out = torch.full((T, H * dv), float("nan"), dtype=torch.float32, device=dev)
    partial = torch.full((max(rows, 1), H * (dv + 2)), float("nan"), dtype=torch.float32, device=dev)
    ops.talking_attention_mma(d(q), d(gate), d(cache), d(table), page, d(torch.from_numpy(q_start)), d(torch.from_numpy(kv_len)),
                              d(work), len(work) // 5, parts > 1, d(talk), d(sink), out, partial if parts > 1 else None,
                              H, G, dk, dv, window, qt, scale, status)
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    err = (out.cpu().double() - ref).abs().max().item() / ref.abs().max().item()
    assert err < 3e-5, err
    # the CUDA-core form over the same cache
    simt_q = min(qt, ops.talking_attention_q_per_cta(H, dk, dv))
    w2 = torch.tensor([(s, q0) for s, (kv, n) in enumerate(seqs) for q0 in range(0, n, simt_q)], dtype=torch.int32).flatten()
    out2 = torch.full((T, H * dv), float("nan"), dtype=torch.float32, device=dev)
    ops.talking_attention(d(q), d(gate), d(cache), d(table), page, d(torch.from_numpy(q_start)), d(torch.from_numpy(kv_len)),
                          d(w2), len(w2) // 2, d(talk), d(sink), out2, H, G, dk, dv, window, simt_q, scale, status)
    torch.cuda.synchronize()
    assert (out2.cpu().double() - ref).abs().max().item() / ref.abs().max().item() < 3e-5
    # a bfloat16 result is the rounding of the same numbers
    out3 = torch.zeros((T, H * dv), dtype=torch.bfloat16, device=dev)
    ops.talking_attention_mma(d(q), d(gate), d(cache), d(table), page, d(torch.from_numpy(q_start)), d(torch.from_numpy(kv_len)),
                              d(work), len(work) // 5, parts > 1, d(talk), d(sink), out3, partial if parts > 1 else None,
                              H, G, dk, dv, window, qt, scale, status)
    torch.cuda.synchronize()
    assert (out3.float() - out).abs().max().item() <= 2 ** -8 * out.abs().max().item()

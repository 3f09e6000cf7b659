"""The Kozasun decoder inside the engine against the plain float64 implementation (tests/plain_kozasun.py).

Every mechanism alone (one-layer models), whole prompts against token-by-token decoding, portions down to two tokens,
mixed batches against each request alone, pages and state slots that are freed and used again, keys just inside and
just outside every block and window in prompts and in decoding, far keys and page borders with peaked attention, sinks
that matter and states that last, the first tokens of a sequence, long decoding, several sizes, the residual stream
layer by layer, greedy generation through the scheduler, and the command line.
"""
import copy
import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import kozasun_models as M
import plain_kozasun as P
from helpers import ROOT

pytestmark = pytest.mark.gpu

TOL = {"float32": 2e-5, "bfloat16": 4e-2}         # max |difference| / max |reference logit|
# With peaked attention a rounding of a score moves the weights of the keys by as much more, and a state that lasts
# for hundreds of tokens adds up as many roundings.
TOL_SHARP = {"float32": 1.5e-3, "bfloat16": 8e-2}
DTYPES = ["float32", "bfloat16"]


def rel_err(got, ref):
    ref = np.asarray(ref, dtype=np.float64)
    return float(np.max(np.abs(np.asarray(got, dtype=np.float64) - ref)) / np.max(np.abs(ref)))


def runner_for(path, dtype, page_size=16, pool_tokens=1024, max_seqs=4, max_batch_tokens=1024):
    from rustingstrata_b200.config import EngineConfig
    from rustingstrata_b200.engine import ModelRunner
    eng = EngineConfig(dtype=dtype, page_size=page_size, num_pages=(pool_tokens + page_size - 1) // page_size,
                       max_seqs=max_seqs, max_batch_tokens=max_batch_tokens, max_logit_rows=max_batch_tokens)
    return ModelRunner.from_dir(path, eng)


def tokens_for(cfg, n, seed):
    return np.random.default_rng(seed).integers(0, cfg["vocab"], size=n).tolist()


def plain_logits(cfg, w, toks):
    return P.forward(cfg, w, toks).numpy()


_MODELS = {}


def model(tmp_path_factory, key, cfg, seed=0, sharp=False, steady=False):
    """The bfloat16 engine rounds the router's input, so its models get corrections that decide the choice alone."""
    if key not in _MODELS:
        path = str(tmp_path_factory.mktemp("kozasun") / key)
        _MODELS[key] = (path,) + M.make(path, cfg, seed, sharp, steady)
    return _MODELS[key]


def model_for(tmp_path_factory, dtype, key, cfg, seed=0, sharp=False):
    """The model a test runs in this element type.  The bfloat16 engine gets a steady router, and half the sharpening:
    its queries, keys and latents are rounded to 8 bits, and scores that are scaled up sixfold carry that rounding into
    the weights sixfold."""
    steady = dtype == "bfloat16"
    return model(tmp_path_factory, key + ("_steady" if steady else ""), cfg, seed, 0.5 * sharp if steady else sharp, steady)


def assert_rows_within(err, tol, what):
    """Per-position errors of a run with sharpened weights: none beyond one and a half times the tolerance and at most
    one position in fifty beyond the tolerance itself (where a query weighs two keys nearly alike, the rounding of a
    score tips the balance; a fault of a mask, a page or a state moves whole stretches of positions by far more)."""
    err = np.asarray(err)
    over = err > tol
    first = int(np.argmax(over)) if over.any() else -1
    assert err.max() <= 1.5 * tol and over.sum() <= max(1, 0.02 * len(err)), \
        f"{what}: worst {err.max():.3e}, {int(over.sum())} of {len(err)} positions over {tol}, the first at {first}"


def step_all(r, rid, toks, want=None):
    from rustingstrata_b200.engine import StepEntry
    out = r.step([StepEntry(rid, toks, list(range(len(toks))) if want is None else want)])
    r.check_status()
    return None if out is None else out.cpu().numpy()


# ----------------------------------------------------------------------------- each mechanism alone
ONE_LAYER = {
    "attention_grouped_rotated_prefix_blocks": M.config(97, 64, [(M.attention(6, 3, 16, 8, rot=(8, 50.0), chunk=11), None)], streams=2),
    "attention_one_kv_head_no_rotation_no_blocks": M.config(97, 64, [(M.attention(3, 1, 24, 40, scale=0.3), None)], streams=2),
    "attention_all_rotated_heads_equal": M.config(97, 72, [(M.attention(2, 2, 12, 12, rot=(12, 1000.0), chunk=32), None)], eps=1e-5),
    "attention_one_head_blocks_of_one_page": M.config(97, 64, [(M.attention(1, 1, 32, 16, rot=(4, 7.0), chunk=16), None)], streams=1),
    "retention_padded_rows_rotated": M.config(97, 64, [(M.retention(3, 24, 20, (0.9, 0.99, 0.6), rot=(24, 100.0)), None)], streams=2),
    "retention_rotated_prefix_two_column_blocks": M.config(97, 64, [(M.retention(2, 40, 36, (0.95, 0.999), rot=(10, 1e4)), None)]),
    "retention_no_rotation_few_columns": M.config(97, 64, [(M.retention(1, 8, 4, (0.97,)), None)], streams=3),
    "latent_window": M.config(97, 64, [(M.latent(3, 16, 24, 40, window=9, scale=0.4), None)], streams=2),
    "latent_no_window_one_head": M.config(97, 72, [(M.latent(1, 32, 8, 16), None)], eps=1e-5),
    "latent_rank_that_needs_padding": M.config(97, 64, [(M.latent(4, 8, 16, 21, window=16), None)], streams=2),
    "dense_feed_forward": M.config(97, 64, [(M.retention(1, 8, 8, (0.9,)), M.dense(120))], streams=2, embedding_scale=3.0),
    "experts_in_groups": M.config(97, 64, [(M.retention(1, 8, 8, (0.9,)), M.moe(12, 3, 24, scale=2.0, groups=(4, 2), shared=40))], streams=2),
    "experts_one_group_kept": M.config(97, 64, [(M.retention(1, 8, 8, (0.9,)), M.moe(10, 4, 16, scale=0.7, groups=(2, 1), shared=8))]),
    "experts_all_groups_kept": M.config(97, 64, [(M.retention(1, 8, 8, (0.9,)), M.moe(6, 2, 16, groups=(3, 3)))], streams=2),
    "experts_top_one_no_groups_no_shared": M.config(97, 64, [(M.retention(1, 8, 8, (0.9,)), M.moe(5, 1, 32, scale=1.0))], streams=4),
    "shared_layer_runs_twice": M.config(97, 64, [(M.retention(2, 16, 16, (0.9, 0.99)), M.dense(48)), 0, (M.latent(2, 16, 16, 24, window=6), None), 2],
                                        streams=2),
}
# a layer that runs another layer's tensors with a window of its own
ONE_LAYER["shared_layer_with_its_own_window"] = M.config(97, 64, [(M.latent(2, 16, 16, 24, window=6), M.dense(48)), 0], streams=2)
ONE_LAYER["shared_layer_with_its_own_window"]["layers"][1]["mixer"]["mask"]["size"] = 11


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", sorted(ONE_LAYER))
def test_mechanism_alone(tmp_path_factory, name, dtype):
    """One mechanism per model: the stream after every layer run and the logits of every position, whole and in portions."""
    cfg = ONE_LAYER[name]
    path, cfg, w = model_for(tmp_path_factory, dtype, "one_" + name, cfg, seed=5)
    toks = tokens_for(cfg, 45, 3)
    streams = []
    ref = P.forward(cfg, w, toks, on_layer=lambda i, x: streams.append(x.clone())).numpy()
    r = runner_for(path, dtype, page_size=8, pool_tokens=256)
    from rustingstrata_b200.engine import StepEntry
    got_streams = []
    logits = r.step([StepEntry("a", toks, list(range(len(toks))))],
                    on_layer=lambda k, x: got_streams.append(x.float().cpu().numpy().copy()))
    r.check_status()
    assert len(got_streams) == len(streams) == len(cfg["layers"])
    for i, (g, s) in enumerate(zip(got_streams, streams)):
        assert rel_err(g, s.numpy()) <= TOL[dtype], f"{name} {dtype}: stream after layer run {i}"
    assert rel_err(logits.cpu().numpy(), ref) <= TOL[dtype]
    r.release("a")
    got, pos = [], 0
    for n in [2, 5, 1, 2, 17, 3, 2, 13]:
        got.append(step_all(r, "b", toks[pos:pos + n]))
        pos += n
    assert pos == len(toks)
    assert rel_err(np.concatenate(got), ref) <= TOL[dtype], f"{name} {dtype}: portions"


# ----------------------------------------------------------------------------- whole models, every cutting
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["P", "Q", "R", "S"])
def test_cuttings_of_a_prompt(tmp_path_factory, name, dtype):
    """Whole, last tokens one by one (captured steps), portions of several sizes down to two tokens."""
    path, cfg, w = model_for(tmp_path_factory, dtype, name, name, seed=11)
    toks = tokens_for(cfg, 150, 5)
    ref = plain_logits(cfg, w, toks)
    r = runner_for(path, dtype, page_size=16, pool_tokens=512)
    assert rel_err(step_all(r, "w", toks), ref) <= TOL[dtype], "whole"
    r.release("w")
    n = len(toks) - 40
    got = [step_all(r, "d", toks[:n])] + [step_all(r, "d", [t]) for t in toks[n:]]
    assert rel_err(np.concatenate(got), ref) <= TOL[dtype], "decoding"
    if r.model.capturable:
        assert r.graph_replays > 0
    r.release("d")
    got, pos, k = [], 0, 0
    sizes = [7, 2, 13, 2, 5, 3, 29, 2, 16, 4, 11, 2, 1, 1, 31]
    while pos < len(toks):
        m = min(sizes[k % len(sizes)], len(toks) - pos)
        got.append(step_all(r, "p", toks[pos:pos + m]))
        pos, k = pos + m, k + 1
    assert rel_err(np.concatenate(got), ref) <= TOL[dtype], "portions"


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["P", "R"])
def test_mixed_batches_with_pages_and_slots_used_again(tmp_path_factory, name, dtype):
    """Up to three live requests of unequal length in a pool that cannot hold all seven at once: portions of some
    beside single tokens of others, requests left out of steps, and every row equal to the request run alone.  A slot
    that a request with a long-lived state has left is taken by the next one, which must start from zero."""
    from rustingstrata_b200.engine import StepEntry
    path, cfg, w = model_for(tmp_path_factory, dtype, name + "_sharp", name, seed=21, sharp=True)
    tol = TOL_SHARP[dtype]
    lengths = [70, 33, 121, 9, 64, 1, 47]
    toks = {f"r{i}": tokens_for(cfg, n, 40 + i) for i, n in enumerate(lengths)}
    ref = {k: plain_logits(cfg, w, t) for k, t in toks.items()}
    scale = max(np.max(np.abs(v)) for v in ref.values())      # one scale for all requests: a one-token request has no spread of its own
    r = runner_for(path, dtype, page_size=16, pool_tokens=256, max_seqs=3)
    rng = np.random.default_rng(9)
    waiting, live, pos = list(toks), [], {}
    worst, rows, slots_seen, errs = 0.0, 0, {}, []
    while waiting or live:
        while waiting and len(live) < 3 and sum((len(toks[x]) + 15) // 16 for x in live + [waiting[0]]) <= 16:
            live.append(waiting.pop(0))
            pos[live[-1]] = 0
        chosen = [x for x in live if rng.random() < 0.7] or [live[0]]
        entries, where = [], []
        for rid in chosen:
            left = len(toks[rid]) - pos[rid]
            n = 1 if left <= 12 else int(min(rng.choice([2, 3, 5, 9, 17, 31]), left - 12))
            want = list(range(n))
            entries.append(StepEntry(rid, toks[rid][pos[rid]:pos[rid] + n], want))
            where += [(rid, pos[rid] + j) for j in want]
            pos[rid] += n
        out = r.step(entries).cpu().numpy()
        r.check_status()
        for rid in chosen:
            slots_seen.setdefault(r.cache.slot(rid), set()).add(rid)
        for row, (rid, p) in zip(out, where):
            e = float(np.max(np.abs(row - ref[rid][p])) / scale)
            worst, rows = max(worst, e), rows + 1
            errs.append(e)
            assert e <= 1.5 * tol, f"{name} {dtype}: request {rid} position {p}: {e:.3e}"
        for rid in [x for x in live if pos[x] == len(toks[x])]:
            live.remove(rid)
            r.release(rid)
    r.cache.check()
    assert rows == sum(lengths)
    assert_rows_within(errs, tol, "mixed batches")
    print(f"mixed {name} {dtype}: worst {worst:.3e}")
    assert max(len(v) for v in slots_seen.values()) >= 2, "no state slot was used again"
    assert all(p.reuses > 0 for p in r.cache.pools), "no page was used again"


# ----------------------------------------------------------------------------- edges of blocks and windows
def edge_positions(cfg, n):
    """Positions whose query has a key just inside or just outside an edge: the first and last of every block, and
    every position from a window's size on."""
    out = set()
    for L in cfg["layers"]:
        size = (L["mixer"].get("mask") or {}).get("size")
        if not size:
            continue
        if L["type"] == "attention":
            out.update(p for p in range(n) if p >= size and p % size in (0, 1, size - 1))
        else:
            out.update(range(size - 1, n))
    return sorted(out)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["P", "R", "S"])
def test_edges_of_blocks_and_windows(tmp_path_factory, name, dtype):
    """Peaked attention, so that a key more or a key less shows.  The premise first, on the plain implementation: with
    every block and window one key larger, and one key smaller, the logits at many edge positions move by more than
    three times the tolerance (an engine that is one key off would be wrong there by twice the tolerance).  Then the engine: the prompt whole, a prompt that ends in the middle of a block and of a
    window followed by single tokens that cross their edges, and portions that start and end on and beside the edges."""
    path, cfg, w = model_for(tmp_path_factory, dtype, name + "_sharp", name, seed=21, sharp=True)
    tol = TOL_SHARP[dtype]
    n = {"P": 150, "R": 460, "S": 60}[name]
    toks = tokens_for(cfg, n, 31)
    ref = plain_logits(cfg, w, toks)
    edges = edge_positions(cfg, n)
    assert len(edges) >= 10
    scale = np.max(np.abs(ref))
    for delta in (1, -1):
        off = plain_logits(M.with_mask_sizes(cfg, delta), w, toks)
        moved = np.max(np.abs(off - ref)[edges], axis=1) / scale
        assert (moved > 3 * tol).sum() >= max(5, 0.1 * len(edges)), f"premise: mask sizes {delta:+d}"
    r = runner_for(path, dtype, page_size=16, pool_tokens=512, max_batch_tokens=512)
    err = np.max(np.abs(step_all(r, "w", toks) - ref), axis=1) / scale
    assert_rows_within(err, tol, "whole")
    r.release("w")
    sizes = sorted({(L["mixer"].get("mask") or {}).get("size") or 1 for L in cfg["layers"]})
    cut = n - min(n - 2, max(sizes) + 40)              # single tokens from here on: across every edge at least once
    got = [step_all(r, "d", toks[:cut])] + [step_all(r, "d", [t]) for t in toks[cut:]]
    err = np.max(np.abs(np.concatenate(got) - ref), axis=1) / scale
    assert_rows_within(err, tol, f"decoding from {cut}")
    r.release("d")
    marks = sorted({0, n} | {p + d for s in sizes if s > 1 for p in range(s, n, s) for d in (-1, 0, 1) if 0 < p + d < n})
    marks = marks[:: max(1, len(marks) // 40)] + [n] if len(marks) > 40 else marks
    got = [step_all(r, "p", toks[a:b]) for a, b in zip(marks[:-1], marks[1:]) if b > a]
    err = np.max(np.abs(np.concatenate(got) - ref), axis=1) / scale
    assert_rows_within(err, tol, "portions cut at the edges")


def without_masks(cfg):
    c = copy.deepcopy(cfg)
    for L in c["layers"]:
        L["mixer"].pop("mask", None)
    return c


@pytest.mark.parametrize("dtype", DTYPES)
def test_far_keys_page_borders_and_long_state(tmp_path_factory, dtype):
    """No blocks and no windows, peaked attention (each query looks at one or two keys, at any distance), raised sinks
    and retention states that last for hundreds of tokens, over 700 positions: every position of the prompt, then
    decoding across page borders and the borders of the attention's key tiles, against the plain implementation."""
    path, cfg, w = model_for(tmp_path_factory, dtype, "R_far", without_masks(M.CONFIGS["R"]), seed=21, sharp=True)
    toks = tokens_for(cfg, 700, 77)
    ref = plain_logits(cfg, w, toks)
    r = runner_for(path, dtype, page_size=16, pool_tokens=768, max_batch_tokens=768)
    n = 600
    got = [step_all(r, "a", toks[:n])] + [step_all(r, "a", [t]) for t in toks[n:n + 60]] + [step_all(r, "a", toks[n + 60:])]
    got = np.concatenate(got)
    err = np.max(np.abs(got - ref), axis=1) / np.max(np.abs(ref))
    print(f"far keys {dtype}: worst {err.max():.3e}")
    assert_rows_within(err, TOL_SHARP[dtype], "far keys")


def test_sharp_weights_look_far_back_keep_state_and_feel_the_sink():
    """The premises of the tests with sharp weights, checked on the plain implementation: dropping the oldest 100 tokens
    changes the last logits by more than twice the widest tolerance (so a lost far key would show in either engine),
    and so does taking the sinks out of the denominators; a retention layer alone still feels tokens 200 back by ten
    times the 32-bit engine's tolerance."""
    cfg = without_masks(M.CONFIGS["R"])
    w = M.draw_weights(cfg, 21, sharp=True)
    toks = tokens_for(cfg, 700, 77)
    full = plain_logits(cfg, w, toks)[-20:]
    cut = plain_logits(cfg, w, toks[100:])[-20:]
    big = 2 * TOL_SHARP["bfloat16"]
    assert np.max(np.abs(full - cut)) / np.max(np.abs(full)) > big
    short = toks[:120]
    full = plain_logits(cfg, w, short)
    no_sink = dict(w, **{k: torch.full_like(v, -60.0) for k, v in w.items() if k.endswith("mix.sink")})
    assert np.max(np.abs(full - plain_logits(cfg, no_sink, short))) / np.max(np.abs(full)) > big
    c1 = ONE_LAYER["retention_rotated_prefix_two_column_blocks"]
    w1 = M.draw_weights(c1, 5, sharp=True)
    t1 = tokens_for(c1, 400, 9)
    a, b = plain_logits(c1, w1, t1)[-5:], plain_logits(c1, w1, t1[200:])[-5:]
    assert np.max(np.abs(a - b)) / np.max(np.abs(a)) > 10 * TOL_SHARP["float32"]


@pytest.mark.parametrize("dtype", DTYPES)
def test_first_tokens_and_short_sequences(tmp_path_factory, dtype):
    """Single-token prompts and a first step of one token beside longer ones in the same batch; then each grows token
    by token."""
    from rustingstrata_b200.engine import StepEntry
    path, cfg, w = model_for(tmp_path_factory, dtype, "R", "R", seed=11)
    r = runner_for(path, dtype, page_size=16, pool_tokens=256)
    seqs = {"one": tokens_for(cfg, 1, 1), "two": tokens_for(cfg, 2, 2), "three": tokens_for(cfg, 3, 3), "ten": tokens_for(cfg, 10, 4)}
    out = r.step([StepEntry(k, t, list(range(len(t)))) for k, t in seqs.items()]).cpu().numpy()
    r.check_status()
    at = 0
    for k, t in seqs.items():
        assert rel_err(out[at:at + len(t)], plain_logits(cfg, w, t)) <= TOL[dtype], k
        at += len(t)
    for _ in range(4):
        for k in seqs:
            seqs[k] = seqs[k] + tokens_for(cfg, 1, len(seqs[k]) + 50)
        out = r.step([StepEntry(k, t[-1:], [0]) for k, t in seqs.items()]).cpu().numpy()
        for row, (k, t) in zip(out, seqs.items()):
            assert rel_err(row, plain_logits(cfg, w, t)[-1]) <= TOL[dtype], k


@pytest.mark.parametrize("dtype", DTYPES)
def test_long_decoding(tmp_path_factory, dtype):
    """300 tokens one by one after a short prompt (replayed graphs, pages taken and given back as it goes, states that
    last, many blocks and a window that passes over decoded tokens only)."""
    path, cfg, w = model_for(tmp_path_factory, dtype, "P_sharp", "P", seed=21, sharp=True)
    toks = tokens_for(cfg, 320, 8)
    ref = plain_logits(cfg, w, toks)
    r = runner_for(path, dtype, page_size=8, pool_tokens=384)
    got = [step_all(r, "a", toks[:20])] + [step_all(r, "a", [t]) for t in toks[20:]]
    err = np.max(np.abs(np.concatenate(got) - ref), axis=1) / np.max(np.abs(ref))
    print(f"long decoding {dtype}: worst {err.max():.3e}")
    assert_rows_within(err, TOL_SHARP[dtype], "long decoding")


WIDE = {
    # 20 query heads over 5 kv heads with heads of 96 / 128, state heads of 128 x 128 and of 256 rows, a latent of 256,
    # 40 experts in 8 groups, 8 streams, widths that reach the 128 x 128 tiles of the tensor-core products
    "wide_heads": M.config(500, 512, [
        (M.attention(20, 5, 96, 128, rot=(32, 1e5), chunk=192), M.dense(1024)),
        (M.retention(4, 128, 128, (0.9, 0.99, 0.995, 0.999), rot=(128, 1e4)), M.moe(40, 4, 64, scale=2.5, groups=(8, 3), shared=256)),
        (M.latent(8, 64, 64, 256, window=300), M.dense(512)),
        (M.retention(2, 256, 64, (0.98, 0.96), rot=(64, 1e6)), None)], eps=1e-5, streams=8),
    # many small heads, state heads wider than they are tall, shared layers
    "many_heads": M.config(300, 256, [
        (M.retention(16, 16, 96, tuple(1 - 2.0 ** -(3 + i % 6) for i in range(16)), rot=(16, 1e4)), M.dense(384)),
        (M.attention(16, 16, 16, 16, rot=(16, 1e4), chunk=64), None),
        (M.latent(16, 16, 16, 48, window=50), M.moe(16, 8, 32, scale=1.0, groups=(2, 2))), 1, 0], streams=2),
}


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", sorted(WIDE))
def test_wider_shapes_and_long_portions(tmp_path_factory, name, dtype):
    """A portion of 500 tokens, 30 single tokens, a portion of 110: the forms of the kernels that only large steps and
    wide heads reach."""
    path, cfg, w = model_for(tmp_path_factory, dtype, "wide_" + name, WIDE[name], seed=7)
    toks = tokens_for(cfg, 640, 3)
    ref = plain_logits(cfg, w, toks)
    r = runner_for(path, dtype, page_size=16, pool_tokens=768, max_batch_tokens=768)
    got = [step_all(r, "a", toks[:500])] + [step_all(r, "a", [t]) for t in toks[500:530]] + [step_all(r, "a", toks[530:])]
    err = np.max(np.abs(np.concatenate(got) - ref), axis=1) / np.max(np.abs(ref))
    print(f"wide {name} {dtype}: worst {err.max():.3e}")
    assert err.max() <= TOL[dtype], f"first wrong position {int(np.argmax(err > TOL[dtype]))}"


# ----------------------------------------------------------------------------- kernels against torch
def test_router_choice_in_groups_against_torch():
    """The router kernel with sigmoid scores, groups and a scale, against the same rule written with torch.topk."""
    from rustingstrata_b200.kernels import ops
    g = torch.Generator().manual_seed(3)
    for E, top, groups, keep, scale in [(12, 3, 4, 2, 2.0), (8, 3, 2, 1, 0.5), (64, 6, 8, 4, 1.0), (6, 2, 6, 3, 1.5), (40, 1, 0, 0, 3.0)]:
        T = 70
        logits = torch.randn(T, E, generator=g) * 2
        corr = torch.randn(E, generator=g) * 0.3
        s = torch.sigmoid(logits.double())
        pick = s + corr.double()
        if groups:
            per = pick.view(T, groups, E // groups)
            worth = per.topk(min(2, E // groups), dim=-1).values.sum(-1)
            best = worth.topk(keep, dim=-1).indices
            ok = torch.zeros(T, groups, dtype=torch.bool).scatter_(1, best, True).repeat_interleave(E // groups, dim=1)
            pick = pick.masked_fill(~ok, -float("inf"))
        want = pick.topk(top, dim=-1).indices
        choice = torch.empty(T * top, dtype=torch.int32, device="cuda")
        weights = torch.empty(T * top, dtype=torch.float32, device="cuda")
        status = torch.zeros(1, dtype=torch.int32, device="cuda")
        ops.router_topk(logits.cuda(), corr.cuda(), top, T, choice, weights, status, sigmoid=True, groups=groups, keep=keep,
                        scale=scale, renormalize=False)
        assert int(status.item()) == 0
        got = choice.view(T, top).cpu().long()
        assert torch.equal(got.sort(dim=1).values, want.sort(dim=1).values), (E, top, groups, keep)
        assert torch.allclose(weights.view(T, top).cpu().double(), s.gather(1, got) * scale, rtol=1e-5, atol=1e-6)


# ----------------------------------------------------------------------------- the engine's own entry points
@pytest.mark.parametrize("chunk", [None, 7])
def test_greedy_generation_through_the_scheduler(tmp_path_factory, chunk):
    """Engine.generate (scheduler, admission, prompt portions of 7 tokens, decode steps launched ahead) gives the plain
    implementation's greedy tokens in 32-bit, for several prompts of unequal length at once."""
    from rustingstrata_b200 import Engine
    path, cfg, w = model(tmp_path_factory, "P", "P", seed=11)
    prompts = [tokens_for(cfg, n, 60 + n) for n in (5, 23, 1, 40)]
    want = []
    for p in prompts:
        seq = list(p)
        for _ in range(12):
            seq.append(int(np.argmax(plain_logits(cfg, w, seq)[-1])))
        want.append(seq[len(p):])
    eng = Engine(path, dtype="float32", page_size=8, max_tokens=512, max_batch_tokens=64, max_seqs=4, prefill_chunk=chunk)
    assert eng.generate(prompts, max_new_tokens=12) == want
    # and once more through the same engine: slots and pages of the finished requests are taken again
    assert eng.generate(prompts[::-1], max_new_tokens=12) == want[::-1]


def test_bfloat16_generation_picks_top_tokens(tmp_path_factory):
    from rustingstrata_b200 import Engine
    path, cfg, w = model(tmp_path_factory, "R_steady", "R", seed=11, steady=True)
    prompt = tokens_for(cfg, 30, 2)
    eng = Engine(path, dtype="bfloat16", page_size=16, max_tokens=256, max_batch_tokens=64, max_seqs=2)
    got = eng.generate(prompt, max_new_tokens=10)
    logits = plain_logits(cfg, w, prompt + got)
    for i, t in enumerate(got):
        row = logits[len(prompt) - 1 + i]
        assert row[t] >= row.max() - 0.08 * np.abs(logits).max()


def read_model_folder(folder):
    """A safetensors file read by hand: name → float64 tensor."""
    import struct
    with open(os.path.join(folder, "model.safetensors"), "rb") as f:
        n = struct.unpack("<Q", f.read(8))[0]
        header = json.loads(f.read(n))
        blob = f.read()
    out = {}
    for name, ent in header.items():
        if name == "__metadata__":
            continue
        lo, hi = ent["data_offsets"]
        bits = np.frombuffer(blob[lo:hi], dtype=np.uint16).astype(np.uint32) << 16
        out[name] = torch.from_numpy(bits.view(np.float32).astype(np.float64)).reshape(ent["shape"])
    return out


def test_trace_replay_and_command_line(tmp_path_factory, tmp_path):
    """bin/trace_run on a model folder (logits of a request cut in two steps beside a second request), and
    ``init-random`` + ``generate`` of the package's command line for this architecture."""
    path, cfg, w = model(tmp_path_factory, "Q", "Q", seed=11)
    toks = tokens_for(cfg, 40, 1)
    steps = [{"step": 0, "entries": [{"id": "x", "tokens": toks[:25], "want": [0, 24]}], "end": []},
             {"step": 1, "entries": [{"id": "x", "tokens": toks[25:], "want": [14]}, {"id": "y", "tokens": toks[:3], "want": [2]}],
              "end": ["x", "y"]}]
    out = tmp_path / "out"
    res = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", path, "--dtype", "float32",
                          "--out", str(out), "--max-tokens", "128"], input="".join(json.dumps(s) + "\n" for s in steps),
                         capture_output=True, text=True, timeout=600)
    assert res.returncode == 0, res.stderr[-2000:]
    assert [ln for ln in res.stdout.splitlines() if ln.startswith("done")] == ["done 0", "done 1"]
    ref = plain_logits(cfg, w, toks)
    a = np.fromfile(out / "0.f32", dtype="<f4").reshape(2, cfg["vocab"])
    b = np.fromfile(out / "1.f32", dtype="<f4").reshape(2, cfg["vocab"])
    assert rel_err(a, ref[[0, 24]]) <= TOL["float32"] and rel_err(b, ref[[39, 2]]) <= TOL["float32"]
    cfg_path = tmp_path / "config.json"
    cfg_path.write_text(json.dumps(M.CONFIGS["P"]))
    made = tmp_path / "made"
    cli = [sys.executable, "-m", "rustingstrata_b200"]
    env = dict(os.environ, PYTHONPATH=ROOT)
    r1 = subprocess.run(cli + ["init-random", "--config", str(cfg_path), "--out", str(made), "--seed", "3"],
                        capture_output=True, text=True, timeout=600, env=env)
    assert r1.returncode == 0, r1.stderr[-2000:]
    r2 = subprocess.run(cli + ["generate", "--model", str(made), "--prompt", "1,2,3,4", "-n", "6", "--dtype", "float32"],
                        capture_output=True, text=True, timeout=600, env=env)
    assert r2.returncode == 0, r2.stderr[-2000:]
    # the folder it wrote, read by this file's own reader, generates the same tokens in the plain implementation
    w2 = read_model_folder(str(made))
    seq = [1, 2, 3, 4]
    for _ in range(6):
        seq.append(int(np.argmax(plain_logits(M.CONFIGS["P"], w2, seq)[-1])))
    assert ",".join(str(t) for t in seq[4:]) in r2.stdout.replace(" ", "") or " ".join(str(t) for t in seq[4:]) in r2.stdout, r2.stdout

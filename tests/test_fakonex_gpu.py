"""Fakonex on the GPU against the float64 oracle (tests/fakonex_oracle.py): small made-up configurations with random or
hand-made weights.  Covered: each mechanism alone, the residual stream layer by layer, prefill against token-by-token decoding,
portions down to two tokens, unequal batches, reuse of pages and slots, keys far back / at page borders / just inside and just
outside a chunk, the sink's share, the first tokens, long decoding, other sizes, the tensor-core paths, a model folder, and
greedy generation through the scheduler."""
import json

import numpy as np
import pytest

from distributed_inference_server_b200 import ContinuousBatcher, InferenceParams, models
from tests import _fakonex_util as U
from tests import fakonex_oracle as FO

pytestmark = pytest.mark.gpu
F32_TOL = 2e-5


def toks(n, vocab=50, seed=0):
    return [int(x) for x in np.random.default_rng(seed).integers(0, vocab, n)]


MECHANISMS = {
    "attention_no_mask": dict(layers=[(U.attention(chunk=0), None)]),
    "attention_chunks_of_five": dict(layers=[(U.attention(chunk=5), None)]),
    "attention_chunk_of_one": dict(layers=[(U.attention(chunk=1), None)]),
    "attention_one_kv_head": dict(layers=[(U.attention(heads=3, kv_heads=1, dim=6, vdim=6, chunk=17), None)]),
    "attention_as_many_kv_heads": dict(layers=[(U.attention(heads=2, kv_heads=2, dim=10, vdim=4, chunk=64), None)]),
    "borrowed_keys_and_values": dict(layers=[(U.attention(chunk=9), None), (U.attention(chunk=30, kv_from=0), None)]),
    "experts_without_groups_or_shared": dict(layers=[(U.attention(), U.moe(groups=None, shared=0))]),
    "experts_one_per_token": dict(layers=[(U.attention(), U.moe(experts=5, top=1, groups=None, shared=0))]),
    "experts_all_of_the_kept_groups": dict(layers=[(U.attention(), U.moe(experts=8, top=4, groups=(4, 2), shared=0))]),
    "experts_one_group_kept": dict(layers=[(U.attention(), U.moe(experts=10, top=4, groups=(2, 1), shared=0))]),
    "experts_groups_of_one": dict(layers=[(U.attention(), U.moe(experts=4, top=2, groups=(4, 3), shared=0))]),
    "experts_every_group_kept": dict(layers=[(U.attention(), U.moe(experts=6, top=3, groups=(3, 3), shared=0))]),
    "shared_expert": dict(layers=[(U.attention(), U.moe(experts=2, top=1, groups=None, shared=20))]),
    "no_soft_cap": dict(layers=[(U.attention(), U.moe())], softcap=0),
    "tight_soft_cap": dict(layers=[(U.attention(), U.moe())], softcap=0.7),
}


@pytest.mark.parametrize("name", sorted(MECHANISMS))
def test_each_mechanism_alone(name):
    cfg = U.config(**MECHANISMS[name])
    W = U.weights(cfg, seed=3)
    t = toks(70, seed=1)
    want = U.oracle_logits(cfg, W, t)
    assert U.rel_err(U.run_whole(cfg, W, t), want) < F32_TOL
    assert U.bf16_close(U.run_whole(cfg, W, t, dtype="bfloat16"), want)


def test_router_choice_with_decisive_scores():
    """Router rows that make the scores of single experts stand out: the correction moves the choice but not the weights, a
    group is ranked by its two best members, and an expert outside the kept groups is never taken however good it is."""
    cfg = U.config([(U.attention(), U.moe(experts=6, top=2, groups=(3, 1), shared=0))], width=16)
    W = U.weights(cfg, seed=5)
    t = toks(40, seed=2)
    # expert 0 alone is excellent, but its group (0, 1) loses to group (4, 5) whose two members are both good
    W["l0.mlp.router"] = np.zeros((6, 16), np.float32)
    W["l0.mlp.correction"] = np.asarray([3.0, -3.0, -1.0, -1.0, 1.0, 0.75], np.float32)
    base = U.oracle_logits(cfg, W, t)
    assert U.rel_err(U.run_whole(cfg, W, t), base) < F32_TOL
    assert FO.choose_experts(FO.sigmoid(np.zeros(6)), W["l0.mlp.correction"], 2, (3, 1)) == [4, 5]
    # with every group kept the excellent expert is taken: the group limit is what kept it out
    cfg2 = U.config([(U.attention(), U.moe(experts=6, top=2, groups=(3, 3), shared=0))], width=16)
    other = U.oracle_logits(cfg2, W, t)
    assert U.rel_err(other, base) > 1e-3
    assert U.rel_err(U.run_whole(cfg2, W, t), other) < F32_TOL
    # a correction so negative that the choice scores of the kept group are below zero: still chosen (the others are out, not 0)
    W["l0.mlp.correction"] = np.asarray([-5.0, -6.0, -9.0, -9.0, -9.0, -9.5], np.float32)
    neg = U.oracle_logits(cfg, W, t)
    assert FO.choose_experts(FO.sigmoid(np.zeros(6)), W["l0.mlp.correction"], 2, (3, 1)) == [0, 1]
    assert U.rel_err(U.run_whole(cfg, W, t), neg) < F32_TOL


STACK = [(U.attention(), U.moe()), (U.attention(heads=6, kv_heads=3, dim=10, vdim=6, chunk=7), U.moe(experts=4, top=3, groups=(2, 2), shared=0)),
         (U.attention(chunk=40, kv_from=0), None), (U.attention(heads=6, kv_heads=3, dim=10, vdim=6, chunk=0, kv_from=1), U.moe(experts=3, top=1, groups=None)),
         (U.attention(heads=2, kv_heads=1, dim=12, vdim=8, chunk=16), U.moe(experts=9, top=2, groups=(3, 1), shared=6))]


def test_residual_stream_after_every_layer_matches():
    """Models cut after each layer reproduce the oracle layer by layer."""
    t = toks(45, seed=2)
    for n in range(1, len(STACK) + 1):
        cfg = U.config(STACK[:n])
        W = U.weights(cfg, seed=5)
        assert U.rel_err(U.run_whole(cfg, W, t), U.oracle_logits(cfg, W, t)) < F32_TOL, n


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_prefill_against_token_by_token_decoding(dtype):
    cfg = U.config(STACK)
    W = U.weights(cfg, seed=7)
    t = toks(60, seed=3)
    want = U.oracle_logits(cfg, W, t)
    whole = U.run_whole(cfg, W, t, dtype)
    single = U.run_portions(cfg, W, t, [], dtype)
    if dtype == "float32":
        assert U.rel_err(whole, want) < F32_TOL and U.rel_err(single, want) < F32_TOL
    else:
        assert U.bf16_close(whole, want) and U.bf16_close(single, want)
        assert U.bf16_close(whole, single, tol=6e-2)


@pytest.mark.parametrize("sizes", [[2, 2, 2, 3, 2], [5, 1, 17, 2, 40], [64, 2, 63], [1, 70, 2], [33, 33, 33, 33], [23, 2, 24, 25, 47]])
def test_portions_of_several_sizes(sizes):
    """Portions cut anywhere: inside a page (8 tokens), a chunk of the mask (7, 16, 24, 40) and a key tile (32)."""
    cfg = U.config(STACK)
    W = U.weights(cfg, seed=11)
    t = toks(140, seed=4)
    want = U.oracle_logits(cfg, W, t)
    assert U.rel_err(U.run_portions(cfg, W, t, sizes), want) < F32_TOL
    assert U.bf16_close(U.run_portions(cfg, W, t, sizes, "bfloat16"), want)


TENSOR_CORE_SHAPES = {
    # bfloat16 with dim % 8 == 0 and vdim % 16 == 0 runs attention on the tensor cores; the float32 run of the same model takes the
    # fp32-arithmetic kernel
    "dim8_vdim16_chunk100": [(U.attention(heads=4, kv_heads=4, dim=8, vdim=16, chunk=100), None)],
    "dim24_vdim32_six_per_group_chunk64": [(U.attention(heads=6, kv_heads=1, dim=24, vdim=32, chunk=64), None)],
    "dim72_vdim80_no_mask": [(U.attention(heads=2, kv_heads=1, dim=72, vdim=80, chunk=0), None)],
    "dim128_vdim128_chunk_257_borrowed": [(U.attention(heads=8, kv_heads=2, dim=128, vdim=128, chunk=257), None),
                                           (U.attention(heads=8, kv_heads=2, dim=128, vdim=128, chunk=33, kv_from=0), None)],
    "seventy_per_group_chunk300": [(U.attention(heads=70, kv_heads=1, dim=16, vdim=16, chunk=300), None)],
}


@pytest.mark.parametrize("name", sorted(TENSOR_CORE_SHAPES))
def test_attention_on_tensor_cores(name):
    """Whole prompt, ragged portions (blocks that end inside a key tile or a chunk) and decoding over a sliced history."""
    cfg = U.config(TENSOR_CORE_SHAPES[name], width=40)
    W = U.weights(cfg, seed=21)
    t = toks(330, seed=7)
    want = U.oracle_logits(cfg, W, t)
    assert U.rel_err(U.run_portions(cfg, W, t, [100, 3, 150, 64], page_size=16), want) < F32_TOL
    e16 = U.row_errs(U.run_whole(cfg, W, t, "bfloat16", page_size=16), want)
    assert float(np.quantile(e16, 0.8)) < 3e-2 and float(e16.max()) < 0.3
    e16 = U.row_errs(U.run_portions(cfg, W, t, [100, 3, 150, 64], "bfloat16", page_size=16), want)
    assert float(np.quantile(e16, 0.8)) < 3e-2 and float(e16.max()) < 0.3


def test_attention_over_slices_of_the_history():
    """A single decoding sequence with a long visible history has its keys cut into slices that a second kernel merges (the
    sink must count once, in one slice).  A layer without a mask slices the whole history, one with long chunks its own chunk,
    one with short chunks not at all -- all in one model, in prompts and in decoding, in both compute types."""
    cfg = U.config([(U.attention(dim=16, vdim=16, chunk=0), None), (U.attention(dim=16, vdim=16, chunk=300), U.moe()),
                    (U.attention(dim=16, vdim=16, chunk=48, kv_from=0), None)])
    W = U.weights(cfg, seed=15)
    t = toks(700, seed=6)
    want = U.oracle_logits(cfg, W, t)
    for dtype in ("float32", "bfloat16"):
        e = U.engine(cfg, W, dtype, pool_tokens=768, page_size=64)
        f = U.Feeder(e)
        f.step([("a", t, 290)])
        f.step([("a", t, 5)])      # one query block, 295 keys: slices
        f.step([("a", t, 340)])
        for _ in range(65):
            f.step([("a", t, 1)])
        got = f.end("a")
        e.close()
        assert U.rel_err(got, want) < F32_TOL if dtype == "float32" else U.bf16_close(got, want)


def test_large_passes_take_the_tensor_core_expert_products(monkeypatch):
    """A pass of 1280 prompt tokens in bfloat16: per-expert tensor-core products over rows sorted by expert, the shared
    expert's gate-up product with the SiLU epilogue.  Against the oracle, and against the same pass on the tiled fp32-FMA
    products (DIS_STACK_TC=0), which round the same operands."""
    cfg = U.config([(U.attention(heads=4, kv_heads=2, dim=16, vdim=16, chunk=96), U.moe(experts=4, top=2, ff=64, groups=(2, 1), shared=128))],
                   width=64, vocab=64)
    W = U.weights(cfg, seed=27)
    seqs = [toks(320, vocab=64, seed=80 + i) for i in range(4)]
    want = np.concatenate([U.oracle_logits(cfg, W, sq)[[5, 200, 319]] for sq in seqs])
    res = []
    for flag in ("1", "0"):
        monkeypatch.setenv("DIS_STACK_TC", flag)
        e = U.engine(cfg, W, "bfloat16", max_batch=4, pool_tokens=4 * 384, page_size=64, max_step_tokens=4 * 320, rows=64)
        P = InferenceParams(max_tokens=1 << 20, temperature=0.0)
        slots = [e.seq_add(sq, P) for sq in seqs]
        for sl in slots:
            e.seq_probe(sl, [5, 200])
        e.step(slots)
        res.append(e.last_logits(e.last_logit_rows()).copy())
        e.close()
    assert res[0].shape == (4 * 3, 64)
    assert U.bf16_close(res[0], want) and U.bf16_close(res[1], want)
    assert U.bf16_close(res[0], res[1], tol=3e-2)


def test_batches_of_unequal_requests_against_each_alone():
    cfg = U.config(STACK)
    W = U.weights(cfg, seed=13)
    seqs = {k: toks(n, seed=20 + i) for i, (k, n) in enumerate([("a", 90), ("b", 33), ("c", 7), ("d", 58)])}
    want = {k: U.oracle_logits(cfg, W, v) for k, v in seqs.items()}
    e = U.engine(cfg, W, max_batch=4, pool_tokens=512)
    f = U.Feeder(e)
    f.step([("a", seqs["a"], 50), ("b", seqs["b"], 2)])
    f.step([("a", seqs["a"], 1), ("b", seqs["b"], 20), ("c", seqs["c"], 7)])
    f.step([("d", seqs["d"], 30), ("a", seqs["a"], 1), ("b", seqs["b"], 1)])
    while any(f.fed[k] < len(seqs[k]) for k in seqs):
        f.step([(k, seqs[k], min(3 if k == "d" else 1, len(seqs[k]) - f.fed[k])) for k in seqs if f.fed[k] < len(seqs[k])])
    for k in seqs:
        assert U.rel_err(f.end(k), want[k]) < F32_TOL, k
    e.close()


def test_pages_and_slots_are_freed_and_used_again():
    """Two slots and a pool of 12 pages: six sequences pass through them; the cached keys and values of the sequence before
    (also those a later layer borrows) must not reach the next one."""
    cfg = U.config(STACK)
    W = U.weights(cfg, seed=17)
    e = U.engine(cfg, W, max_batch=2, pool_tokens=96, page_size=8)
    f = U.Feeder(e)
    lens = [40, 17, 48, 9, 33, 41]
    seqs = [toks(n, seed=40 + i) for i, n in enumerate(lens)]
    live = []
    for i, s in enumerate(seqs):
        if len(live) == 2:
            k = live.pop(0)
            while f.fed[k] < len(seqs[k]):
                f.step([(k, seqs[k], 1)] + [(o, seqs[o], 1) for o in live if f.fed[o] < len(seqs[o])])
            assert U.rel_err(f.end(k), U.oracle_logits(cfg, W, seqs[k])) < F32_TOL, k
        f.step([(i, s, len(s) - 5)] + [(o, seqs[o], 1) for o in live if f.fed[o] < len(seqs[o])])
        live.append(i)
    for k in live:
        while f.fed[k] < len(seqs[k]):
            f.step([(k, seqs[k], 1)])
        assert U.rel_err(f.end(k), U.oracle_logits(cfg, W, seqs[k])) < F32_TOL, k
    assert e.status().kv_pages_free == e.status().kv_pages_total
    e.close()


@pytest.mark.parametrize("decode_tail", [0, 40])
def test_far_keys_and_page_borders_with_peaked_weights(decode_tail):
    """A large score scale makes every query put its weight on one key (or on the sink), wherever in its chunk the key lies: a
    key that is lost, shifted by one or read from the wrong page changes the output by its full size."""
    cfg = U.config([(U.attention(scale=6.0, chunk=0), None), (U.attention(scale=5.0, chunk=130), None)])
    W = U.weights(cfg, seed=19, gain=2.0)
    t = toks(300, seed=6)
    want = U.oracle_logits(cfg, W, t)
    e = U.engine(cfg, W, pool_tokens=320, page_size=16)
    f = U.Feeder(e)
    f.step([("a", t, 300 - decode_tail)])
    for _ in range(decode_tail):
        f.step([("a", t, 1)])
    got = f.end("a")
    e.close()
    assert U.rel_err(got, want) < 1e-4


def _feed(e, t, cuts):
    """One sequence through a live engine: portions of the given sizes, the rest token by token; its logits; its slot and pages
    go back to the engine."""
    f = U.Feeder(e)
    fed = 0
    for n in cuts:
        n = min(n, len(t) - fed)
        if n > 0:
            f.step([("a", t, n)])
            fed += n
    while fed < len(t):
        f.step([("a", t, 1)])
        fed += 1
    return f.end("a")


def _planted(n, chunk, sink=0.0, heads=1):
    """Hand-made weights for one layer of width n with one-hot token embeddings (an RMS norm keeps a one-hot row's direction):
    the query of token 2 points, in every head, at the key of token 1 and at nothing else; every other token's query is zero.
    `sink` is the first head's; further heads have none to speak of."""
    cfg = U.config([(U.attention(heads=heads, kv_heads=1, dim=n, vdim=n, scale=1.0, chunk=chunk), None)], vocab=n, width=n, softcap=0)
    W = U.weights(cfg, seed=23)
    eye = np.eye(n, dtype=np.float32)
    W["embed"] = eye.copy()
    W["l0.norm1"] = np.ones(n, np.float32)
    q = np.zeros((heads * n, n), np.float32)
    q[1::n, 2] = 1.0
    W["l0.mix.q"], W["l0.mix.k"], W["l0.mix.v"] = q, eye.copy(), eye.copy()
    for b in ("q.b", "k.b", "v.b"):
        W["l0.mix." + b] = np.zeros_like(W["l0.mix." + b])
    # unit-rms queries and keys: the planted pair scores 3 n, every other pair 0
    W["l0.mix.q.norm"], W["l0.mix.k.norm"] = np.full(n, 3.0, np.float32), np.ones(n, np.float32)
    W["l0.mix.sink"] = np.asarray([sink] + [-30.0] * (heads - 1), np.float32)
    W["l0.mix.g"] = np.zeros((heads, n), np.float32)
    return cfg, W


@pytest.mark.parametrize("n,dtype", [(8, "float32"), (16, "bfloat16")])
def test_a_key_planted_far_back_is_found(n, dtype):
    """Token 1 occurs once among 260 tokens of one chunk; the last token (2) looks for it and finds nearly all of its weight
    there, wherever it stands: next to a page border on either side, at the very start, or just before the query."""
    cfg, W = _planted(n, chunk=512)
    base = [int(x) for x in np.random.default_rng(1).integers(3, n, 260)]
    base[-1] = 2
    without = U.oracle_logits(cfg, W, base)[-1]
    e = U.engine(cfg, W, dtype, pool_tokens=320, page_size=64)
    for where in (0, 31, 32, 63, 64, 127, 128, 191, 192, 258):
        t = list(base)
        t[where] = 1
        want = U.oracle_logits(cfg, W, t)
        assert np.abs(want[-1] - without).max() > 0.05  # the planted key decides the output
        for tail in (0, 3):  # the query inside a prompt portion, and decoded alone
            assert U.rel_err(_feed(e, t, [260 - tail]), want) < (1e-4 if dtype == "float32" else 2e-2), (where, tail)
    e.close()


@pytest.mark.parametrize("n,dtype", [(8, "float32"), (16, "bfloat16")])
@pytest.mark.parametrize("chunk", [100, 64, 37])
def test_keys_just_inside_and_just_outside_a_chunk(n, dtype, chunk):
    """The query (last token) sits in the chunk that starts at `lo`.  A planted key at lo or lo + 1 is seen, one at lo - 1 or
    lo - 2 is not -- the output is then exactly that of the sequence without it -- also when the query is the first token of
    its chunk, when the prompt was cut right at the edge, and when the query is decoded alone."""
    cfg, W = _planted(n, chunk)
    e = U.engine(cfg, W, dtype, pool_tokens=448, page_size=16)
    for length in (2 * chunk + 31, 3 * chunk + 1, 2 * chunk + 2):
        lo = (length - 1) // chunk * chunk
        base = [int(x) for x in np.random.default_rng(2).integers(3, n, length)]
        base[-1] = 2
        without = U.oracle_logits(cfg, W, base)
        for where in (lo - 2, lo - 1, lo, lo + 1):
            if where >= length - 1:
                continue
            t = list(base)
            t[where] = 1
            want = U.oracle_logits(cfg, W, t)
            if where >= lo:
                assert np.abs(want[-1] - without[-1]).max() > 0.05
            else:
                assert np.abs(want[-1] - without[-1]).max() == 0.0
            for cuts in ([length], [lo, length - lo], [lo - 1, 2, length], [length - 1, 1], [lo + 1, length]):
                assert U.rel_err(_feed(e, t, cuts), want) < (1e-4 if dtype == "float32" else 2e-2), (length, where, cuts)
    e.close()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_the_sink_takes_its_share(dtype):
    """With the planted key scoring 3 n, a sink logit of the same size halves the key's weight in its head, a much larger one
    leaves that head's output near zero, and a very negative one changes nothing; a second head without a sink keeps its output,
    so the sum changes direction (the norm behind the mixer would hide a mere change of size).  The engine follows the oracle
    through all three."""
    n = 16
    t = [int(x) for x in np.random.default_rng(3).integers(3, n, 90)]
    t[40], t[-1] = 1, 2
    outs = []
    for sink in (-30.0, 3.0 * n, 3.0 * n + 12.0):
        cfg, W = _planted(n, chunk=128, sink=sink, heads=2)
        want = U.oracle_logits(cfg, W, t)
        for cuts in ([90], [88, 1, 1]):
            got = U.run_portions(cfg, W, t, cuts, dtype, pool_tokens=128, page_size=16)
            assert U.rel_err(got, want) < (1e-4 if dtype == "float32" else 2e-2), (sink, cuts)
        outs.append(want[-1])
    assert np.abs(outs[0] - outs[1]).max() > 0.05 and np.abs(outs[1] - outs[2]).max() > 0.05


def test_output_gate_per_head():
    cfg = U.config([(U.attention(heads=4, kv_heads=2), None)])
    W = U.weights(cfg, seed=29)
    t = toks(30, seed=8)
    res = []
    for spread in (0.01, 0.5, 2.0):  # gates near one half, mixed, and mostly open or shut
        W["l0.mix.g"] = models.bf16_round(np.random.default_rng(5).normal(0, spread, (4, 32)).astype(np.float32))
        want = U.oracle_logits(cfg, W, t)
        assert U.rel_err(U.run_whole(cfg, W, t), want) < F32_TOL
        res.append(want)
    assert np.abs(res[0] - res[1]).max() > 1e-2 and np.abs(res[1] - res[2]).max() > 1e-2


def test_first_tokens_of_a_sequence():
    cfg = U.config(STACK)
    W = U.weights(cfg, seed=31)
    for n in (1, 2, 3, 5):
        t = toks(n, seed=50 + n)
        assert U.rel_err(U.run_whole(cfg, W, t), U.oracle_logits(cfg, W, t)) < F32_TOL, n
    t = toks(9, seed=60)
    assert U.rel_err(U.run_portions(cfg, W, t, [1, 1, 2, 1, 4]), U.oracle_logits(cfg, W, t)) < F32_TOL


def test_long_decoding_keeps_the_cache_exact():
    cfg = U.config([(U.attention(chunk=150), U.moe()), (U.attention(chunk=0, kv_from=0), None), (U.attention(chunk=64), U.moe(groups=None))])
    W = U.weights(cfg, seed=37)
    t = toks(420, seed=9)
    want = U.oracle_logits(cfg, W, t)
    e = U.engine(cfg, W, pool_tokens=448, page_size=64)
    f = U.Feeder(e)
    f.step([("a", t, 20)])
    for _ in range(400):
        f.step([("a", t, 1)])
    got = f.end("a")
    e.close()
    assert U.rel_err(got, want) < 5e-5


ODD = [(U.attention(heads=6, kv_heads=3, dim=10, vdim=14, chunk=11), U.moe(experts=12, top=5, ff=20, groups=(4, 2), shared=9)),
       (U.attention(heads=5, kv_heads=5, dim=6, vdim=8, chunk=3, scale=0.9), None),
       (U.attention(heads=1, kv_heads=1, dim=40, vdim=68, chunk=0), U.moe(experts=3, top=3, ff=36, groups=None, shared=0)),
       (U.attention(heads=9, kv_heads=3, dim=10, vdim=14, chunk=50, kv_from=0), U.moe(experts=10, top=1, ff=8, groups=(5, 1), shared=40)),
       (U.attention(heads=1, kv_heads=1, dim=40, vdim=68, chunk=20, kv_from=2), None)]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("width,vocab,softcap", [(72, 131, 30.0), (136, 61, 2.0), (50, 33, 0)])
def test_other_sizes(dtype, width, vocab, softcap):
    cfg = U.config(ODD, vocab=vocab, width=width, eps=1e-3, softcap=softcap)
    W = U.weights(cfg, seed=41)
    t = toks(75, vocab=vocab, seed=10)
    want = U.oracle_logits(cfg, W, t)
    got = U.run_portions(cfg, W, t, [33, 2, 1, 1, 30, 8], dtype, page_size=16, pool_tokens=128)
    assert U.rel_err(got, want) < F32_TOL if dtype == "float32" else U.bf16_close(got, want)


def test_model_folder_round_trip(tmp_path):
    """config.json + model.safetensors written by the test, read back through the registry, loaded and run."""
    from tests.test_stack_cpu import write_safetensors
    cfg = U.config(STACK)
    W = U.weights(cfg, seed=43)
    write_safetensors(tmp_path / "model.safetensors", W)
    (tmp_path / "config.json").write_text(json.dumps(cfg))
    assert models.read_config(str(tmp_path))[1].name == "Fakonex"
    t = toks(20, seed=12)
    e = models.load_model(str(tmp_path), dtype="float32", max_batch=2, max_tokens=64, page_size=16, max_step_tokens=64, max_logit_rows=68)
    f = U.Feeder(e)
    f.step([("a", t, 20)])
    got = f.end("a")
    e.close()
    assert U.rel_err(got, U.oracle_logits(cfg, W, t)) < F32_TOL


def test_greedy_generation_through_the_scheduler():
    """Requests of unequal length through the admission queue and the continuous batcher; greedy tokens equal the oracle's,
    except where the oracle's top two logits are closer than float32 noise."""
    cfg = U.config(STACK, vocab=40)
    W = U.weights(cfg, seed=43)
    e = U.engine(cfg, W, max_batch=3, pool_tokens=256, page_size=8, max_step_tokens=64)
    cb = ContinuousBatcher(e, max_active=3)
    cb.set_prefill_budget(16)  # prompts are read in portions beside the running sequences
    prompts = [toks(n, vocab=40, seed=70 + n) for n in (5, 37, 12, 1, 26)]
    new = [9, 6, 12, 7, 5]
    for i, p in enumerate(prompts):
        cb.submit(i, p, InferenceParams(new[i], 0.0))
    res = cb.run_until_idle()
    for i, p in enumerate(prompts):
        seq = list(p)
        got = res[i]["tokens"]
        assert len(got) == new[i]
        for j in range(new[i]):
            lg = U.oracle_logits(cfg, W, seq)[-1]
            top2 = np.sort(lg)[-2:]
            if int(np.argmax(lg)) != got[j]:
                assert top2[1] - top2[0] < 1e-4, (i, j)
            seq.append(got[j])
    cb.close()
    e.close()


def _random_model(rng):
    """A made-up configuration: one or two families of (kv heads, dim, vdim) so that later layers can borrow a cache, any chunk
    length, feed-forwards with and without groups, shared expert and soft cap."""
    width, vocab = int(rng.choice([48, 64, 96, 128, 200, 50])), int(rng.integers(40, 300))
    fams = [dict(kv_heads=int(rng.choice([1, 2, 3, 4])), dim=int(rng.choice([8, 16, 24, 32, 64, 12, 20])), vdim=int(rng.choice([16, 32, 64, 8, 24, 40])))
            for _ in range(int(rng.integers(1, 3)))]
    layers, owners = [], {}
    for i in range(int(rng.integers(2, 7))):
        f = int(rng.integers(0, len(fams)))
        kv_from = int(rng.choice(owners[f])) if f in owners and rng.random() < 0.5 else None
        if kv_from is None:
            owners.setdefault(f, []).append(i)
        mx = U.attention(heads=fams[f]["kv_heads"] * int(rng.choice([1, 2, 4])), kv_heads=fams[f]["kv_heads"], dim=fams[f]["dim"], vdim=fams[f]["vdim"],
                         chunk=int(rng.choice([0, 1, 7, 16, 33, 64, 100])), kv_from=kv_from)
        ml = None
        if rng.random() < 0.8:
            E = int(rng.choice([2, 3, 4, 6, 8, 12, 40]))
            groups, avail = None, E
            if rng.random() < 0.7:
                cnt = int(rng.choice([g for g in (1, 2, 3, 4, 6) if E % g == 0]))
                groups = (cnt, int(rng.integers(1, cnt + 1)))
                avail = E // cnt * groups[1]
            ml = U.moe(experts=E, top=int(rng.integers(1, min(avail, 6) + 1)), ff=int(rng.choice([8, 16, 24, 40])), groups=groups,
                       shared=int(rng.choice([0, 8, 24])))
        layers.append((mx, ml))
    return U.config(layers, vocab=vocab, width=width, eps=float(rng.choice([1e-5, 1e-3])), softcap=float(rng.choice([0, 5.0, 30.0])))


@pytest.mark.parametrize("seed", range(6))
def test_random_configurations_and_schedules(seed):
    """Up to four live requests, random portions beside single tokens, requests left out of a step, a pool that makes pages and
    slots go round: every position's logits against the oracle."""
    rng = np.random.default_rng(1000 + seed)
    cfg = _random_model(rng)
    W = U.weights(cfg, seed=seed)
    seqs = {k: toks(int(rng.choice([1, 2, 5, 23, 64, 65, 130, 200])), vocab=cfg["vocab"], seed=seed * 10 + k) for k in range(int(rng.integers(3, 7)))}
    want = {k: U.oracle_logits(cfg, W, v) for k, v in seqs.items()}
    page = int(rng.choice([8, 16, 64]))
    pool = sum((n + page - 1) // page * page for n in sorted((len(v) for v in seqs.values()), reverse=True)[:4]) + page
    e = U.engine(cfg, W, max_batch=4, pool_tokens=pool, page_size=page, max_step_tokens=pool)
    f = U.Feeder(e)
    waiting, live = list(seqs), []
    while waiting or live:
        while waiting and len(live) < 4:
            live.append(waiting.pop(0))
        step = []
        for k in live:
            rem = len(seqs[k]) - f.fed.get(k, 0)
            if rng.random() < 0.15 and len(live) > 1 and f.fed.get(k, 0) > 0:
                continue  # left out of this step
            r = rng.random()
            step.append((k, seqs[k], 1 if r < 0.4 else int(rng.integers(1, rem + 1)) if r < 0.8 else rem))
        if not step:
            continue
        f.step(step)
        for k, _, _ in step:
            if f.fed[k] == len(seqs[k]):
                assert U.rel_err(f.end(k), want[k]) < 5e-5, (seed, k)
                live.remove(k)
    assert e.status().kv_pages_free == e.status().kv_pages_total
    e.close()

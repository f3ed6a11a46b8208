"""Goperax on the GPU against the float64 oracle (tests/goperax_oracle.py): small made-up configurations with random or
hand-made weights.  Covered: each mechanism alone, the residual stream layer by layer, prefill against token-by-token decoding,
portions down to two tokens, unequal batches, reuse of pages and slots, keys far back / at page borders / just inside and just
outside a window, state carried from far back, the unit sink, the first tokens, long decoding, long spans through the segment
path of the recurrence, other sizes, the tensor-core paths, a model folder, and greedy generation through the scheduler."""
import json

import numpy as np
import pytest

from distributed_inference_server_b200 import ContinuousBatcher, InferenceParams, models
from tests import _goperax_util as U
from tests import goperax_oracle as GO

pytestmark = pytest.mark.gpu
F32_TOL = 2e-5


def toks(n, vocab=50, seed=0):
    return [int(x) for x in np.random.default_rng(seed).integers(0, vocab, n)]


MECHANISMS = {
    "attention_whole_past": dict(layers=[(U.attention(window=0), None)]),
    "attention_window_of_five": dict(layers=[(U.attention(window=5), None)]),
    "attention_window_of_one": dict(layers=[(U.attention(window=1), None)]),
    "attention_no_cap": dict(layers=[(U.attention(softcap=0), None)]),
    "attention_tight_cap": dict(layers=[(U.attention(softcap=0.3, scale=2.0), None)]),
    "attention_one_kv_head": dict(layers=[(U.attention(heads=3, kv_heads=1, dim=6, window=17), None)]),
    "attention_as_many_kv_heads": dict(layers=[(U.attention(heads=2, kv_heads=2, dim=10, window=64), None)]),
    "ssm_alone": dict(layers=[(U.ssm(), None)]),
    "ssm_one_group_one_norm_part": dict(layers=[(U.ssm(heads=3, vdim=5, state=7, groups=1, conv=4, norm_groups=1), None)]),
    "ssm_group_per_head_part_per_head": dict(layers=[(U.ssm(heads=4, vdim=4, state=6, groups=4, conv=2, norm_groups=4), None)]),
    "ssm_convolution_of_one_tap": dict(layers=[(U.ssm(conv=1), None)]),
    "ssm_convolution_of_seven_taps": dict(layers=[(U.ssm(conv=7), None)]),
    "dense_unit": dict(layers=[(U.attention(), U.dense(ff=36))]),
    "experts_without_shared": dict(layers=[(U.attention(), U.moe(shared=0))]),
    "experts_one_per_token": dict(layers=[(U.ssm(), U.moe(experts=5, top=1, shared=0))]),
    "experts_all_of_them": dict(layers=[(U.ssm(), U.moe(experts=3, top=3))]),
    "shared_unit": dict(layers=[(U.attention(), U.moe(experts=2, top=1, shared=20))]),
    "one_plain_residual": dict(layers=[(U.attention(), U.dense()), (U.ssm(), U.moe())], streams=0),
    "one_stream_with_coefficients": dict(layers=[(U.attention(), U.dense()), (U.ssm(), U.moe())], streams=1),
    "eight_streams": dict(layers=[(U.attention(), U.dense()), (U.ssm(), None)], streams=8),
    "loop_over_all": dict(layers=[(U.attention(), U.dense()), (U.ssm(), U.moe())], loop=(0, 2, 3)),
    "loop_once": dict(layers=[(U.attention(), None), (U.ssm(), U.dense()), (U.attention(window=9), None)], loop=(1, 2, 1)),
    "loop_to_the_last": dict(layers=[(U.ssm(), None), (U.attention(), U.dense())], loop=(1, 2, 2)),
}


@pytest.mark.parametrize("name", sorted(MECHANISMS))
def test_each_mechanism_alone(name):
    cfg = U.config(**MECHANISMS[name])
    W = U.weights(cfg, seed=3)
    t = toks(70, seed=1)
    want = U.oracle_logits(cfg, W, t)
    assert U.rel_err(U.run_whole(cfg, W, t), want) < F32_TOL
    assert U.bf16_close(U.run_whole(cfg, W, t, dtype="bfloat16"), want)


def test_router_with_decisive_scores():
    """Router rows that make single experts stand out for single tokens: with one-hot-like inputs the choice is known, and the
    chosen experts' weights are their softmax scores over the chosen sum -- not over all experts."""
    cfg = U.config([(U.attention(), U.moe(experts=4, top=2, shared=0))], width=16, vocab=16)
    W = U.weights(cfg, seed=5)
    W["l0.mlp.router"] = models.bf16_round(np.random.default_rng(1).normal(0, 1.5, (4, 16)).astype(np.float32))
    t = toks(40, vocab=16, seed=2)
    want = U.oracle_logits(cfg, W, t)
    assert U.rel_err(U.run_whole(cfg, W, t), want) < F32_TOL
    cfg3 = U.config([(U.attention(), U.moe(experts=4, top=3, shared=0))], width=16, vocab=16)
    assert U.rel_err(U.oracle_logits(cfg3, W, t), want) > 1e-3
    assert U.rel_err(U.run_whole(cfg3, W, t), U.oracle_logits(cfg3, W, t)) < F32_TOL


STACK = [(U.attention(), U.dense()), (U.ssm(), U.moe()), (U.attention(heads=6, kv_heads=3, dim=10, window=7, softcap=3.0), U.moe(experts=4, top=3, shared=0)),
         (U.ssm(heads=6, vdim=5, state=9, groups=3, conv=4, norm_groups=3), None), (U.attention(heads=2, kv_heads=1, dim=12, window=40), U.moe(experts=9, top=2, shared=6)),
         (U.ssm(heads=2, vdim=16, state=4, groups=1, conv=2, norm_groups=1), U.dense(ff=24))]
LOOP = (1, 4, 2)


def test_residual_stream_after_every_layer_matches():
    """Models cut after each layer (the loop unrolled by hand into separate layers that share their tensors' values) reproduce
    the oracle layer by layer."""
    t = toks(45, seed=2)
    order = GO.layer_order(U.config(STACK, loop=LOOP))
    full = U.weights(U.config(STACK), seed=5)
    for n in range(1, len(order) + 1):
        cfg = U.config([STACK[i] for i in order[:n]])
        W = {k: v for k, v in full.items() if not k.startswith("l")}
        for j, i in enumerate(order[:n]):
            W.update({f"l{j}." + k.split(".", 1)[1]: v for k, v in full.items() if k.startswith(f"l{i}.")})
        assert U.rel_err(U.run_whole(cfg, W, t), U.oracle_logits(cfg, W, t)) < F32_TOL, n
    # and the looped model is its unrolled form
    cfg = U.config(STACK, loop=LOOP)
    assert U.rel_err(U.run_whole(cfg, full, t), U.oracle_logits(U.config([STACK[i] for i in order]), W, t)) < F32_TOL


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_prefill_against_token_by_token_decoding(dtype):
    cfg = U.config(STACK, loop=LOOP)
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


@pytest.mark.parametrize("sizes", [[2, 2, 2, 3, 2], [5, 1, 17, 2, 40], [64, 2, 63], [1, 70, 2], [33, 33, 33, 33], [23, 2, 24, 25, 47], [129, 2]])
def test_portions_of_several_sizes(sizes):
    """Portions cut anywhere: inside a page (8 tokens), a window (7, 24, 40), a segment of the recurrence (64), the
    convolution's reach (2, 3, 4 taps) and a key tile (32)."""
    cfg = U.config(STACK, loop=LOOP)
    W = U.weights(cfg, seed=11)
    t = toks(140, seed=4)
    want = U.oracle_logits(cfg, W, t)
    assert U.rel_err(U.run_portions(cfg, W, t, sizes), want) < F32_TOL
    assert U.bf16_close(U.run_portions(cfg, W, t, sizes, "bfloat16"), want)


TENSOR_CORE_SHAPES = {
    # bfloat16 with dim % 16 == 0 runs attention on the tensor cores; the float32 run of the same model takes the fp32-arithmetic kernel
    "dim16_window100": [(U.attention(heads=4, kv_heads=4, dim=16, window=100), None)],
    "dim32_six_per_group_window64": [(U.attention(heads=6, kv_heads=1, dim=32, window=64), None)],
    "dim80_whole_past_no_cap": [(U.attention(heads=2, kv_heads=1, dim=80, window=0, softcap=0), None)],
    "dim128_window_257_then_33": [(U.attention(heads=8, kv_heads=2, dim=128, window=257), None), (U.attention(heads=8, kv_heads=2, dim=128, window=33), None)],
    "seventy_per_group_window300": [(U.attention(heads=70, kv_heads=1, dim=16, window=300), None)],
    "dim24_not_on_tensor_cores": [(U.attention(heads=4, kv_heads=2, dim=24, window=90), None)],
}


@pytest.mark.parametrize("name", sorted(TENSOR_CORE_SHAPES))
def test_attention_on_tensor_cores(name):
    """Whole prompt, ragged portions (blocks that end inside a key tile or a window) and decoding over a sliced history."""
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
    sink's 1 must count once, in one slice).  A layer without a window slices the whole history, one with a long window its
    window, one with a short window not at all -- all in one model, in prompts and in decoding, in both compute types."""
    cfg = U.config([(U.attention(dim=16, window=0), None), (U.attention(dim=16, window=300), U.moe()), (U.attention(dim=16, window=48), None)])
    W = U.weights(cfg, seed=15)
    t = toks(700, seed=6)
    want = U.oracle_logits(cfg, W, t)
    for dtype in ("float32", "bfloat16"):
        e = U.engine(cfg, W, dtype, pool_tokens=768, page_size=64)
        got = U.feed(e, t, [290, 5, 340])  # the portion of 5: one query block over 295 keys -- slices; then 65 decoded tokens
        e.close()
        assert U.rel_err(got, want) < F32_TOL if dtype == "float32" else U.bf16_close(got, want)


RECURRENCE_SHAPES = {  # (state, vdim): the register shapes of the recurrence kernel and its shared-memory form
    "state8_vdim40": (8, 40), "state48_vdim64": (48, 64), "state64_vdim96": (64, 96), "state128_vdim128": (128, 128), "state20_vdim136": (20, 136),
    "state130_vdim8": (130, 8), "state128_vdim64": (128, 64), "state100_vdim48": (100, 48),
}


@pytest.mark.parametrize("name", sorted(RECURRENCE_SHAPES))
def test_long_spans_through_the_segments_of_the_recurrence(name):
    """Spans longer than 64 tokens run as segments side by side joined by a carry; spans of 64 and fewer in one piece; both must
    agree with the token-by-token oracle, also when a span continues a state (the second portion) and in a batch of two."""
    N, P = RECURRENCE_SHAPES[name]
    cfg = U.config([(U.ssm(heads=2, vdim=P, state=N, groups=1, conv=3, norm_groups=2), None)], width=24)
    W = U.weights(cfg, seed=33)
    a, b = toks(200, seed=11), toks(150, seed=12)
    wa, wb = U.oracle_logits(cfg, W, a), U.oracle_logits(cfg, W, b)
    e = U.engine(cfg, W, pool_tokens=512, page_size=16, max_batch=2)
    f = U.Feeder(e)
    f.step([("a", a, 130), ("b", b, 20)])
    f.step([("a", a, 70), ("b", b, 129)])
    f.step([("b", b, 1)])
    assert U.rel_err(f.end("a"), wa) < 5e-5 and U.rel_err(f.end("b"), wb) < 5e-5
    e.close()


CONVOLUTION_SHAPES = {  # (heads, vdim, state, groups, taps): channels heads * vdim + 2 * groups * state
    "channels_multiple_of_four_taps4": (4, 8, 8, 2, 4), "channels_multiple_of_four_taps7": (2, 6, 6, 1, 7), "channels_odd_taps3": (3, 5, 7, 1, 3),
    "channels_even_taps2": (3, 6, 4, 1, 2), "over_a_thousand_channels_taps5": (8, 96, 80, 2, 5), "one_tap": (4, 8, 8, 2, 1),
}


@pytest.mark.parametrize("name", sorted(CONVOLUTION_SHAPES))
def test_convolution_tail_in_prompts_and_single_tokens(name):
    """The convolution reads four channels at a time where the layout allows it and one otherwise, and moves the slot's tail
    inside the same launch when every span of the pass is one token: prompts, single tokens and both in turn must agree, in a
    batch of two whose second sequence starts later (its first tokens see zeros, not the slot's earlier owner)."""
    H, P, N, G, taps = CONVOLUTION_SHAPES[name]
    cfg = U.config([(U.ssm(heads=H, vdim=P, state=N, groups=G, conv=taps, norm_groups=1), None), (U.ssm(heads=H, vdim=P, state=N, groups=G, conv=taps, norm_groups=H), U.dense())],
                   width=40, streams=2)
    W = U.weights(cfg, seed=5)
    a, b, c = toks(30, seed=21), toks(19, seed=22), toks(9, seed=23)
    wa, wb, wc = (U.oracle_logits(cfg, W, x) for x in (a, b, c))
    e = U.engine(cfg, W, pool_tokens=256, page_size=8, max_batch=2)
    f = U.Feeder(e)
    f.step([("a", a, 1)])
    f.step([("a", a, 1)])
    f.step([("a", a, 3), ("b", b, 1)])
    for _ in range(taps + 1):
        f.step([("a", a, 1), ("b", b, 1)])
    f.step([("a", a, 2), ("b", b, 18 - taps - 1)])
    assert U.rel_err(f.end("b"), wb) < F32_TOL
    f.step([("a", a, 1), ("c", c, 1)])  # c takes the slot that b gave back
    for _ in range(8):
        f.step([("a", a, 1), ("c", c, 1)])
    assert U.rel_err(f.end("c"), wc) < F32_TOL
    f.step([("a", a, 30 - f.fed["a"])])
    assert U.rel_err(f.end("a"), wa) < F32_TOL
    e.close()


@pytest.mark.parametrize("force", ["1", "2"])
def test_many_heads_and_sequences_walk_long_spans_whole(monkeypatch, force):
    """Four prompts of 100 tokens over 40 heads fill the GPU span by span, so the pass walks each span in one piece although
    it is longer than a segment; DIS_STACK_LIGHT_SEGMENTS=2 cuts it all the same.  Both agree with the oracle, and a second
    portion continues either."""
    monkeypatch.setenv("DIS_STACK_LIGHT_SEGMENTS", force)
    cfg = U.config([(U.ssm(heads=40, vdim=4, state=4, groups=5, conv=2, norm_groups=4), None)], width=24, streams=0)
    W = U.weights(cfg, seed=34)
    seqs = {k: toks(130, seed=50 + k) for k in range(4)}
    want = {k: U.oracle_logits(cfg, W, v) for k, v in seqs.items()}
    e = U.engine(cfg, W, pool_tokens=4 * 144, page_size=16, max_batch=4, max_step_tokens=400)
    f = U.Feeder(e)
    f.step([(k, seqs[k], 100) for k in seqs])
    f.step([(k, seqs[k], 30) for k in seqs])
    for k in seqs:
        assert U.rel_err(f.end(k), want[k]) < 5e-5
    e.close()


def test_large_passes_take_the_tensor_core_expert_products(monkeypatch):
    """A pass of 1280 prompt tokens in bfloat16: per-expert tensor-core products over rows sorted by expert and the shared unit
    on the tensor cores.  Against the oracle, and against the same pass on the tiled fp32-FMA products (DIS_STACK_TC=0), which
    round the same operands."""
    cfg = U.config([(U.attention(heads=4, kv_heads=2, dim=16, window=96), U.moe(experts=4, top=2, ff=64, shared=128)),
                    (U.ssm(heads=4, vdim=16, state=16, groups=2), U.dense(ff=192))], width=64, vocab=64)
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


def test_wide_dense_unit_in_a_prompt_pass_squares_the_relu_in_the_product(monkeypatch):
    """2048 prompt tokens through a dense unit of 4736 columns in bfloat16: enough tiles for the persistent tensor-core
    product, whose epilogue then writes relu(.)^2 in bfloat16 itself.  Against the oracle at a few positions, and against the
    same pass with that kernel switched off (DIS_STACK_PERSIST=0: product, then the activation kernel), which rounds the same
    operands and the same activations."""
    cfg = U.config([(U.ssm(heads=2, vdim=8, state=8, groups=1), U.dense(ff=4736)), (U.attention(heads=2, kv_heads=1, dim=16, window=40), U.dense(ff=4736))],
                   width=64, vocab=64, streams=2)
    W = U.weights(cfg, seed=29)
    seqs = [toks(512, vocab=64, seed=90 + i) for i in range(4)]
    want = np.concatenate([U.oracle_logits(cfg, W, sq[:131])[[7, 130]] for sq in seqs])
    res = []
    for flag in ("1", "0"):
        monkeypatch.setenv("DIS_STACK_PERSIST", flag)
        e = U.engine(cfg, W, "bfloat16", max_batch=4, pool_tokens=4 * 512, page_size=64, max_step_tokens=4 * 512, rows=64)
        P = InferenceParams(max_tokens=1 << 20, temperature=0.0)
        slots = [e.seq_add(sq, P) for sq in seqs]
        for sl in slots:
            e.seq_probe(sl, [7, 130, 300])
        e.step(slots)
        res.append(e.last_logits(e.last_logit_rows()).copy())
        e.close()
    assert res[0].shape == (4 * 4, 64)
    first_two = [4 * i + j for i in range(4) for j in (0, 1)]
    assert U.bf16_close(res[0][first_two], want) and U.bf16_close(res[1][first_two], want)
    assert U.bf16_close(res[0], res[1], tol=3e-2)


def test_batches_of_unequal_requests_against_each_alone():
    cfg = U.config(STACK, loop=LOOP)
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
    """Two slots and a pool of 12 pages: six sequences pass through them; neither the cached keys nor the recurrent state nor
    the convolution's tail of the sequence before may reach the next one."""
    cfg = U.config(STACK, loop=LOOP)
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
        # the newcomer starts with one token, two, or most of its prompt: the slot's old tail must not be read
        first = [1, 2, len(s) - 5][i % 3]
        f.step([(i, s, first)] + [(o, seqs[o], 1) for o in live if f.fed[o] < len(seqs[o])])
        live.append(i)
    for k in live:
        while f.fed[k] < len(seqs[k]):
            f.step([(k, seqs[k], 1)])
        assert U.rel_err(f.end(k), U.oracle_logits(cfg, W, seqs[k])) < F32_TOL, k
    assert e.status().kv_pages_free == e.status().kv_pages_total
    e.close()


@pytest.mark.parametrize("decode_tail", [0, 40])
def test_far_keys_and_page_borders_with_peaked_weights(decode_tail):
    """A large score scale under a wide cap makes every query put its weight on one key, wherever in its window the key lies: a
    key that is lost, shifted by one or read from the wrong page changes the output by its full size."""
    cfg = U.config([(U.attention(scale=6.0, window=0, softcap=200.0), None), (U.attention(scale=5.0, window=130, softcap=150.0), None)])
    W = U.weights(cfg, seed=19, gain=2.0)
    t = toks(300, seed=6)
    want = U.oracle_logits(cfg, W, t)
    e = U.engine(cfg, W, pool_tokens=320, page_size=16)
    got = U.feed(e, t, [300 - decode_tail])
    e.close()
    assert U.rel_err(got, want) < 1e-4


def _planted(n, window, heads=1, cap=0.0, scale=1.0):
    """Hand-made weights for one attention layer of width n over near-one-hot inputs (a large embedding factor dwarfs the
    position vector, and an RMS norm keeps a one-hot row's direction): the query of token 2 points, in every head, at the key
    of token 1; every other token's query is next to nothing.  The planted pair scores about n * scale."""
    cfg = U.config([(U.attention(heads=heads, kv_heads=1, dim=n, scale=scale, window=window, softcap=cap), None)], vocab=n, width=n, streams=0,
                   embed_scale=512.0)
    W = U.weights(cfg, seed=23)
    eye = np.eye(n, dtype=np.float32)
    W["embed"] = eye.copy()
    W["l0.norm1"] = np.ones(n, np.float32)
    q = np.zeros((heads * n, n), np.float32)
    q[1::n, 2] = 1.0
    W["l0.mix.q"], W["l0.mix.k"] = q, eye.copy()
    W["l0.mix.o"] = np.tile(eye * 64.0, (1, heads)).astype(np.float32)
    return cfg, W


@pytest.mark.parametrize("n,dtype", [(8, "float32"), (16, "bfloat16")])
def test_a_key_planted_far_back_is_found(n, dtype):
    """Token 1 occurs once among 260 tokens of one window; the last token (2) looks for it and finds nearly all of its weight
    there, wherever it stands: next to a page border on either side, at the very start, or just before the query."""
    cfg, W = _planted(n, window=512)
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
            assert U.rel_err(U.feed(e, t, [260 - tail]), want) < (1e-4 if dtype == "float32" else 2e-2), (where, tail)
    e.close()


@pytest.mark.parametrize("n,dtype", [(8, "float32"), (16, "bfloat16")])
@pytest.mark.parametrize("window", [100, 64, 37])
def test_keys_just_inside_and_just_outside_a_window(n, dtype, window):
    """The query (last token, position p) sees positions p - window + 1 .. p.  A planted key at the window's first position or
    the one after is seen; one at the position before the window, or two before, is not -- the query's output is then exactly
    that of the sequence without it -- also when the prompt was cut right at the edge and when the query is decoded alone."""
    cfg, W = _planted(n, window)
    e = U.engine(cfg, W, dtype, pool_tokens=448, page_size=16)
    for length in (2 * window + 31, 3 * window + 1, window + 2):
        lo = length - window  # first position the last token sees
        base = [int(x) for x in np.random.default_rng(2).integers(3, n, length)]
        base[-1] = 2
        without = U.oracle_logits(cfg, W, base)
        for where in (lo - 2, lo - 1, lo, lo + 1):
            if where < 0 or where >= length - 1:
                continue
            t = list(base)
            t[where] = 1
            want = U.oracle_logits(cfg, W, t)
            if where >= lo:
                assert np.abs(want[-1] - without[-1]).max() > 0.05
            else:
                assert np.abs(want[-1] - without[-1]).max() == 0.0
            for cuts in ([length], [lo, length - lo], [max(lo - 1, 1), 2, length], [length - 1, 1], [lo + 1, length], [length - 3]):
                got = U.feed(e, t, cuts)
                assert U.rel_err(got, want) < (1e-4 if dtype == "float32" else 2e-2), (length, where, cuts)
    e.close()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_the_unit_sink_takes_its_share(dtype):
    """The planted key scores about n * scale.  Where that is near zero every visible key and the sink's 1 weigh the same, so
    the first positions of the sequence give 1/2, 1/3, 1/4 of their weight away (every position's logits are compared, also with
    the first tokens fed one by one); where it is large the sink is nothing.  A second head with longer queries keeps the
    sum from merely changing size."""
    n = 16
    t = [int(x) for x in np.random.default_rng(3).integers(3, n, 90)]
    t[40], t[-1] = 1, 2
    outs = []
    for scale in (1e-3, 0.05, 1.0):
        cfg, W = _planted(n, window=128, heads=2, scale=scale)
        W["l0.mix.q"][n:] *= 7.0  # the second head's queries are longer
        want = U.oracle_logits(cfg, W, t)
        for cuts in ([90], [88, 1, 1], [1, 1, 1, 87]):
            got = U.run_portions(cfg, W, t, cuts, dtype, pool_tokens=128, page_size=16)
            assert U.rel_err(got, want) < (1e-4 if dtype == "float32" else 2e-2), (scale, cuts)
        outs.append(want[-1])
    assert np.abs(outs[0] - outs[1]).max() > 0.05 and np.abs(outs[1] - outs[2]).max() > 0.05


def test_the_score_cap_bites():
    """Scores far above the cap: every visible key of the capped head then weighs nearly the same, and the engine must follow
    the oracle there (a cap applied before the scale, or not at all, gives another answer)."""
    n = 8
    t = [int(x) for x in np.random.default_rng(4).integers(3, n, 60)]
    t[20], t[-1] = 1, 2
    res = []
    for cap in (0.0, 2.0, 40.0):
        cfg, W = _planted(n, window=0, cap=cap, scale=3.0)
        want = U.oracle_logits(cfg, W, t)
        assert U.rel_err(U.run_portions(cfg, W, t, [58], pool_tokens=64), want) < 1e-4
        res.append(want[-1])
    assert np.abs(res[0] - res[1]).max() > 0.05 and np.abs(res[1] - res[2]).max() > 0.05


def _planted_state(n):
    """Hand-made weights for one state-space layer of width n over near-one-hot inputs: token 1 writes into row 1 of the state,
    only token 2 reads, and it reads row 1; nothing decays to speak of.  Without a token 1 before it, token 2's mixer output is
    zero; with one -- however far back -- it is a vector of fixed size."""
    cfg = U.config([(U.ssm(heads=1, vdim=n, state=n, groups=1, conv=1, norm_groups=1), None)], vocab=n, width=n, streams=0, embed_scale=512.0)
    W = U.weights(cfg, seed=29)
    eye, zero = np.eye(n, dtype=np.float32), np.zeros((n, n), np.float32)
    read = zero.copy()
    read[1, 2] = 1.0
    W["embed"], W["l0.norm1"] = eye.copy(), np.ones(n, np.float32)
    W["l0.mix.in"] = np.concatenate([np.ones((n, n), np.float32), eye, eye, read, np.zeros((1, n), np.float32)])  # z | x | B | C | dt
    W["l0.mix.conv"], W["l0.mix.conv.b"] = np.ones((3 * n, 1), np.float32), np.zeros(3 * n, np.float32)
    W["l0.mix.dt_bias"], W["l0.mix.A_log"], W["l0.mix.D"] = np.zeros(1, np.float32), np.full(1, -9.0, np.float32), np.zeros(1, np.float32)
    W["l0.mix.norm"], W["l0.mix.o"] = np.ones(n, np.float32), (eye * 64.0).astype(np.float32)
    return cfg, W


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_state_carried_from_far_back(dtype):
    """Token 1 occurs once among 300 tokens; the last token (2) reads what it left in the state, wherever it stood: at the very
    start, on either side of a border between segments of the recurrence, or just before the reader -- whole, in ragged
    portions, and with the tail decoded through the slot's state."""
    n = 8
    cfg, W = _planted_state(n)
    base = [int(x) for x in np.random.default_rng(5).integers(3, n, 300)]
    base[-1] = 2
    without = U.oracle_logits(cfg, W, base)[-1]
    e = U.engine(cfg, W, dtype, pool_tokens=320, page_size=64)
    for where in (0, 63, 64, 65, 191, 298):
        t = list(base)
        t[where] = 1
        want = U.oracle_logits(cfg, W, t)
        assert np.abs(want[-1] - without).max() > 0.05  # what token 1 left decides the output
        for cuts in ([300], [3, 250, 2, 40], [where + 1, 64, 2], [296]):
            assert U.rel_err(U.feed(e, t, cuts), want) < (1e-4 if dtype == "float32" else 2e-2), (where, cuts)
    e.close()


def test_first_tokens_of_a_sequence():
    cfg = U.config(STACK, loop=LOOP)
    W = U.weights(cfg, seed=31)
    for n in (1, 2, 3, 5):
        t = toks(n, seed=50 + n)
        assert U.rel_err(U.run_whole(cfg, W, t), U.oracle_logits(cfg, W, t)) < F32_TOL, n
    t = toks(9, seed=60)
    assert U.rel_err(U.run_portions(cfg, W, t, [1, 1, 2, 1, 4]), U.oracle_logits(cfg, W, t)) < F32_TOL


def test_long_decoding_keeps_cache_and_state_exact():
    cfg = U.config([(U.attention(window=150), U.moe()), (U.ssm(), None), (U.attention(window=0), U.dense()), (U.ssm(conv=4), U.moe(shared=0))], loop=(0, 2, 2))
    W = U.weights(cfg, seed=37)
    t = toks(420, seed=9)
    want = U.oracle_logits(cfg, W, t)
    e = U.engine(cfg, W, pool_tokens=448, page_size=64)
    got = U.feed(e, t, [20])
    e.close()
    assert U.rel_err(got, want) < 5e-5


ODD = [(U.attention(heads=6, kv_heads=3, dim=10, window=11), U.moe(experts=12, top=5, ff=20, shared=9)),
       (U.ssm(heads=5, vdim=7, state=3, groups=5, conv=5, norm_groups=7), None),
       (U.attention(heads=1, kv_heads=1, dim=40, window=0, scale=0.9, softcap=0), U.moe(experts=3, top=3, ff=36, shared=0)),
       (U.ssm(heads=9, vdim=2, state=11, groups=3, conv=1, norm_groups=1), U.dense(ff=50)),
       (U.attention(heads=9, kv_heads=3, dim=6, window=50, softcap=1.5), U.moe(experts=10, top=1, ff=8, shared=40))]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("width,vocab,streams,loop", [(72, 131, 2, (1, 2, 3)), (136, 61, 5, None), (50, 33, 0, (0, 5, 2)), (33, 40, 1, (3, 5, 2))])
def test_other_sizes(dtype, width, vocab, streams, loop):
    cfg = U.config(ODD, vocab=vocab, width=width, eps=1e-3, streams=streams, loop=loop, embed_scale=1.0)
    W = U.weights(cfg, seed=41)
    t = toks(75, vocab=vocab, seed=10)
    want = U.oracle_logits(cfg, W, t)
    got = U.run_portions(cfg, W, t, [33, 2, 1, 1, 30, 8], dtype, page_size=16, pool_tokens=128)
    if dtype == "float32":
        assert U.rel_err(got, want) < 5e-5, U.row_errs(got, want)  # seven layer runs of odd sizes
    else:
        assert U.bf16_close(got, want)


def test_model_folder_round_trip(tmp_path):
    """config.json + model.safetensors written by the test, read back through the registry, loaded and run."""
    from tests.test_stack_cpu import write_safetensors
    cfg = U.config(STACK, loop=LOOP)
    W = U.weights(cfg, seed=43)
    write_safetensors(tmp_path / "model.safetensors", W)
    (tmp_path / "config.json").write_text(json.dumps(cfg))
    assert models.read_config(str(tmp_path))[1].name == "Goperax"
    t = toks(20, seed=12)
    e = models.load_model(str(tmp_path), dtype="float32", max_batch=2, max_tokens=64, page_size=16, max_step_tokens=64, max_logit_rows=68)
    got = U.feed(e, t, [20])
    e.close()
    assert U.rel_err(got, U.oracle_logits(cfg, W, t)) < F32_TOL


def test_greedy_generation_through_the_scheduler():
    """Requests of unequal length through the admission queue and the continuous batcher; greedy tokens equal the oracle's,
    except where the oracle's top two logits are closer than float32 noise."""
    cfg = U.config(STACK, vocab=40, loop=LOOP)
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
    """A made-up configuration: any order of the two mixers, any window, state and convolution sizes, feed-forwards of every
    kind, with or without streams and a loop."""
    width, vocab = int(rng.choice([48, 64, 96, 128, 200, 50])), int(rng.integers(40, 300))
    layers = []
    for _ in range(int(rng.integers(2, 7))):
        if rng.random() < 0.5:
            g = int(rng.choice([1, 2, 3, 4]))
            mx = U.attention(heads=g * int(rng.choice([1, 2, 4])), kv_heads=g, dim=int(rng.choice([8, 16, 24, 32, 64, 12, 20])),
                             window=int(rng.choice([0, 1, 7, 16, 33, 64, 100])), softcap=float(rng.choice([0, 2.0, 30.0])))
        else:
            g = int(rng.choice([1, 2, 3]))
            H, P = g * int(rng.choice([1, 2, 3])), int(rng.choice([4, 8, 16, 40]))
            parts = int(rng.choice([p for p in (1, 2, 3, 4, 8) if (H * P) % p == 0]))
            mx = U.ssm(heads=H, vdim=P, state=int(rng.choice([4, 8, 16, 33])), groups=g, conv=int(rng.choice([1, 2, 3, 4])), norm_groups=parts)
        r = rng.random()
        E = int(rng.choice([2, 3, 4, 6, 8, 12, 40]))
        ml = None if r < 0.2 else U.dense(ff=int(rng.choice([8, 24, 40]))) if r < 0.5 else \
            U.moe(experts=E, top=int(rng.integers(1, min(E, 6) + 1)), ff=int(rng.choice([8, 16, 24, 40])), shared=int(rng.choice([0, 8, 24])))
        layers.append((mx, ml))
    loop = None
    if rng.random() < 0.6:
        a = int(rng.integers(0, len(layers)))
        loop = (a, int(rng.integers(a + 1, len(layers) + 1)), int(rng.integers(1, 4)))
    return U.config(layers, vocab=vocab, width=width, eps=float(rng.choice([1e-5, 1e-3])), streams=int(rng.choice([0, 1, 2, 4])), loop=loop,
                    embed_scale=float(rng.choice([1.0, 7.5])))


@pytest.mark.parametrize("seed", range(6))
def test_random_configurations_and_schedules(seed):
    """Up to four live requests, random portions beside single tokens, requests left out of a step, a pool that makes pages and
    slots go round: every position's logits against the oracle."""
    rng = np.random.default_rng(2000 + seed)
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

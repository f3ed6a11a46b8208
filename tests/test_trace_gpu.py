"""bin/trace_run end to end: a model folder written by the test, a schedule with portions beside single tokens, four state
slots and a page pool smaller than the sum of the requests, logits compared with the plain implementation."""
import json
import os
import subprocess

import numpy as np
import pytest

from tests import _stack_util as U
from tests.test_stack_cpu import write_safetensors

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.mark.parametrize("dtype,tol", [("float32", 2e-4), ("bfloat16", None)])
def test_trace_replay_matches_the_plain_implementation(tmp_path, dtype, tol):
    cfg = U.config([(U.latent(), U.dense()), (U.lightning(), U.moe()), (U.latent(kv_from=0), None), (U.mingru(), U.dense())], vocab=90, width=40)
    _replay(tmp_path, dtype, tol, cfg, U.weights(cfg, seed=3), U.oracle_logits)


@pytest.mark.parametrize("dtype,tol", [("float32", 2e-4), ("bfloat16", None)])
def test_trace_replay_of_a_motolix_model(tmp_path, dtype, tol):
    """The same schedule through a looped Motolix model: attention pages and recurrent slots of every loop pass are handed on
    from request to request."""
    from tests import _motolix_util as M
    cfg = M.config([(M.parallel(dim=16, vdim=16, rot_dims=8), M.dense()), (M.attention(dim=16, rot_dims=8, scaling=(4.0, 1.0, 4.0, 64)), M.dense()),
                    (M.parallel(heads=2, kv_heads=1, r_heads=2), None)], vocab=90, width=40, loop=(0, 2, 2))
    _replay(tmp_path, dtype, tol, cfg, M.weights(cfg, seed=3), M.oracle_logits)


@pytest.mark.parametrize("dtype,tol", [("float32", 2e-4), ("bfloat16", None)])
def test_trace_replay_of_a_fakonex_model(tmp_path, dtype, tol):
    """The same schedule through a Fakonex model whose chunks (24, 40, 100 positions) and pages (64) never line up, with a layer
    that borrows another's keys and values: pages go from request to request under both."""
    from tests import _fakonex_util as F
    cfg = F.config([(F.attention(dim=16, vdim=16, chunk=24), F.moe()), (F.attention(dim=16, vdim=16, chunk=100, kv_from=0), F.moe(experts=4, top=2, groups=(2, 1), shared=0)),
                    (F.attention(heads=3, kv_heads=3, dim=6, vdim=10, chunk=40), None)], vocab=90, width=40)
    _replay(tmp_path, dtype, tol, cfg, F.weights(cfg, seed=3), F.oracle_logits)


@pytest.mark.parametrize("dtype,tol", [("float32", 2e-4), ("bfloat16", None)])
def test_trace_replay_of_a_goperax_model(tmp_path, dtype, tol):
    """The same schedule through a looped Goperax model: windows of 24 and 100 positions against pages of 64, recurrent state and
    convolution tails of every loop pass handed on from request to request."""
    from tests import _goperax_util as G
    cfg = G.config([(G.attention(dim=16, window=24), G.dense()), (G.ssm(), G.moe()), (G.attention(heads=3, kv_heads=3, dim=6, window=100), None),
                    (G.ssm(heads=2, vdim=16, state=16, groups=1, conv=4, norm_groups=1), G.moe(experts=4, top=1, shared=0))], vocab=90, width=40,
                   loop=(1, 3, 2))
    _replay(tmp_path, dtype, tol, cfg, G.weights(cfg, seed=3), G.oracle_logits)


def _replay(tmp_path, dtype, tol, cfg, W, oracle_logits):
    model = tmp_path / "model"
    model.mkdir()
    (model / "config.json").write_text(json.dumps(cfg))
    write_safetensors(model / "model.safetensors", W)
    rng = np.random.default_rng(4)
    reqs = {k: rng.integers(0, 90, n).tolist() for k, n in [("a", 150), ("b", 70), ("c", 1), ("d", 64), ("e", 129), ("f", 40)]}
    want = {k: oracle_logits(cfg, W, v) for k, v in reqs.items()}
    # steps: (id, count) lists; at most four requests live, 320 tokens of pages (64 each) for 454 tokens in total
    plan = [[("a", 100), ("b", 2)], [("a", 1), ("b", 60), ("c", 1)], [("a", 1), ("b", 1), ("d", 64)], [("a", 48), ("b", 7), ("d", 0)],
            [("e", 3), ("f", 39)], [("e", 2), ("f", 1)], [("e", 124)]]
    at, lines, asked = {k: 0 for k in reqs}, [], []
    for n, st in enumerate(plan):
        entries, end = [], []
        for k, cnt in st:
            if cnt == 0:
                continue
            lo, hi = at[k], at[k] + cnt
            w = sorted(set(rng.integers(0, cnt, min(cnt, 5)).tolist() + [cnt - 1]))
            entries.append({"id": k, "tokens": reqs[k][lo:hi], "want": w})
            asked.append((n, [(k, lo + j) for j in w]))
            at[k] = hi
            if hi == len(reqs[k]):
                end.append(k)
        lines.append(json.dumps({"step": n, "entries": entries, "end": end}))
    out = tmp_path / "out"
    r = subprocess.run([os.path.join(ROOT, "bin", "trace_run"), "--model", str(model), "--dtype", dtype, "--out", str(out),
                        "--max-tokens", "320"], input="\n".join(lines) + "\n", capture_output=True, text=True, cwd=ROOT, timeout=900)
    assert r.returncode == 0, r.stderr[-2000:]
    assert [ln for ln in r.stdout.splitlines() if ln.startswith("done")] == [f"done {n}" for n in range(len(plan))]
    per_step = {}
    for n, rows in asked:
        per_step.setdefault(n, []).extend(rows)
    got_all, want_all = [], []
    for n, rows in per_step.items():
        got = np.fromfile(out / f"{n}.f32", "<f4").reshape(len(rows), 90)
        got_all.append(got)
        want_all.append(np.stack([want[k][p] for k, p in rows]))
    got_all, want_all = np.concatenate(got_all), np.concatenate(want_all)
    if tol is not None:
        assert U.rel_err(got_all, want_all) < tol
    else:
        assert U.bf16_close(got_all, want_all)

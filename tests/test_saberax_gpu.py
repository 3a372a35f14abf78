"""Saberax in the engine against the plain implementation (tests/plain_saberax.py).

Small configurations with weights of their own (tests/saberax_tiny.py).  The 32-bit engine is
held to 2e-4 of the largest logit against the float64 oracle and, cut against cut, to bitwise
equality (every kernel of that path sums in an order that depends on the token's own place
only); the bfloat16 engine's error, position by position, to a fraction of the logits' spread in
the bulk of the positions.  Every engine runs with the cache's check mode on (pages that go back
are overwritten) and with fewer state slots than requests, so pages and slots are used again.
"""
import copy

import numpy as np
import pytest
import torch

import plain_saberax as plain
import replay
import saberax_tiny as st

pytestmark = pytest.mark.gpu

YARN = (4.0, 64, 8.0, 1.0)
BANDS = (8.0, 64, 1.0, 4.0)
# every size differs from model to model, and some are the degenerate values: one head, heads == kv_heads, groups of
# three query heads, one block, one tap, top == 1, top == experts, one group kept, groups == experts, no shared unit,
# a window and a chunk of one, no mask, no rotation, all dimensions rotated, no query scale, widths that are multiples
# of neither 8 nor 32, layers without feed-forward, a residual factor of one, layers on another layer's tensors
MODELS = {
    "mix": dict(layers=[(st.pair(st.normed(4, 2, 16, 24, q_temp=(0.3, 8)), st.recurrent(24, 3, 4)), st.dense(48)),
                        (st.pair(st.windowed(4, 2, 16, 16, window=11, rot=8, scaling=YARN), st.linear_attention(2, 8, 12, 8.0)),
                         st.moe(6, 2, 24, 2.0, groups=(3, 2), shared=16)),
                        (st.chunked(4, 2, 16, chunk=13, rot=8, scaling=BANDS), st.moe(6, 2, 24, 2.0, groups=(3, 2), shared=16)),
                        0, 1], vocab=97, width=40, eps=1e-5, mult=0.7, page=8, rank=6),
    "odd": dict(layers=[(st.chunked(3, 3, 10, chunk=1, rot=10, base=500.0), st.moe(5, 1, 10, 1.0, shared=None)),
                        (st.pair(st.windowed(3, 1, 10, 7, window=7, rot=6, base=500.0), st.linear_attention(1, 13, 35, 2.0)), st.dense(30)),
                        (st.pair(st.normed(1, 1, 24, 40, q_temp=None), st.recurrent(13, 1, 1)), None),
                        (st.chunked(6, 2, 12, chunk=None, rot=None), st.moe(4, 4, 16, 0.5, groups=(4, 4), shared=9)),
                        (st.pair(st.windowed(6, 6, 12, 12, window=1, rot=12, scaling=(16.0, 32, 4.0, 0.5)), st.linear_attention(3, 5, 3, 30.0)),
                         st.moe(8, 3, 6, 3.0, groups=(2, 1), shared=5)),
                        (st.pair(st.normed(2, 2, 6, 5, q_temp=(-0.2, 1)), st.recurrent(35, 5, 6)), st.dense(11)),
                        2], vocab=61, width=36, eps=1e-6, mult=1.0, page=16, rank=3),
    # sizes that the tensor-core kernels take in bfloat16 (multiples of 16 and 32 throughout, the grouped expert
    # products from 64 prompt tokens on)
    "even": dict(layers=[(st.pair(st.windowed(8, 2, 32, 64, window=44, rot=32, scaling=(8.0, 128, 16.0, 1.0)), st.linear_attention(4, 32, 48, 16.0)),
                          st.moe(8, 2, 64, 2.0, groups=(4, 2), shared=32)),
                         (st.pair(st.normed(4, 2, 64, 32, q_temp=(0.3, 32)), st.recurrent(96, 3, 4)), st.dense(128)),
                         (st.chunked(8, 2, 16, chunk=70, rot=8, scaling=(4.0, 32, 1.0, 4.0)), st.moe(8, 2, 64, 1.5, shared=64))],
                 vocab=80, width=64, eps=1e-6, mult=0.5, page=16, rank=16),
}
LENGTHS = {"mix": [1, 2, 9, 23, 40, 77], "odd": [3, 30, 64, 51], "even": [150, 70, 90]}


@pytest.fixture(scope="module")
def made(tmp_path_factory):
    root = tmp_path_factory.mktemp("saberax")
    out = {}
    for k, (name, m) in enumerate(MODELS.items()):
        raw = st.config(m["layers"], m["vocab"], m["width"], m["eps"], m["mult"])
        w = st.weights(raw, seed=5 + k, rank=m["rank"])
        rng = np.random.default_rng(40 + k)
        requests = {f"q{i}": rng.integers(0, m["vocab"], size=n).tolist() for i, n in enumerate(LENGTHS[name])}
        want = {rid: plain.forward(raw, w, toks).float() for rid, toks in requests.items()}
        out[name] = dict(raw=raw, weights=w, folder=st.write(raw, w, root / name), requests=requests, want=want,
                         page=m["page"])
    return out


_engines = {}


def engine(made, name, dtype, max_tokens=None, max_requests=3, graph=False):
    from fastllm_py_b200 import Model

    key = (name, dtype, max_tokens, max_requests, graph)
    if key not in _engines:
        _engines[key] = Model.load(made[name]["folder"], dtype=dtype, page_size=made[name]["page"],
                                   max_tokens=max_tokens or 512, max_requests=max_requests, max_batched_tokens=256,
                                   max_model_len=256, cuda_graph=graph, check_cache=True)
    return _engines[key]


def load(folder, dtype, page=4, tokens=64, requests=2, longest=64, check=True):
    from fastllm_py_b200 import Model

    return Model.load(folder, dtype=dtype, page_size=page, max_tokens=tokens, max_requests=requests,
                      max_batched_tokens=max(64, longest), max_model_len=longest, cuda_graph=False, check_cache=check).engine


def cuts(requests, live):
    return {"whole": replay.whole(requests), "tail": replay.tail_decode(requests, 12),
            "portions": replay.portions(requests), "small": replay.portions(requests, (2, 3, 2, 5, 2)),
            "mixed": replay.mixed(requests, live=live, seed=3, prefill_sizes=(9, 2, 17, 5), decode_tail=6)}


def worst(got, want):
    return max(float((got[(rid, p)] - want[rid][p]).abs().max()) for (rid, p) in got)


@pytest.mark.parametrize("name", list(MODELS))
def test_every_cut_in_32_bit_equals_the_oracle_and_the_other_cuts(made, name):
    m = made[name]
    top = max(float(v.abs().max()) for v in m["want"].values())
    results = {}
    for cut, steps in cuts(m["requests"], live=3).items():
        pool = replay.peak_tokens(steps, m["page"]) + (0 if cut == "mixed" else m["page"])
        eng = engine(made, name, "float32", pool).engine
        got = replay.run_in_process(eng, steps)
        assert len(got) == sum(len(t) for t in m["requests"].values())
        assert worst(got, m["want"]) <= 2e-4 * max(1.0, top), cut
        results[cut] = got
        assert not eng.cache.live
    for cut, got in results.items():
        for key, row in got.items():
            assert torch.equal(row, results["whole"][key]), (cut, key)
    assert engine(made, name, "float32", replay.peak_tokens(cuts(m["requests"], 3)["mixed"], m["page"])) \
        .engine.cache.pages_poisoned > 0


@pytest.mark.parametrize("name", list(MODELS))
def test_every_cut_in_bfloat16_stays_near_the_oracle(made, name):
    m = made[name]
    spread = float(torch.cat([v.flatten() for v in m["want"].values()]).std())
    for cut, steps in cuts(m["requests"], live=3).items():
        eng = engine(made, name, "bfloat16", replay.peak_tokens(steps, m["page"]) + m["page"]).engine
        got = replay.run_in_process(eng, steps)
        # a rounding error can flip an expert choice at single positions (and what follows them through the
        # states), so the bound is on the bulk of the positions, not on the worst one
        errs = np.array([float((got[k] - m["want"][k[0]][k[1]]).pow(2).mean().sqrt()) for k in got])
        assert np.median(errs) <= 0.08 * spread, cut
        assert np.quantile(errs, 0.9) <= 0.3 * spread, cut


def one_layer(mixer, mlp, **kw):
    return st.config([(mixer, mlp)], **kw)


SMALL = dict(width=24, vocab=50)
SINGLE = {
    "normed": one_layer(st.pair(st.normed(2, 1, 8, 40, q_temp=(0.4, 5)), st.recurrent(8, 1, 2)), None, **SMALL),
    "normed_wide_key": one_layer(st.pair(st.normed(2, 2, 72, 8, q_temp=None), st.recurrent(8, 2, 3)), None, **SMALL),
    "normed_wide_value": one_layer(st.pair(st.normed(3, 1, 8, 200), st.recurrent(8, 2, 3)), None, **SMALL),
    "recurrent": one_layer(st.pair(st.normed(1, 1, 4, 4), st.recurrent(40, 5, 4)), None, **SMALL),
    "recurrent_many_taps": one_layer(st.pair(st.normed(1, 1, 4, 4), st.recurrent(33, 3, 9)), None, mult=1.3, **SMALL),
    "windowed": one_layer(st.pair(st.windowed(2, 1, 8, 40, window=6, rot=4), st.linear_attention(1, 4, 4)), None, **SMALL),
    "windowed_all": one_layer(st.pair(st.windowed(3, 3, 8, 8, window=None, rot=8, scaling=YARN), st.linear_attention(1, 4, 4)), None, **SMALL),
    "windowed_no_turn": one_layer(st.pair(st.windowed(2, 2, 8, 8, window=9, rot=None), st.linear_attention(1, 4, 4)), None, **SMALL),
    "linear": one_layer(st.pair(st.windowed(1, 1, 4, 4, window=3, rot=2), st.linear_attention(2, 8, 40, 4.0)), None, **SMALL),
    "linear_wide_key": one_layer(st.pair(st.windowed(1, 1, 4, 4, window=3, rot=2), st.linear_attention(2, 72, 8, 16.0)), None, **SMALL),
    "linear_widest_key": one_layer(st.pair(st.windowed(1, 1, 4, 4, window=3, rot=2), st.linear_attention(1, 136, 33, 64.0)), None, **SMALL),
    "chunked": one_layer(st.chunked(2, 1, 8, chunk=6, rot=4), None, **SMALL),
    "chunked_all": one_layer(st.chunked(3, 3, 8, chunk=None, rot=8, scaling=BANDS), None, **SMALL),
    "chunked_wide": one_layer(st.chunked(2, 2, 72, chunk=17, rot=30, base=250000.0, scaling=(4.0, 16, 1.0, 4.0)), None, **SMALL),
    "dense": one_layer(st.chunked(1, 1, 8, chunk=4, rot=2), st.dense(36), **SMALL),
    "routed": one_layer(st.chunked(1, 1, 8, chunk=4, rot=2), st.moe(8, 3, 12, 2.0, groups=(4, 2), shared=10), **SMALL),
    "routed_pairs": one_layer(st.chunked(1, 1, 8, chunk=4, rot=2), st.moe(12, 3, 6, 0.7, groups=(2, 1), shared=None), **SMALL),
    "routed_free": one_layer(st.chunked(1, 1, 8, chunk=4, rot=2), st.moe(7, 3, 12, 1.0, shared=20), **SMALL),
}


@pytest.mark.parametrize("kind", list(SINGLE))
def test_each_mechanism_alone(tmp_path, kind):
    from fastllm_py_b200 import StepEntry

    raw = SINGLE[kind]
    w = st.weights(raw, seed=17, rank=5)
    folder = st.write(raw, w, tmp_path / kind)
    toks = np.random.default_rng(1).integers(0, raw["vocab"], size=45).tolist()
    want = plain.forward(raw, w, toks).float()
    eng = load(folder, "float32")
    eng.begin("a")
    head = eng.step([StepEntry("a", toks[:20], list(range(20)))]).cpu().clone()
    rest = [eng.step([StepEntry("a", [t], [0])]).cpu().clone() for t in toks[20:]]
    got = torch.cat([head] + rest)
    assert float((got - want).abs().max()) <= 2e-4 * max(1.0, float(want.abs().max()))


EDGES = st.config([(st.pair(st.windowed(2, 1, 16, 16, window=9, rot=8, scale=1.2), st.linear_attention(1, 4, 4)), st.dense(16)),
                   (st.chunked(2, 2, 16, chunk=17, rot=16, scale=1.2), None),
                   (st.pair(st.windowed(4, 2, 16, 32, window=23, rot=4, scale=1.2), st.linear_attention(1, 4, 4)), None),
                   (st.chunked(2, 1, 32, chunk=10, rot=8, scale=0.6), None)], width=32, vocab=40)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_window_and_chunk_edges_decide_the_output(tmp_path, dtype):
    """Scores so large that single keys decide a row: the oracle with every window and chunk one token
    wider or narrower is far from the engine, the oracle itself is not."""
    w = st.weights(EDGES, seed=3)
    folder = st.write(EDGES, w, tmp_path / "edges")
    toks = np.random.default_rng(2).integers(0, 40, size=70).tolist()
    want = plain.forward(EDGES, w, toks).float()
    small = load(folder, dtype, page=8, tokens=48, longest=128)
    roomy = load(folder, dtype, page=8, tokens=80, longest=128)
    bound = 2e-4 * float(want.abs().max()) if dtype == "float32" else 0.05 * float(want.std())
    for eng, steps in ((small, replay.tail_decode({"a": toks}, 40)), (small, replay.portions({"a": toks}, (5, 2, 9, 3))),
                       (roomy, replay.whole({"a": toks}))):
        got = replay.run_in_process(eng, steps)       # a small pool: pages behind the windows and chunks must go back
        if dtype == "float32":
            err = worst(got, {"a": want})
        else:
            err = float(np.median([float((got[k] - want[k[1]]).pow(2).mean().sqrt()) for k in got]))
        assert err <= bound
        for alter in ("wider", "narrower"):
            other = plain.forward(EDGES, w, toks, alter={alter}).float()
            if dtype == "float32":
                assert float((other - want).abs().max()) > 100 * max(err, 1e-5)
            else:
                assert float(np.median((other - want).pow(2).mean(dim=1).sqrt().numpy()[25:])) > 5 * bound


def test_every_mechanism_moves_the_logits(tmp_path):
    """The engine equals the oracle, and the oracle with one reading changed (no sink, no gate per head, no query
    scale, the other pairing) is far from both."""
    raw = st.config([(st.pair(st.normed(2, 1, 8, 8, q_temp=(0.5, 4), scale=1.0), st.recurrent(12, 2, 3)), st.dense(16)),
                     (st.pair(st.windowed(2, 1, 8, 8, window=14, rot=8, scale=1.5), st.linear_attention(2, 4, 6, 4.0)), None),
                     (st.chunked(2, 2, 8, chunk=15, rot=4, scale=1.5), None)], width=24, vocab=30)
    w = st.weights(raw, seed=1)
    folder = st.write(raw, w, tmp_path / "m")
    toks = np.random.default_rng(3).integers(0, 30, size=40).tolist()
    want = plain.forward(raw, w, toks).float()
    got = replay.run_in_process(load(folder, "float32"), replay.portions({"a": toks}, (7, 2, 11)))
    err = worst(got, {"a": want})
    assert err <= 2e-4 * float(want.abs().max())
    for alter in ("no_sink", "no_gate", "no_temp", "other_pairing"):
        other = plain.forward(raw, w, toks, alter={alter}).float()
        assert float((other - want).abs().max()) > 100 * max(err, 1e-5), alter


def test_a_far_key_among_hundreds_stands_out(tmp_path):
    """No mask: one early key is made to dominate a late query (its row of the embedding is scaled so that
    query and key align, and the query's scale has grown with its position), and the engine's logits there
    follow the oracle's; without that key, or without the growing scale, the oracle is far away."""
    raw = st.config([(st.pair(st.normed(2, 1, 16, 16, q_temp=(0.6, 32), scale=0.5), st.recurrent(8, 1, 2)), None)], width=32, vocab=40)
    w = st.weights(raw, seed=8)
    w["l0.mix.left.k"] = (w["l0.mix.left.q"].float()[:16] * 3.0).to(torch.bfloat16)     # keys point where head 0's queries do
    w["l0.mix.left.q.norm"] = torch.ones(16, dtype=torch.bfloat16)
    w["l0.mix.left.k.norm"] = torch.ones(16, dtype=torch.bfloat16)
    w["l0.norm1.b"] = torch.zeros(32, dtype=torch.bfloat16)
    folder = st.write(raw, w, tmp_path / "far")
    rng = np.random.default_rng(5)
    toks = rng.integers(0, 39, size=300).tolist()
    toks[3] = 39
    toks[290] = 39
    want = plain.forward(raw, w, toks).float()
    without = plain.forward(raw, w, toks[:3] + [0] + toks[4:]).float()
    flat = plain.forward(raw, w, toks, alter={"no_temp"}).float()
    eng = load(folder, "float32", page=16, tokens=320, requests=1, longest=320)
    for steps in (replay.whole({"a": toks}), replay.tail_decode({"a": toks}, 20)):
        got = replay.run_in_process(eng, steps)
        err = worst(got, {"a": want})
        assert err <= 2e-4 * float(want.abs().max())
        assert float((without[290] - want[290]).abs().max()) > 100 * max(err, 1e-5)
        assert float((flat[290] - want[290]).abs().max()) > 100 * max(err, 1e-5)


def test_a_far_token_reaches_through_the_states(tmp_path):
    """Decays close to one: the first token still moves the last logits through the recurrent unit's and the
    linear attention's states alone (the attentions beside them see one token), and the engine follows the oracle
    through 150 single-token steps after a short prompt."""
    raw = st.config([(st.pair(st.windowed(1, 1, 4, 4, window=1, rot=2), st.linear_attention(2, 16, 16, 64.0)), st.dense(16)),
                     (st.pair(st.normed(1, 1, 4, 4, q_temp=None), st.recurrent(16, 2, 3)), None)], width=24, vocab=40)
    raw["layers"][1]["mixer"]["left"]["mask"] = {"size": 1}
    w = st.weights(raw, seed=9, slow=True)
    folder = st.write(raw, w, tmp_path / "far")
    toks = np.random.default_rng(4).integers(0, 40, size=160).tolist()
    want = plain.forward(raw, w, toks).float()
    changed = plain.forward(raw, w, [(toks[0] + 1) % 40] + toks[1:]).float()
    eng = load(folder, "float32", page=16, tokens=256, longest=256, check=False)
    got = replay.run_in_process(eng, replay.tail_decode({"a": toks}, 150))
    err = worst(got, {"a": want})
    assert err <= 2e-4 * float(want.abs().max())
    assert float((changed[-1] - want[-1]).abs().max()) > 100 * max(err, 1e-5)


def test_a_slot_used_again_starts_clean(made):
    """Two requests one after the other in an engine with a single slot equal the same requests in
    fresh engines, bit for bit."""
    m = made["mix"]
    (ra, ta), (rb, tb) = list(m["requests"].items())[3:5]
    eng = engine(made, "mix", "float32", 128, max_requests=1).engine
    first = replay.run_in_process(eng, replay.portions({ra: ta}))
    second = replay.run_in_process(eng, replay.portions({rb: tb}))
    alone = replay.run_in_process(engine(made, "mix", "float32", 512).engine, replay.whole({rb: tb}))
    assert all(torch.equal(second[k], alone[k]) for k in alone)
    assert worst(first, m["want"]) <= 2e-4 * 30.0


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_greedy_generation_through_the_scheduler(made, dtype):
    """Model.generate (scheduler, sampler, captured decode steps) against the oracle's greedy loop;
    where the oracle's two best logits are close the engine may take either."""
    m = made["mix"]
    model = engine(made, "mix", dtype, 512, max_requests=3, graph=True)
    prompts = [m["requests"]["q2"], m["requests"]["q3"], m["requests"]["q1"], m["requests"]["q4"][:20]]
    outs = model.generate(prompts, max_new_tokens=12)
    assert model.generate(prompts, max_new_tokens=12, use_graph=False) == outs          # replayed steps change nothing
    gaps = []                                                    # how far below the oracle's best each token is, in spreads
    for prompt, new in zip(prompts, outs):
        seq = list(prompt)
        for tok in new:
            logits = plain.forward(m["raw"], m["weights"], seq)[-1]
            gaps.append(float(logits.max() - logits[tok]) / float(logits.std()))
            seq.append(tok)
        assert len(new) == 12
    if dtype == "float32":
        assert max(gaps) < 1e-3
    else:
        assert sum(g > 0.2 for g in gaps) <= 3 and max(gaps) < 1.0, sorted(gaps)[-5:]


def test_trace_program_on_a_folder(made, tmp_path):
    m = made["odd"]
    steps = replay.mixed(m["requests"], live=2, seed=1, prefill_sizes=(7, 2, 30), decode_tail=3)
    got = replay.run_program(m["folder"], "float32", steps, tmp_path / "out", replay.peak_tokens(steps, 64),
                             m["raw"]["vocab"], extra_args=("--max-requests", "2"))
    top = max(float(v.abs().max()) for v in m["want"].values())
    assert worst(got, m["want"]) <= 2e-4 * max(1.0, top)


def test_command_line_on_a_random_weights_folder(tmp_path):
    """bin/make_model writes a folder from a configuration, bin/generate loads it by its architecture
    string and generates through the scheduler."""
    import json
    import subprocess
    import sys

    raw = st.config([(st.pair(st.normed(2, 1, 16, 16), st.recurrent(32, 2, 4)), st.moe(4, 2, 16, groups=(2, 1))),
                     (st.chunked(2, 1, 16, chunk=20, rot=16), st.dense(32)), 0], width=32, vocab=64)
    (tmp_path / "config.json").write_text(json.dumps(raw))
    made_ = subprocess.run([sys.executable, str(replay.ROOT / "bin" / "make_model"), str(tmp_path / "config.json"),
                            str(tmp_path / "m"), "--seed", "4", "--std", "0.2"], capture_output=True, text=True)
    assert made_.returncode == 0 and "Saberax" in made_.stdout, made_.stderr
    run = subprocess.run([sys.executable, str(replay.ROOT / "bin" / "generate"), str(tmp_path / "m"), "-", "9",
                          "bfloat16", "--random-prompt", "30", "--seed", "1"], capture_output=True, text=True)
    assert run.returncode == 0, run.stderr[-2000:]
    lines = run.stdout.strip().splitlines()
    assert "Saberax: 3L width=32" in lines[0]
    assert len([int(t) for t in lines[1].split(",")]) == 9


# ------------------------------------------------------------------ kernels alone

def test_router_choice_by_the_sum_of_a_groups_two_best():
    from fastllm_py_b200.native import ops

    gen = torch.Generator().manual_seed(3)
    for experts, top, groups in ((12, 3, (4, 2)), (20, 4, (5, 3)), (6, 2, (6, 2)), (6, 1, (6, 1)), (8, 8, (2, 2)), (9, 2, None),
                                 (40, 5, (5, 2)), (12, 3, (2, 1))):
        z = torch.randn(70, experts, generator=gen) * 2.0
        corr = torch.randn(experts, generator=gen) * 0.7
        r = {"experts": experts, "top": top, "scale": 2.5}
        if groups:
            r["groups"] = {"count": groups[0], "keep": groups[1]}
        # the oracle's route() takes h and a router matrix: an identity router makes its logits z itself
        want_e, want_w = plain.route(z.double(), torch.eye(experts, dtype=torch.float64), corr.double(), r)
        chosen = torch.empty(70, top, dtype=torch.int32, device="cuda")
        weights = torch.empty(70, top, device="cuda")
        ops.moe_pick(z.cuda(), corr.cuda(), chosen, weights, top, False, True, groups and groups[0], groups and groups[1],
                     1e-20, group_top=2, weight_scale=2.5)
        got_e, got_w = chosen.cpu().long(), weights.cpu().double()
        assert torch.equal(got_e.sort(dim=1).values, want_e.sort(dim=1).values), (experts, top, groups)
        assert torch.allclose(got_w.gather(1, got_e.argsort(dim=1)), want_w.gather(1, want_e.argsort(dim=1)), atol=1e-6)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_layer_norm_mix_and_activation_kernels(dtype):
    from fastllm_py_b200.native import ops

    gen = torch.Generator().manual_seed(1)
    tol = 2e-6 if dtype == torch.float32 else 2e-2
    for rows, width in ((19, 44), (3, 1000), (40, 192)):
        x = torch.randn(rows, width, generator=gen).cuda() * 3.0 + 1.5
        d = torch.randn(rows, width, generator=gen).to(dtype).cuda()
        w = (1 + 0.2 * torch.randn(width, generator=gen)).to(torch.bfloat16).cuda()
        b = (0.3 * torch.randn(width, generator=gen)).to(torch.bfloat16).cuda()
        out = torch.empty(rows, width, dtype=dtype, device="cuda")
        total = x.double() + 0.7 * d.double()
        mu = total.mean(dim=1, keepdim=True)
        normed = (total - mu) / torch.sqrt(((total - mu) ** 2).mean(dim=1, keepdim=True) + 1e-5) * w.double() + b.double()
        xs = x.clone()
        ops.add_layernorm(xs, d, 0.7, w, b, out, 1e-5)
        assert float((xs.double() - total).abs().max()) <= 1e-6
        assert float((out.double() - normed).abs().max()) <= 4 * tol
        pick = torch.tensor([rows - 1, 0, 2], dtype=torch.int32, device="cuda")
        xs, few = x.clone(), torch.empty(3, width, dtype=dtype, device="cuda")
        ops.add_layernorm(xs, d, 0.7, w, b, few, 1e-5, pick)
        assert torch.equal(xs, x)                                               # gathered rows leave the stream alone
        assert float((few.double() - normed[pick.cpu().long()]).abs().max()) <= 4 * tol
        ops.add_layernorm(xs, None, 1.0, w, b, out, 1e-5)                       # nothing pending
        mu = x.double().mean(dim=1, keepdim=True)
        plain_ln = (x.double() - mu) / torch.sqrt(((x.double() - mu) ** 2).mean(dim=1, keepdim=True) + 1e-5) * w.double() + b.double()
        assert float((out.double() - plain_ln).abs().max()) <= 4 * tol

        a2 = torch.randn(rows, width, generator=gen).to(dtype).cuda() * 2.0
        b2 = torch.randn(rows, width, generator=gen).to(dtype).cuda() * 0.1
        ops.rms_mix(a2, b2, w, b, out, 1e-5, 0.5)
        want = 0.5 * (plain.rms(a2.double(), 1e-5) * w.double() + plain.rms(b2.double(), 1e-5) * b.double())
        assert float((out.double() - want).abs().max()) <= tol
        ops.activation(a2, out, "relu_squared")
        squared = torch.relu(a2.double()) ** 2
        assert float(((out.double() - squared).abs() / (1.0 + squared)).max()) <= tol
        xs = x.clone()
        ops.scaled_add(xs, d, -1.3)
        assert float((xs.double() - (x.double() - 1.3 * d.double())).abs().max()) <= 1e-6


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_experts_without_a_gate_both_ways_through_them(dtype):
    """The per-token kernels against dense matrices, added to what the output holds; in bfloat16 the grouped
    tensor-core products against the per-token kernels, with an expert that gets no row."""
    from fastllm_py_b200.native import ops

    gen = torch.Generator().manual_seed(2)
    n, width, ff, experts, top = 150, 64, 96, 7, 2
    h = torch.randn(n, width, generator=gen).to(dtype).cuda()
    up = (torch.randn(experts, ff, width, generator=gen) / 8).to(torch.bfloat16).cuda()
    down = (torch.randn(experts, width, ff, generator=gen) / 10).to(torch.bfloat16).cuda()
    chosen = torch.randint(0, experts - 1, (n, top), generator=gen, dtype=torch.int32).cuda()      # the last expert gets no row
    weights = torch.rand(n, top, generator=gen).cuda()
    held = torch.randn(n, width, generator=gen).to(dtype).cuda()
    want = held.double().cpu().clone()
    for t in range(n):
        for k in range(top):
            e = int(chosen[t, k])
            want[t] += float(weights[t, k]) * (torch.relu(h[t].double().cpu() @ up[e].double().cpu().T) ** 2 @ down[e].double().cpu().T)
    out = held.clone()
    act = torch.empty(n * top, ff, device="cuda")
    ops.moe_experts(h, up, down, chosen, weights, act, out, "relu_squared", gated=False, accumulate=True)
    tol = 1e-4 if dtype == torch.float32 else 0.05
    assert float((out.double().cpu() - want).abs().max()) <= tol
    if dtype == torch.bfloat16:
        assert ops.moe_group_takes(dtype, up.dtype, width, ff)
        rows = ops.moe_group_rows(n, top, experts)
        ints = torch.empty(rows + n * top + rows // 64 + 1, dtype=torch.int32, device="cuda")
        acts = torch.empty(rows, ff, dtype=torch.bfloat16, device="cuda")
        y = torch.empty(rows, width, device="cuda")
        grouped = held.clone()
        ops.moe_experts_grouped(h, up, down, chosen, weights, ints, acts, y, grouped, "relu_squared", gated=False, accumulate=True)
        assert float((grouped.double().cpu() - want).abs().max()) <= tol


def _paged(gen, kv_heads, row_w, ctx_lens, q_lens, page=16):
    n_pages = sum(-(-(c + q) // page) for c, q in zip(ctx_lens, q_lens))
    order = torch.randperm(n_pages + 5, generator=gen)[:n_pages].tolist()
    cache = (torch.randn(n_pages + 5, kv_heads, page, row_w, generator=gen) * 0.7).to(torch.bfloat16)
    bt = torch.zeros(len(q_lens), 16, dtype=torch.int32)
    for r, (c, ql) in enumerate(zip(ctx_lens, q_lens)):
        for i in range(-(-(c + ql) // page)):
            bt[r, i] = order.pop()
    return cache, bt


@pytest.mark.parametrize("dim,vdim,window,chunk,heads,kv_heads,sink", [
    (32, 64, 70, None, 4, 2, False), (16, 16, None, 50, 6, 2, True), (64, 64, None, 33, 3, 3, True),
    (48, 80, 81, 64, 8, 1, False), (96, 48, None, None, 4, 2, False), (128, 128, None, 90, 2, 1, True)])
def test_tensor_core_and_split_key_attention_equal_the_cuda_core_one(dim, vdim, window, chunk, heads, kv_heads, sink):
    """Scattered pages, a prompt portion behind cached tokens beside single tokens, a standout key just inside the
    window or at the start of the chunk of one query."""
    from types import SimpleNamespace

    from fastllm_py_b200.native import ops

    gen = torch.Generator().manual_seed(dim + vdim)
    page = 16
    ctx_lens, q_lens = [37, 150, 0, 201], [100, 1, 70, 1]
    cache, bt = _paged(gen, kv_heads, dim + vdim, ctx_lens, q_lens, page)
    n = sum(q_lens)
    q = (torch.randn(n, heads * dim, generator=gen) * 0.7).to(torch.bfloat16)
    # request 0, row 60 (position 97): the first key it sees answers it loudly
    if window or chunk:
        edge = max(97 - window + 1 if window else 0, 97 // chunk * chunk if chunk else 0)
        pg, off = int(bt[0, edge // page]), edge % page
        cache[pg, 0, off, :dim] = q[60, :dim].float().mul(4.0).to(torch.bfloat16)
    tok_req = torch.tensor(sum(([r] * ql for r, ql in enumerate(q_lens)), []), dtype=torch.int32)
    positions = torch.tensor(sum((list(range(c, c + ql)) for c, ql in zip(ctx_lens, q_lens)), []), dtype=torch.int32)
    starts = [0]
    for ql in q_lens:
        starts.append(starts[-1] + ql)
    dev = lambda t: t.cuda()
    step = SimpleNamespace(req_start=dev(torch.tensor(starts, dtype=torch.int32)),
                           req_ctx=dev(torch.tensor(ctx_lens, dtype=torch.int32)),
                           req_qlen=dev(torch.tensor(q_lens, dtype=torch.int32)), n_requests=4)
    sinks = dev(torch.randn(heads, generator=gen)) if sink else None
    want = torch.empty(n, heads * vdim, dtype=torch.bfloat16, device="cuda")
    got = torch.empty_like(want)
    ops.sink_attention_simt(dev(q), want, dev(cache), dev(bt), dev(tok_req), dev(positions), heads, kv_heads, dim, vdim,
                            window, 0, dim ** -0.5, None, None, None, sinks, page, chunk=chunk)
    # the plain arithmetic of it for one row, from the cache as it lies in memory
    for row, r in ((60, 0), (starts[3], 3)):
        pos = int(positions[row])
        lo = max(pos - window + 1, 0) if window else 0
        if chunk:
            lo = max(lo, pos // chunk * chunk)
        keys = torch.stack([cache[int(bt[r, j // page]), 0, j % page] for j in range(lo, pos + 1)]).double()
        s = keys[:, :dim] @ q[row, :dim].double() * dim ** -0.5
        e = torch.exp(s - s.max())
        den = e.sum() + (torch.exp(sinks[0].double().cpu() - s.max()) if sink else 0.0)
        assert float((want[row, :vdim].double().cpu() - (e[:, None] * keys[:, dim:]).sum(0) / den).abs().max()) <= 0.03
    ops.sink_attention_tc(dev(q), got, dev(cache), dev(bt), step, heads, kv_heads, dim, vdim, window, 0, dim ** -0.5, None,
                          None, None, sinks, page, chunk=chunk)
    torch.cuda.synchronize()
    err = (got.float() - want.float()).abs()
    assert float(err.max()) <= 0.06 and float(err.mean()) <= 0.006, (float(err.max()), float(err.mean()))
    # the single tokens through the split-key kernel, the portions through the tensor-core one
    assert ops.sink_decode_takes(heads, kv_heads, dim, vdim)
    singles = dev(torch.tensor([starts[1], starts[3]], dtype=torch.int32))
    n_splits, kept = ops.sink_decode_splits(window, 0, 202, chunk)
    partial = torch.empty(2 * heads * n_splits * (vdim + 2), device="cuda")
    both = torch.zeros_like(want)
    ops.sink_attention_tc(dev(q), both, dev(cache), dev(bt), step, heads, kv_heads, dim, vdim, window, 0, dim ** -0.5, None,
                          None, None, sinks, page, include_single=False, chunk=chunk)
    assert float(both[starts[1]].float().abs().max()) == 0.0 and float(both[starts[3]].float().abs().max()) == 0.0
    ops.sink_decode(dev(q), both, dev(cache), dev(bt), dev(tok_req), dev(positions), singles, partial, n_splits, kept, heads,
                    kv_heads, dim, vdim, window, 0, dim ** -0.5, None, None, None, sinks, page, chunk=chunk)
    torch.cuda.synchronize()
    err = (both.float() - want.float()).abs()
    assert float(err.max()) <= 0.06 and float(err.mean()) <= 0.006, (float(err.max()), float(err.mean()))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_recurrence_and_linear_attention_kernels_over_three_steps(dtype):
    """Two requests through three steps of unequal portions (one of them starts later in a slot used before)
    against the oracle's functions on the whole sequences."""
    from types import SimpleNamespace

    from fastllm_py_b200.native import ops

    gen = torch.Generator().manual_seed(4)
    dev = lambda t: t.cuda()
    width, blocks, taps = 40, 5, 4
    heads, dim, vdim, rank, tau = 2, 12, 20, 3, 6.0
    lens = [23, 17]
    # ---- the inputs of whole sequences, as the projections would leave them
    proj_r = [(torch.randn(n, 2 * width, generator=gen)).to(dtype) for n in lens]
    proj_g = [(torch.randn(n, 2 * heads * dim + 2 * heads * vdim + rank, generator=gen)).to(dtype) for n in lens]
    m_r = {"width": width, "blocks": blocks, "conv": taps}
    t_r = {"y": torch.eye(2 * width)[:width], "x": torch.eye(2 * width)[width:], "y.b": torch.randn(width, generator=gen) * 0.3,
           "x.b": torch.randn(width, generator=gen) * 0.3, "conv": torch.randn(width, taps, generator=gen) * 0.5,
           "conv.b": torch.randn(width, generator=gen) * 0.3, "ra": torch.randn(blocks, 8, 8, generator=gen) * 0.5,
           "ri": torch.randn(blocks, 8, 8, generator=gen) * 0.5, "ra.b": torch.randn(blocks, 8, generator=gen) * 0.3,
           "ri.b": torch.randn(blocks, 8, generator=gen) * 0.3, "lam": torch.randn(width, generator=gen) - 3.0,
           "o": torch.eye(width)}
    t_r = {k: v.double() for k, v in t_r.items()}
    cols = 2 * heads * dim + 2 * heads * vdim + rank
    eye = torch.eye(cols, dtype=torch.float64)
    hd, hv = heads * dim, heads * vdim
    t_g = {"q": eye[:hd], "k": eye[hd:2 * hd], "v": eye[2 * hd:2 * hd + hv], "g": eye[2 * hd + hv:2 * hd + 2 * hv],
           "a1": eye[2 * hd + 2 * hv:], "a2": torch.randn(hd, rank, generator=gen).double(),
           "a2.b": torch.randn(hd, generator=gen).double() + 2.0, "norm": (1 + 0.3 * torch.randn(vdim, generator=gen)).double(),
           "o": torch.eye(hv, dtype=torch.float64)}
    m_g = {"heads": heads, "dim": dim, "vdim": vdim, "tau": tau}
    want_r = [plain.gated_recurrence(p.double(), t_r, m_r)[0] for p in proj_r]
    want_g = [plain.gated_linear_attention(p.double(), t_g, m_g, 1e-5)[0] for p in proj_g]
    # ---- the kernels' operands
    f32 = lambda t: dev(t.float().contiguous())
    bias = f32(torch.cat([t_r["y.b"], t_r["x.b"]]))
    rate = f32(-8.0 * torch.nn.functional.softplus(t_r["lam"]))
    state_r = torch.full((3, width * taps), 1e4, device="cuda")
    state_g = torch.full((3, heads * vdim * dim), 1e4, device="cuda")
    got_r = [torch.zeros(n, width) for n in lens]
    got_g = [torch.zeros(n, hv) for n in lens]
    # request 0 in slot 2 from the first step; request 1 joins at the second step in slot 0
    schedule = [[(0, 0, 9)], [(0, 9, 1), (1, 0, 11)], [(1, 11, 6), (0, 10, 13)]]
    for entries in schedule:
        n = sum(e[2] for e in entries)
        starts = [0]
        for e in entries:
            starts.append(starts[-1] + e[2])
        step = SimpleNamespace(
            tok_req=dev(torch.tensor(sum(([i] * e[2] for i, e in enumerate(entries)), []), dtype=torch.int32)),
            positions=dev(torch.tensor(sum((list(range(e[1], e[1] + e[2])) for e in entries), []), dtype=torch.int32)),
            req_start=dev(torch.tensor(starts, dtype=torch.int32)), req_ctx=dev(torch.tensor([e[1] for e in entries], dtype=torch.int32)),
            req_qlen=dev(torch.tensor([e[2] for e in entries], dtype=torch.int32)),
            req_slot=dev(torch.tensor([2 if e[0] == 0 else 0 for e in entries], dtype=torch.int32)), n_requests=len(entries))
        pr = dev(torch.cat([proj_r[e[0]][e[1]:e[1] + e[2]] for e in entries]))
        pg = dev(torch.cat([proj_g[e[0]][e[1]:e[1] + e[2]] for e in entries]))
        u, a, bx = (torch.empty(n, width, device="cuda") for _ in range(3))
        out = torch.empty(n, width, dtype=dtype, device="cuda")
        ops.rglru(pr, bias, f32(t_r["conv"]), f32(t_r["conv.b"]), f32(t_r["ra"]), f32(t_r["ri"]), f32(t_r["ra.b"].reshape(-1)),
                  f32(t_r["ri.b"].reshape(-1)), rate, state_r, step, u, a, bx, out, width, blocks, taps)
        work = torch.empty(n, 3 * hd + hv, device="cuda")
        o = torch.empty(n, hv, device="cuda")
        y = torch.empty(n, hv, dtype=dtype, device="cuda")
        ops.gla_prep(pg, f32(t_g["a2"].T), f32(t_g["a2.b"]), work, heads, dim, vdim, rank, dim ** -0.5, tau)
        ops.gla_scan(work, o, state_g, step, heads, dim, vdim)
        ops.gla_gated_norm(o, pg[:, 2 * hd + hv:2 * hd + 2 * hv], f32(t_g["norm"]), y, heads, vdim, 1e-5)
        for i, e in enumerate(entries):
            got_r[e[0]][e[1]:e[1] + e[2]] = out[starts[i]:starts[i + 1]].float().cpu()
            got_g[e[0]][e[1]:e[1] + e[2]] = y[starts[i]:starts[i + 1]].float().cpu()
    tol = 2e-5 if dtype == torch.float32 else 0.03
    for k in range(2):
        assert float((got_r[k].double() - want_r[k]).abs().max()) <= tol * max(1.0, float(want_r[k].abs().max()))
        assert float((got_g[k].double() - want_g[k]).abs().max()) <= tol * max(1.0, float(want_g[k].abs().max()))


@pytest.mark.parametrize("mode,pairing,v_from_k", [("weighted", "half", False), ("unit", "interleaved", False),
                                                   ("unit", "half", True), (None, "interleaved", False)])
def test_preparation_head_by_head_follows_the_oracle(mode, pairing, v_from_k):
    from fastllm_py_b200.native import ops

    gen = torch.Generator().manual_seed(6)
    heads, kv_heads, dim, rot, n, page = 3, 1, 20, 12, 9, 4
    vdim = dim if v_from_k else 7
    cols = heads * dim + kv_heads * dim + (0 if v_from_k else kv_heads * vdim)
    proj = torch.randn(n, cols, generator=gen).cuda()
    bias = torch.randn(cols, generator=gen).cuda() * 0.3
    q_w, k_w = (1 + 0.3 * torch.randn(dim, generator=gen)).cuda(), (1 + 0.3 * torch.randn(dim, generator=gen)).cuda()
    positions = torch.tensor([5, 6, 7, 8, 9, 10, 11, 0, 1], dtype=torch.int32)
    f, gain = plain.rotary_frequencies(rot, 300.0, None)
    ang = torch.arange(16, dtype=torch.float64)[:, None] * f[None, :]
    cos, sin = torch.cos(ang).float().cuda(), torch.sin(ang).float().cuda()
    slots = torch.tensor([8, 9, 10, 11, 0, 1, 2, 20, 21], dtype=torch.int32).cuda()
    cache = torch.zeros(6, kv_heads, page, dim + vdim, device="cuda")
    q_out = torch.empty(n, heads * dim, device="cuda")
    ops.head_prep(proj, bias, q_w if mode == "weighted" else None, k_w if mode == "weighted" else None,
                  {None: 0, "weighted": 1, "unit": 2}[mode], 1e-5, rot, pairing == "interleaved", cos, sin, positions.cuda(),
                  (0.4, 3), v_from_k, q_out, heads, kv_heads, dim, vdim, slots, cache, page)
    x = (proj + bias).double().cpu()
    q, k = x[:, :heads * dim].view(n, heads, dim), x[:, heads * dim:(heads + kv_heads) * dim].view(n, kv_heads, dim)
    v = k.clone() if v_from_k else x[:, (heads + kv_heads) * dim:].view(n, kv_heads, vdim)
    if mode == "weighted":
        q, k = plain.rms(q, 1e-5) * q_w.double().cpu(), plain.rms(k, 1e-5) * k_w.double().cpu()
    spec = {"dims": rot, "base": 300.0}
    q, k = plain.rotate(q, positions, spec, pairing), plain.rotate(k, positions, spec, pairing)
    if mode == "unit":
        q, k = plain.rms(q, 1e-5), plain.rms(k, 1e-5)
    q = q * (1.0 + 0.4 * torch.log(torch.floor((positions.double() + 1) / 3) + 1.0))[:, None, None]
    assert float((q_out.double().cpu() - q.reshape(n, -1)).abs().max()) <= 1e-5
    stored = torch.stack([cache[int(s) // page, 0, int(s) % page] for s in slots]).double().cpu()
    assert float((stored[:, :dim] - k[:, 0]).abs().max()) <= 1e-5
    assert float((stored[:, dim:] - v[:, 0]).abs().max()) <= 1e-5


def test_recurrence_in_segments_equals_token_by_token():
    """A prompt portion of 333 tokens behind 7 cached ones beside a short one: the form that runs a request's tokens in
    segments side by side against the token-by-token form (equal within rounding, states and kept inputs included)."""
    from types import SimpleNamespace

    from fastllm_py_b200.native import ops

    gen = torch.Generator().manual_seed(7)
    dev = lambda t: t.cuda()
    width, blocks, taps, lens, ctxs = 72, 3, 4, [333, 40], [7, 0]
    n = sum(lens)
    proj = dev(torch.randn(n, 2 * width, generator=gen).to(torch.bfloat16))
    bias = dev(torch.randn(2 * width, generator=gen) * 0.3)
    conv_w, conv_b = dev(torch.randn(width, taps, generator=gen) * 0.5), dev(torch.randn(width, generator=gen) * 0.3)
    w_a = dev((torch.randn(blocks, 24, 24, generator=gen) * 0.4).to(torch.bfloat16))
    w_i = dev((torch.randn(blocks, 24, 24, generator=gen) * 0.4).to(torch.bfloat16))
    b_a, b_i = dev(torch.randn(width, generator=gen) * 0.3), dev(torch.randn(width, generator=gen) * 0.3)
    rate = dev(-8.0 * torch.nn.functional.softplus(torch.randn(width, generator=gen) - 4.0))
    step = SimpleNamespace(
        tok_req=dev(torch.tensor([0] * lens[0] + [1] * lens[1], dtype=torch.int32)),
        positions=dev(torch.tensor(list(range(7, 7 + lens[0])) + list(range(lens[1])), dtype=torch.int32)),
        req_start=dev(torch.tensor([0, lens[0], n], dtype=torch.int32)), req_ctx=dev(torch.tensor(ctxs, dtype=torch.int32)),
        req_qlen=dev(torch.tensor(lens, dtype=torch.int32)), req_slot=dev(torch.tensor([1, 0], dtype=torch.int32)), n_requests=2)
    results = []
    for fixed in (True, False):
        state = dev(torch.randn(2, width * taps, generator=torch.Generator().manual_seed(8)))
        u, a, bx = (torch.empty(n, width, device="cuda") for _ in range(3))
        out = torch.empty(n, width, dtype=torch.bfloat16, device="cuda")
        ops.rglru(proj, bias, conv_w, conv_b, w_a, w_i, b_a, b_i, rate, state, step, u, a, bx, out, width, blocks, taps,
                  fixed_order=fixed)
        results.append((out.float().cpu(), state.cpu()))
    (seq_out, seq_state), (seg_out, seg_state) = results
    assert float((seq_out - seg_out).abs().max()) <= 0.02 * float(seq_out.abs().max())
    assert float((seq_state - seg_state).abs().max()) <= 1e-5 * max(1.0, float(seq_state.abs().max()))
    assert float(seq_state[1, :width].abs().max()) > 0                      # slot 1 carried its state in and out


def _drawn_model(rng):
    """A configuration drawn at random: layer kinds in any order, layers on another layer's tensors, sizes from lists
    that hold the awkward ones (one head, twelve query heads a key/value head, keys of 72, blocks of 13, one tap)."""
    ch = rng.choice
    width, vocab = ch([24, 40, 64, 136]), rng.randint(50, 200)

    def sizes():
        kv, group = ch([1, 2, 3]), ch([1, 1, 2, 3, 4, 12])
        return kv * group, kv, ch([8, 12, 16, 24, 32, 48, 64, 72])

    def rotation(dim, yarn):
        if rng.random() < 0.2:
            return None, None
        scaling = None
        if rng.random() < 0.6:
            scaling = (ch([2.0, 4.0, 32.0]), ch([16, 64, 1024]), ch([8.0, 32.0]), ch([0.5, 1.0])) if yarn else \
                (ch([2.0, 8.0]), ch([16, 64, 512]), ch([0.5, 1.0]), ch([2.0, 4.0]))
        return 2 * rng.randint(1, dim // 2), scaling

    def mlp():
        r = rng.random()
        if r < 0.2:
            return None
        if r < 0.5:
            return st.dense(ch([16, 30, 64]))
        experts = ch([4, 6, 8, 12, 16])
        top = rng.randint(1, min(experts, 5))
        groups = None
        if rng.random() < 0.6:
            count = ch([g for g in (1, 2, 3, 4, 6, 8) if experts % g == 0])
            keep = rng.randint(1, count)
            if keep * (experts // count) >= top:
                groups = (count, keep)
        return st.moe(experts, top, ch([8, 16, 32]), ch([0.5, 1.0, 2.5]), groups, ch([None, 8, 24]))

    layers, own = [], []
    for _ in range(rng.randint(3, 6)):
        if own and rng.random() < 0.2:
            layers.append(ch(own))
            continue
        kind = ch(["parallel", "parallel_2", "attention"])
        heads, kv, dim = sizes()
        scale, mask = ch([dim ** -0.5, 0.1, 0.3]), ch([None, 1, 2, 5, 17, 33])
        if kind == "attention":
            dims, scaling = rotation(dim, False)
            mixer = st.chunked(heads, kv, dim, chunk=mask, rot=dims, base=ch([500.0, 250000.0]), scaling=scaling, scale=scale)
        elif kind == "parallel":
            bw, blocks = ch([4, 8, 13, 16, 32]), ch([1, 2, 3, 5])
            temp = None if rng.random() < 0.3 else (ch([0.1, 0.3, -0.1]), ch([1, 4, 16]))
            mixer = st.pair(st.normed(heads, kv, dim, ch([4, 8, 24, 48, 100]), q_temp=temp, scale=scale),
                            st.recurrent(bw * blocks, blocks, ch([1, 2, 4, 7])))
        else:
            dims, scaling = rotation(dim, True)
            mixer = st.pair(st.windowed(heads, kv, dim, ch([4, 8, 24, 48, 100]), window=mask, rot=dims, base=ch([500.0, 50000.0]),
                                        scaling=scaling, scale=scale),
                            st.linear_attention(ch([1, 2, 3]), ch([4, 8, 20, 32, 64, 100]), ch([4, 12, 16, 32, 80]), ch([1.0, 4.0, 64.0])))
        own.append(len(layers))
        layers.append((mixer, mlp()))
    return st.config(layers, vocab, width, ch([1e-5, 1e-6]), ch([0.7, 1.0, 0.35])), ch([1, 3, 8, 33])


@pytest.mark.parametrize("seed", [0, 3, 10, 11])
def test_configurations_drawn_at_random(tmp_path, seed):
    import random

    rng = random.Random(seed)
    raw, rank = _drawn_model(rng)
    w = st.weights(raw, seed=seed, rank=rank)
    requests = {f"q{i}": np.random.default_rng(seed + i).integers(0, raw["vocab"], size=n).tolist()
                for i, n in enumerate([rng.randint(1, 45) for _ in range(3)])}
    want = {rid: plain.forward(raw, w, toks).float() for rid, toks in requests.items()}
    folder = st.write(raw, w, tmp_path / "m")
    steps = replay.mixed(requests, live=2, seed=seed, prefill_sizes=(9, 2, 17, 5), decode_tail=6)
    top = max(float(v.abs().max()) for v in want.values())
    got = replay.run_in_process(load(folder, "float32", page=8, tokens=replay.peak_tokens(steps, 8) + 8), steps)
    assert worst(got, want) <= 2e-4 * max(1.0, top), raw
    got = replay.run_in_process(load(folder, "bfloat16", page=8, tokens=replay.peak_tokens(steps, 8) + 8), steps)
    errs = np.array([float((got[k] - want[k[0]][k[1]]).pow(2).mean().sqrt()) for k in got])
    assert np.median(errs) <= 0.08 * float(torch.cat([v.flatten() for v in want.values()]).std()), raw


def test_a_layer_on_anothers_tensors_with_a_window_of_its_own(tmp_path):
    """The same tensors under another window and chunk: the engine gives each such layer parts of its own."""
    raw = st.config([(st.pair(st.windowed(2, 1, 8, 8, window=4, rot=8, scale=1.2), st.linear_attention(2, 4, 6, 4.0)), st.dense(16)),
                     (st.chunked(2, 2, 8, chunk=5, rot=4, scale=1.2), st.moe(4, 2, 8, 2.0, shared=8)), 0, 1], width=24, vocab=30)
    raw["layers"][2]["mixer"]["left"]["mask"]["size"] = 9
    raw["layers"][3]["mixer"]["mask"]["size"] = 11
    w = st.weights(raw, seed=2)
    folder = st.write(raw, w, tmp_path / "m")
    toks = np.random.default_rng(3).integers(0, 30, size=40).tolist()
    want = plain.forward(raw, w, toks).float()
    got = replay.run_in_process(load(folder, "float32"), replay.portions({"a": toks}, (7, 2, 11)))
    err = worst(got, {"a": want})
    assert err <= 2e-4 * float(want.abs().max())
    same = copy.deepcopy(raw)
    same["layers"][2]["mixer"]["left"]["mask"]["size"] = 4
    same["layers"][3]["mixer"]["mask"]["size"] = 5
    assert float((plain.forward(same, w, toks).float() - want).abs().max()) > 100 * max(err, 1e-5)

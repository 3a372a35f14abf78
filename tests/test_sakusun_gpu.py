"""Sakusun in the engine against the plain implementation (tests/plain_sakusun.py).

Small configurations with weights of their own (tests/sakusun_tiny.py).  The 32-bit engine is held to
2e-4 of the largest logit against the float64 oracle and, cut against cut, to bitwise equality (every
kernel of that path sums in an order that depends on the token's own place only); the bfloat16 engine's
error, position by position, to a fraction of the logits' spread in the bulk of the positions.  Every
engine runs with the cache's check mode on (pages that go back are overwritten) and with fewer state
slots than requests, so pages and slots are used again.
"""
import numpy as np
import pytest
import torch

import plain_sakusun as plain
import replay
import sakusun_tiny as st

pytestmark = pytest.mark.gpu

# every size differs from model to model, and some are the degenerate values: one head, heads == kv_heads, groups of
# three query heads, a window of one, no mask at all, no kept tokens, more kept tokens than the window is wide, one
# tap, two and four taps, no pair table, equal multipliers, no cap, no distance bias, a bias table of two rows, one
# blending layer only, three of them with a layer between that does not blend, layers without feed-forward, widths
# that are multiples of neither 8 nor 32, query and key/value latents of equal size
MODELS = {
    "mix": dict(layers=[(st.attention(4, 2, 16, 24, window=11, keep_first=3, v_mix=True), st.dense(48)),
                        (st.latent(3, 16, 8, 12, 20, 28), None),
                        (st.attention(4, 2, 8, 24, window=5, keep_first=0, v_mix=True, bias_rows=6, bias_max=9), st.dense(20)),
                        (st.latent(1, 8, 4, 8, 12, 12, base=300.0), st.dense(24))],
                vocab=97, width=40, eps=1e-5, scale=0.7, bigram=(53, 31, 5), taps=3, page=8),
    "odd": dict(layers=[(st.attention(3, 3, 10, 7, window=None, softcap=None, bias_max=None), st.dense(30)),
                        (st.attention(6, 2, 12, 9, window=4, keep_first=9, v_mix=True, softcap=2.0, bias_rows=2, bias_max=3), None),
                        (st.latent(2, 6, 10, 5, 9, 7, base=50.0), st.dense(10)),
                        (st.attention(1, 1, 24, 18, window=1, keep_first=2, v_mix=False, bias_rows=16, bias_max=100), None),
                        (st.attention(2, 2, 4, 9, window=7, keep_first=1, v_mix=True, bias_rows=4, bias_max=5), st.dense(12)),
                        (st.attention(3, 1, 4, 18, window=30, keep_first=5, v_mix=True, bias_rows=10, bias_max=23.5), None)],
                vocab=61, width=36, eps=1e-6, scale=1.0, bigram=None, taps=2, page=16),
    # sizes that the tensor-core kernels take in bfloat16 (multiples of 16 and 32 throughout)
    "even": dict(layers=[(st.latent(4, 32, 16, 32, 64, 32), st.dense(128)),
                         (st.attention(8, 2, 32, 64, window=44, keep_first=10, v_mix=True, bias_rows=32, bias_max=60), st.dense(64)),
                         (st.latent(2, 64, 32, 16, 32, 96), None),
                         (st.attention(4, 4, 64, 32, window=70, keep_first=33, bias_rows=12, bias_max=200), st.dense(64))],
                 vocab=80, width=64, eps=1e-6, scale=0.5, bigram=(7, 3, 3), taps=4, page=16),
}
LENGTHS = {"mix": [1, 2, 9, 23, 40, 77], "odd": [3, 30, 64, 51], "even": [150, 70, 90]}


def build(m):
    return st.config(m["layers"], m["vocab"], m["width"], m["eps"], m["scale"], m["bigram"], m["taps"])


@pytest.fixture(scope="module")
def made(tmp_path_factory):
    root = tmp_path_factory.mktemp("sakusun")
    out = {}
    for k, (name, m) in enumerate(MODELS.items()):
        raw, rows = build(m)
        w = st.weights(raw, rows, seed=5 + k, sharp=3.0)
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
        # (a model without a windowed layer gives no page back before a request ends: the pool holds every live request)
        pool = replay.peak_tokens(steps, m["page"]) + m["page"]
        eng = engine(made, name, "float32", pool).engine
        got = replay.run_in_process(eng, steps)
        assert len(got) == sum(len(t) for t in m["requests"].values())
        assert worst(got, m["want"]) <= 2e-4 * max(1.0, top), cut
        results[cut] = got
        assert not eng.cache.live
    for cut, got in results.items():
        for key, row in got.items():
            assert torch.equal(row, results["whole"][key]), (cut, key)
    assert engine(made, name, "float32", replay.peak_tokens(cuts(m["requests"], 3)["mixed"], m["page"]) + m["page"]) \
        .engine.cache.pages_poisoned > 0


@pytest.mark.parametrize("name", list(MODELS))
def test_every_cut_in_bfloat16_stays_near_the_oracle(made, name):
    m = made[name]
    spread = float(torch.cat([v.flatten() for v in m["want"].values()]).std())
    for cut, steps in cuts(m["requests"], live=3).items():
        eng = engine(made, name, "bfloat16", replay.peak_tokens(steps, m["page"]) + m["page"]).engine
        got = replay.run_in_process(eng, steps)
        errs = np.array([float((got[k] - m["want"][k[0]][k[1]]).pow(2).mean().sqrt()) for k in got])
        assert np.median(errs) <= 0.08 * spread, cut
        assert np.quantile(errs, 0.9) <= 0.3 * spread, cut


def one_layer(mixer, mlp, **kw):
    return st.config([(mixer, mlp)], **kw)


SINGLE = {
    "attention": one_layer(st.attention(2, 1, 8, 40, window=6, keep_first=2), None, width=24, vocab=50),
    "attention_all": one_layer(st.attention(3, 3, 8, 8, window=None), None, width=24, vocab=50, taps=0),
    "attention_wide_key": one_layer(st.attention(2, 2, 72, 8, window=50, keep_first=7), None, width=24, vocab=50, taps=1),
    "attention_wide_value": one_layer(st.attention(2, 1, 8, 200, window=9, keep_first=0), None, width=24, vocab=50),
    "attention_kept_only": one_layer(st.attention(2, 1, 8, 8, window=1, keep_first=12, bias_rows=2, bias_max=7), None, width=24, vocab=50),
    "latent": one_layer(st.latent(2, 8, 4, 40, 10, 6), None, width=24, vocab=50),
    "latent_all_rotated_wide": one_layer(st.latent(1, 2, 30, 6, 136, 3), None, width=24, vocab=50, taps=5),
    "dense": one_layer(st.latent(1, 8, 2, 8, 6, 6), st.dense(36), width=24, vocab=50, embed_scale=7.0),
    "no_pairs": one_layer(st.latent(1, 8, 2, 8, 6, 6), st.dense(8), width=24, vocab=50, bigram=None),
    "one_bucket": one_layer(st.latent(1, 8, 2, 8, 6, 6), None, width=24, vocab=50, bigram=(1, 1, 1)),
}


@pytest.mark.parametrize("kind", list(SINGLE))
def test_each_mechanism_alone(tmp_path, kind):
    from fastllm_py_b200 import Model, StepEntry

    raw, rows = SINGLE[kind]
    w = st.weights(raw, rows, seed=17, sharp=4.0)
    folder = st.write(raw, w, tmp_path / kind)
    toks = np.random.default_rng(1).integers(0, raw["vocab"], size=45).tolist()
    want = plain.forward(raw, w, toks).float()
    eng = Model.load(folder, dtype="float32", page_size=4, max_tokens=64, max_requests=2, max_batched_tokens=64,
                     max_model_len=64, cuda_graph=False, check_cache=True).engine
    eng.begin("a")
    head = eng.step([StepEntry("a", toks[:20], list(range(20)))]).cpu().clone()
    rest = [eng.step([StepEntry("a", [t], [0])]).cpu().clone() for t in toks[20:]]
    got = torch.cat([head] + rest)
    assert float((got - want).abs().max()) <= 2e-4 * max(1.0, float(want.abs().max()))


def sharp_model():
    raw, rows = st.config([(st.attention(2, 1, 16, 16, window=9, keep_first=4, v_mix=True, bias_rows=8, bias_max=30), st.dense(16)),
                           (st.latent(2, 16, 8, 16, 16, 16), None),
                           (st.attention(2, 2, 16, 8, window=17, keep_first=2, v_mix=True, bias_rows=12, bias_max=50), None)],
                          width=32, vocab=40)
    return raw, rows, st.weights(raw, rows, seed=3, sharp=8.0)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_edges_of_windows_and_of_the_kept_tokens_decide_the_output(tmp_path, dtype):
    """Attention so sharp that single keys decide a row: the oracle with every window one token wider or narrower,
    or with one kept token more or fewer, is far from the engine; the oracle itself is not.  Prompt portions and
    single tokens both cross the edges, in a pool so small that pages between the kept tokens and the window go back."""
    raw, rows, w = sharp_model()
    folder = st.write(raw, w, tmp_path / "edges")
    toks = np.random.default_rng(2).integers(0, 40, size=70).tolist()
    want = plain.forward(raw, w, toks).float()
    from fastllm_py_b200 import Model

    eng = Model.load(folder, dtype=dtype, page_size=8, max_tokens=80, max_requests=2, max_batched_tokens=64,
                     max_model_len=128, cuda_graph=False, check_cache=True).engine
    bound = 2e-4 * float(want.abs().max()) if dtype == "float32" else 0.05 * float(want.std())
    for steps in (replay.tail_decode({"a": toks}, 40), replay.portions({"a": toks}, (5, 2, 9, 3))):
        got = replay.run_in_process(eng, steps)
        if dtype == "float32":
            err = worst(got, {"a": want})
        else:
            err = float(np.median([float((got[k] - want[k[1]]).pow(2).mean().sqrt()) for k in got]))
        assert err <= bound
        for alter in ({"window": -1}, {"window": 1}, {"keep_first": -1}, {"keep_first": 1}):
            other = plain.forward(raw, w, toks, alter).float()
            if dtype == "float32":
                assert float((other - want).abs().max()) > 100 * max(err, 1e-5), alter
            else:
                assert float(np.median((other - want).pow(2).mean(dim=1).sqrt().numpy()[30:])) > 3 * bound, alter
    assert eng.cache.pages_poisoned > 0


def test_every_mechanism_shows_in_the_logits(tmp_path):
    """The oracle with one mechanism left out or misread (sink, distance bias, cap, rotary pairing, input convolution,
    residual gate, value blend, pair table) is far from the engine in 32-bit; so none of them can be missing unnoticed."""
    raw, rows = st.config([(st.attention(2, 1, 16, 16, window=20, keep_first=4, v_mix=True, softcap=1.5, bias_rows=8, bias_max=30), st.dense(16)),
                           (st.latent(2, 16, 8, 16, 16, 16), None),
                           (st.attention(2, 1, 16, 16, window=17, keep_first=2, v_mix=True, softcap=1.5, bias_rows=12, bias_max=50), None)],
                          width=32, vocab=40)
    w = st.weights(raw, rows, seed=11, sharp=3.0)
    folder = st.write(raw, w, tmp_path / "all")
    toks = np.random.default_rng(7).integers(0, 40, size=50).tolist()
    want = plain.forward(raw, w, toks).float()
    from fastllm_py_b200 import Model

    eng = Model.load(folder, dtype="float32", page_size=8, max_tokens=64, max_requests=1, max_batched_tokens=64,
                     max_model_len=64, cuda_graph=False, check_cache=True).engine
    got = replay.run_in_process(eng, replay.portions({"a": toks}, (7, 2, 13, 1, 1, 1)))
    err = worst(got, {"a": want})
    assert err <= 2e-4 * float(want.abs().max())
    for alter in ({"no_sink": True}, {"no_bias": True}, {"no_cap": True}, {"pairing": "halves"}, {"no_conv": True},
                  {"no_gate": True}, {"no_blend": True}, {"no_pairs": True}):
        other = plain.forward(raw, w, toks, alter).float()
        assert float((other - want).abs().max()) > 100 * max(err, 1e-5), alter


def test_far_keys_among_hundreds_stand_out(tmp_path):
    """One early token is made loud (its embedding row is scaled, and the windowed layer's keys are made to point
    where its queries do): a kept first token 290 positions back, beyond hundreds of keys the window has passed,
    decides the late rows of the windowed layer, and the latent layer sees every key; the engine follows the oracle
    whole, in portions and token by token, and the oracle without that token is far away."""
    raw, rows = st.config([(st.attention(2, 1, 16, 16, window=12, keep_first=5, bias_rows=8, bias_max=30), None),
                           (st.latent(2, 16, 8, 16, 16, 16), None)], width=32, vocab=40, bigram=None, taps=2)
    w = st.weights(raw, rows, seed=8, sharp=2.0)
    w["embed"] = w["embed"].float().clone()
    w["embed"][39] *= 5.0
    w["embed"] = w["embed"].to(torch.bfloat16)
    w["l0.mix.k"] = (w["l0.mix.q"].float()[:16] * 2.0).to(torch.bfloat16)
    folder = st.write(raw, w, tmp_path / "far")
    toks = np.random.default_rng(5).integers(0, 39, size=300).tolist()
    toks[3] = 39
    toks[293] = 39
    want = plain.forward(raw, w, toks).float()
    without = plain.forward(raw, w, toks[:3] + [0] + toks[4:]).float()
    from fastllm_py_b200 import Model

    eng = Model.load(folder, dtype="float32", page_size=16, max_tokens=320, max_requests=1, max_batched_tokens=512,
                     max_model_len=320, cuda_graph=False, check_cache=True).engine
    for steps in (replay.whole({"a": toks}), replay.tail_decode({"a": toks}, 20), replay.portions({"a": toks}, (64, 2, 31))):
        got = replay.run_in_process(eng, steps)
        err = worst(got, {"a": want})
        assert err <= 2e-4 * float(want.abs().max())
        assert float((without[293:] - want[293:]).abs().max()) > 100 * max(err, 1e-5)


def test_long_decoding_follows_the_oracle(made):
    """A short prompt, then 140 single tokens: windows pass over decoded tokens, pages go back, the convolution's
    kept rows and the last token are carried from step to step."""
    m = made["even"]
    toks = m["requests"]["q0"]
    eng = engine(made, "even", "float32", 256, max_requests=1).engine
    got = replay.run_in_process(eng, replay.tail_decode({"q0": toks}, 140))
    assert worst(got, m["want"]) <= 2e-4 * max(1.0, float(m["want"]["q0"].abs().max()))


def test_a_slot_used_again_starts_clean(made):
    """Two requests one after the other in an engine with a single slot equal the same requests in fresh engines,
    bit for bit: nothing of the first one's kept rows, last token or pages reaches the second."""
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
    """Model.generate (scheduler, sampler, captured decode steps, steps launched ahead of the host) against the
    oracle's greedy loop; where the oracle's two best logits are close the engine may take either."""
    m = made["mix"]
    model = engine(made, "mix", dtype, 512, max_requests=3, graph=True)
    prompts = [m["requests"]["q2"], m["requests"]["q3"], m["requests"]["q1"], m["requests"]["q4"][:20]]
    outs = model.generate(prompts, max_new_tokens=12)
    assert model.generate(prompts, max_new_tokens=12, use_graph=False) == outs          # replayed steps change nothing
    gaps = []
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
    """bin/make_model writes a folder from a configuration, bin/generate loads it by its architecture string and
    generates through the scheduler."""
    import json
    import subprocess
    import sys

    raw, _ = st.config([(st.latent(2, 16, 8, 16, 32, 32), st.dense(32)),
                        (st.attention(2, 1, 16, 32, window=20, keep_first=4, v_mix=True), st.dense(32))], width=32, vocab=64)
    (tmp_path / "config.json").write_text(json.dumps(raw))
    made_ = subprocess.run([sys.executable, str(replay.ROOT / "bin" / "make_model"), str(tmp_path / "config.json"),
                            str(tmp_path / "m"), "--seed", "4", "--std", "0.2"], capture_output=True, text=True)
    assert made_.returncode == 0 and "Sakusun" in made_.stdout, made_.stderr
    run = subprocess.run([sys.executable, str(replay.ROOT / "bin" / "generate"), str(tmp_path / "m"), "-", "9",
                          "bfloat16", "--random-prompt", "30", "--seed", "1"], capture_output=True, text=True)
    assert run.returncode == 0, run.stderr[-2000:]
    lines = run.stdout.strip().splitlines()
    assert "Sakusun: 2L width=32" in lines[0]
    assert len([int(t) for t in lines[1].split(",")]) == 9


# ------------------------------------------------------------------ kernels alone

def _scattered_cache(n_tokens, page, kv_heads, row_w, dtype, gen):
    """A request's keys and values on pages in shuffled order among pages full of 1e4."""
    n_pages = -(-n_tokens // page)
    order = torch.randperm(2 * n_pages + 3, generator=gen)[:n_pages]
    cache = torch.full((2 * n_pages + 3, kv_heads, page, row_w), 1.0e4, dtype=dtype)
    rows = torch.randn(n_tokens, kv_heads, row_w, generator=gen)
    for j in range(n_tokens):
        cache[order[j // page], :, j % page] = rows[j].to(dtype)
    return cache.cuda(), order.to(torch.int32).view(1, -1).cuda(), rows.to(dtype).double()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_attention_kernel_on_scattered_pages_with_loud_keys_at_the_edges(dtype):
    """The CUDA-core kernel against torch on pages in shuffled order: one loud key sits just inside the window, one
    just outside it, one is the last kept token and one the first that is not kept."""
    from fastllm_py_b200.native import ops
    from fastllm_py_b200.parts.sink_attention import distance_buckets

    gen = torch.Generator().manual_seed(2)
    heads, kv_heads, dim, vdim, page, n = 6, 2, 24, 40, 8, 200
    window, keep, cap, scale = 37, 6, 4.0, 0.3
    cache, table, rows = _scattered_cache(n, page, kv_heads, dim + vdim, dtype, gen)
    positions = torch.tensor([199, 150, 36, 37, 43, 5, 0], dtype=torch.int32)
    q = torch.randn(len(positions), heads * dim, generator=gen).to(dtype)
    rel = torch.randn(10, heads, generator=gen)
    sink = torch.randn(heads, generator=gen)
    buckets = distance_buckets(10, 55.0)
    out = torch.empty(len(positions), heads * vdim, dtype=dtype, device="cuda")
    # loud keys: rows at the edges of the first query's window and of the kept tokens point along its head-0 query
    for j in (199 - window + 1, 199 - window, keep - 1, keep):
        loud = q[0, :dim].double() * 3.0
        rows[j, 0, :dim] = loud
        cache[table[0, j // page].item(), 0, j % page, :dim] = loud.to(dtype).cuda()
        rows[j, 0, :dim] = loud.to(dtype).double()
    ops.sink_attention_simt(q.cuda(), out, cache, table, torch.zeros(len(positions), dtype=torch.int32, device="cuda"),
                            positions.cuda(), heads, kv_heads, dim, vdim, window, keep, scale, cap,
                            torch.tensor(buckets, dtype=torch.int32, device="cuda"), rel.cuda(), sink.cuda(), page)
    torch.cuda.synchronize()
    qd = q.double().view(-1, heads, dim)
    for t, pos in enumerate(positions.tolist()):
        seen = [j for j in range(pos + 1) if pos - j < window or j < keep]
        for h in range(heads):
            g = h // (heads // kv_heads)
            s = torch.stack([qd[t, h] @ rows[j, g, :dim] for j in seen]) * scale
            s = cap * torch.tanh(s / cap) + torch.stack([rel[buckets[min(pos - j, len(buckets) - 1)], h] for j in seen]).double()
            e = torch.exp(s - s.max())
            p = e / (e.sum() + torch.exp(sink[h].double() - s.max()))
            want = p @ torch.stack([rows[j, g, dim:] for j in seen])
            got = out[t, h * vdim:(h + 1) * vdim].double().cpu()
            tol = 2e-5 if dtype == torch.float32 else 3e-2
            assert float((got - want).abs().max()) <= tol * max(1.0, float(want.abs().max())), (t, h)


def test_tensor_core_attention_equals_the_cuda_core_kernel_on_scattered_pages():
    """A prompt portion over cached rows and a single token in one launch, pages in shuffled order; the pages between
    the kept first tokens and the earliest window hold 1e4, as pages that went back do."""
    from types import SimpleNamespace
    from fastllm_py_b200.native import ops
    from fastllm_py_b200.parts.sink_attention import distance_buckets

    gen = torch.Generator().manual_seed(9)
    for heads, kv_heads, dim, vdim, window, keep, cap in ((4, 2, 32, 64, 70, 9, 3.0), (2, 1, 64, 48, 0, 0, 0.0),
                                                          (3, 3, 16, 16, 5, 130, 1.0), (8, 2, 128, 128, 200, 64, 50.0)):
        page, n = 16, 330
        bf = torch.bfloat16
        cache, table, rows = _scattered_cache(n, page, kv_heads, dim + vdim, bf, gen)
        table = torch.cat([table, table]).contiguous()
        if window:                                                    # pages wholly between the kept tokens and every window
            first_lo = 100 - window + 1
            for pg in range(-(-keep // page), max(0, first_lo) // page):
                cache[table[0, pg].item()] = 1.0e4
        ctx, qlen = [100, 329], [150, 1]
        positions = torch.tensor(list(range(100, 250)) + [329], dtype=torch.int32)
        tok_req = torch.tensor([0] * 150 + [1], dtype=torch.int32)
        q = (torch.randn(151, heads * dim, generator=gen) * 0.5).to(bf)
        rel = torch.randn(12, heads, generator=gen)
        sink = torch.randn(heads, generator=gen)
        buckets = torch.tensor(distance_buckets(12, 300.0), dtype=torch.int32, device="cuda")
        step = SimpleNamespace(req_start=torch.tensor([0, 150, 151], dtype=torch.int32, device="cuda"),
                               req_ctx=torch.tensor(ctx, dtype=torch.int32, device="cuda"),
                               req_qlen=torch.tensor(qlen, dtype=torch.int32, device="cuda"), n_requests=2)
        got = torch.empty(151, heads * vdim, dtype=bf, device="cuda")
        want = torch.empty_like(got)
        table[1] = table[0]                                           # both requests read the same sequence's pages
        ops.sink_attention_tc(q.cuda(), got, cache, table, step, heads, kv_heads, dim, vdim, window, keep, 0.2, cap,
                              buckets, rel.cuda(), sink.cuda(), page)
        ops.sink_attention_simt(q.cuda(), want, cache, table, tok_req.cuda(), positions.cuda(), heads, kv_heads, dim, vdim,
                                window, keep, 0.2, cap, buckets, rel.cuda(), sink.cuda(), page)
        torch.cuda.synchronize()
        err = float((got.float() - want.float()).abs().max())
        assert err <= 3e-2 * max(1.0, float(want.float().abs().max())), (heads, dim, vdim, err)
        assert float(want.float().abs().max()) < 50.0                 # no poisoned row was read by either


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_split_key_kernel_for_single_tokens_equals_the_cuda_core_kernel(dtype):
    """Single tokens at several depths of one sequence (before the window leaves the kept tokens behind, just after,
    far after; at a split's first and last key), groups of one, three and eight query heads."""
    from fastllm_py_b200.native import ops
    from fastllm_py_b200.parts.sink_attention import distance_buckets

    gen = torch.Generator().manual_seed(12)
    for heads, kv_heads, dim, vdim, window, keep, cap in ((6, 2, 24, 40, 37, 6, 4.0), (8, 1, 64, 48, 150, 130, 50.0),
                                                          (2, 2, 16, 200, 0, 0, 0.0), (4, 2, 8, 8, 300, 3, 1.0)):
        page, n = 8, 700
        cache, table, _ = _scattered_cache(n, page, kv_heads, dim + vdim, dtype, gen)
        pos = [0, 1, 5, 36, 37, 43, 127, 128, 129, 255, 256, 300, 511, 640, 699]
        positions = torch.tensor(pos, dtype=torch.int32).cuda()
        tok_req = torch.zeros(len(pos), dtype=torch.int32).cuda()
        rows = torch.arange(len(pos), dtype=torch.int32).cuda()
        q = (torch.randn(len(pos), heads * dim, generator=gen) * 0.5).to(dtype).cuda()
        rel = torch.randn(12, heads, generator=gen).cuda()
        sink = torch.randn(heads, generator=gen).cuda()
        buckets = torch.tensor(distance_buckets(12, 300.0), dtype=torch.int32, device="cuda")
        n_splits, kept_splits = ops.sink_decode_splits(window, keep, 700)
        partial = torch.empty(len(pos) * heads * n_splits * (vdim + 2), device="cuda")
        got = torch.empty(len(pos), heads * vdim, dtype=dtype, device="cuda")
        want = torch.empty_like(got)
        assert ops.sink_decode_takes(heads, kv_heads, dim, vdim)
        ops.sink_decode(q, got, cache, table, tok_req, positions, rows, partial, n_splits, kept_splits, heads, kv_heads,
                        dim, vdim, window, keep, 0.2, cap, buckets, rel, sink, page)
        ops.sink_attention_simt(q, want, cache, table, tok_req, positions, heads, kv_heads, dim, vdim, window, keep, 0.2,
                                cap, buckets, rel, sink, page)
        torch.cuda.synchronize()
        err = float((got.float() - want.float()).abs().max())
        tol = 2e-5 if dtype == torch.float32 else 2e-2
        assert err <= tol * max(1.0, float(want.float().abs().max())), (heads, dim, vdim, err)


def test_distance_buckets_follow_the_oracle():
    from fastllm_py_b200.parts.sink_attention import distance_buckets

    for rows, far in ((32, 250), (8, 30), (2, 3), (10, 23.5), (16, 100), (6, 9), (64, 5000)):
        table = distance_buckets(rows, far)
        for n in range(int(far) + 40):
            assert table[min(n, len(table) - 1)] == plain.distance_row(n, rows, far), (rows, far, n)
        assert table[-1] == rows - 1 and table[0] == 0


@pytest.mark.parametrize("width, taps", [(20, 4), (18, 3), (1300, 2), (4100, 5)])
def test_block_kernels_carry_rows_from_step_to_step(width, taps):
    """input_conv + gated_norm_add over three steps of two requests with unequal portions (one of them a single
    token at a time) against a whole-sequence computation in float64; the ring is filed by position.  Widths that
    take four channels a thread and one, and rows wider than a block."""
    from types import SimpleNamespace
    from fastllm_py_b200.native import ops

    gen = torch.Generator().manual_seed(4)
    w = torch.randn(width, taps, generator=gen)
    gate_w = torch.randn(width, generator=gen)
    bias = torch.randn(width, generator=gen)
    xs = {0: torch.randn(9, width, generator=gen), 1: torch.randn(5, width, generator=gen)}
    ys = {r: torch.randn(len(x), width, generator=gen) for r, x in xs.items()}
    gs = {r: torch.randn(len(x), width, generator=gen) for r, x in xs.items()}
    ring = torch.full((4, (taps - 1) * width), 7.0e3, device="cuda")
    done = {0: 0, 1: 0}
    slots = {0: 2, 1: 0}
    for portions in ({0: 2, 1: 1}, {0: 6, 1: 1}, {0: 1, 1: 3}):
        rows, pos, req, start, qlen = [], [], [], [0], []
        for r, n in portions.items():
            rows += [(r, done[r] + i) for i in range(n)]
            pos += [done[r] + i for i in range(n)]
            req += [len(qlen)] * n
            qlen.append(n)
            start.append(start[-1] + n)
        dev = lambda v: torch.tensor(v, dtype=torch.int32, device="cuda")
        step = SimpleNamespace(positions=dev(pos), tok_req=dev(req), req_start=dev(start), req_qlen=dev(qlen),
                               req_slot=dev([slots[r] for r in portions]))
        x = torch.stack([xs[r][i] for r, i in rows]).cuda()
        h, hc = torch.empty_like(x), torch.empty_like(x)
        ops.input_conv(x, w.cuda(), taps, ring, step, h, hc)
        for k, (r, i) in enumerate(rows):
            want = xs[r][i].double().clone()
            for j in range(taps):
                s = i - taps + 1 + j
                if s >= 0:
                    want += w[:, j].double() * xs[r][s].double()
            assert torch.allclose(hc[k].double().cpu(), want, atol=1e-5), (r, i)
            assert torch.equal(h[k].cpu(), xs[r][i])
        y = torch.stack([ys[r][i] for r, i in rows]).cuda()
        g = torch.stack([gs[r][i] for r, i in rows]).cuda()
        ops.gated_norm_add(x, y, g, bias.cuda(), gate_w.cuda(), 1e-5, step, ring, taps)
        for k, (r, i) in enumerate(rows):
            z = ys[r][i].double() * torch.sigmoid(gs[r][i].double() + bias.double())
            want = xs[r][i].double() + z / torch.sqrt((z * z).mean() + 1e-5) * gate_w.double()
            assert torch.allclose(x[k].double().cpu(), want, atol=2e-5), (r, i)
        for r, n in portions.items():
            done[r] += n


def test_pair_embedding_keeps_the_last_token_of_a_request():
    from types import SimpleNamespace
    from fastllm_py_b200.native import ops

    gen = torch.Generator().manual_seed(6)
    vocab, width, buckets = 30, 12, 11
    table, pairs = torch.randn(vocab, width, generator=gen), torch.randn(buckets + 1, width, generator=gen)
    seqs = {0: [3, 29, 29, 0, 17, 4], 1: [8, 8, 1]}
    last = torch.full((3,), 123456, dtype=torch.int32, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    done = {0: 0, 1: 0}
    for portions in ({0: 1, 1: 2}, {0: 3}, {1: 1, 0: 2}):
        ids, req, start, ctx, qlen, slot = [], [], [0], [], [], []
        for r, n in portions.items():
            ids += seqs[r][done[r]:done[r] + n]
            req += [len(qlen)] * n
            ctx.append(done[r]); qlen.append(n); slot.append(2 - r); start.append(start[-1] + n)
        dev = lambda v: torch.tensor(v, dtype=torch.int32, device="cuda")
        step = SimpleNamespace(token_ids=dev(ids), tok_req=dev(req), req_start=dev(start), req_ctx=dev(ctx),
                               req_qlen=dev(qlen), req_slot=dev(slot), status=status, token_feed=None)
        out = torch.empty(len(ids), width, device="cuda")
        ops.pair_embed(table.cuda(), pairs.cuda(), out, step, last, buckets, 5, 3, 0.5)
        k = 0
        for r, n in portions.items():
            for i in range(done[r], done[r] + n):
                row = buckets if i == 0 else (seqs[r][i - 1] * 5 + seqs[r][i] * 3) % buckets
                assert torch.allclose(out[k].cpu(), table[seqs[r][i]] * 0.5 + pairs[row], atol=1e-6), (r, i)
                k += 1
            done[r] += n
    assert int(status.item()) == 0


@pytest.mark.parametrize("width", [70, 72, 2052])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_gated_norm_add_adds_up_partial_sums_like_the_reduce_kernel(dtype, width):
    """A product left as split-K slabs gives, bit for bit, what the reduce kernel followed by the plain form gives."""
    from types import SimpleNamespace
    from fastllm_py_b200.native import ops
    from fastllm_py_b200.native.gemm_tc import Partial

    gen = torch.Generator().manual_seed(9)
    n, splits, ld = 5, 3, -(-width // 4) * 4
    slabs = torch.randn(splits, n, ld, generator=gen).cuda()
    gate_slabs = torch.randn(2, n, ld, generator=gen).cuda()
    gate_part = Partial(gate_slabs, 2, n, width, ld, slabs.device, side=True)
    gate = gate_part.reduce_into(torch.empty(n, width, device="cuda", dtype=dtype))
    bias, w = torch.randn(width, generator=gen).cuda(), torch.randn(width, generator=gen).cuda()
    dev = lambda v: torch.tensor(v, dtype=torch.int32, device="cuda")
    step = SimpleNamespace(positions=dev(list(range(n))), tok_req=dev([0] * n), req_start=dev([0, n]), req_qlen=dev([n]),
                           req_slot=dev([0]))
    x0 = torch.randn(n, width, generator=gen).cuda()
    part = Partial(slabs, splits, n, width, ld, slabs.device)
    y = torch.empty(n, width, device="cuda", dtype=dtype)
    part.reduce_into(y)
    a, b, c = x0.clone(), x0.clone(), x0.clone()
    ops.gated_norm_add(a, y, gate, bias, w, 1e-6, step)
    ops.gated_norm_add(b, part, gate, bias, w, 1e-6, step)
    ops.gated_norm_add(c, part, gate_part, bias, w, 1e-6, step, dtype=dtype)
    assert torch.equal(a, b) and torch.equal(a, c)
    z = slabs.double().sum(0)[:, :width].to(dtype).double() * torch.sigmoid(gate.double() + bias.double())
    want = x0.double() + z / torch.sqrt((z * z).mean(-1, keepdim=True) + 1e-6) * w.double()
    assert torch.allclose(a.double(), want, atol=2e-5 if dtype == torch.float32 else 2e-2)


def test_gate_in_the_per_head_product_equals_the_gate_kernel():
    from fastllm_py_b200.native import ops

    gen = torch.Generator().manual_seed(10)
    n, heads, k, vd = 70, 3, 64, 40
    a = torch.randn(n, heads * k, generator=gen).cuda().bfloat16()
    w = (torch.randn(heads, vd, k, generator=gen) / 8).cuda().bfloat16()
    wide = torch.randn(n, 16 + heads * vd, generator=gen).cuda().bfloat16()
    gate = wide[:, 16:]                                       # a column block of a wider buffer, as in the mixer
    plain_out, fused = torch.empty(n, heads * vd, device="cuda", dtype=torch.bfloat16), torch.empty(n, heads * vd, device="cuda", dtype=torch.bfloat16)
    ops.gemm_batched(a, k, w, plain_out, vd)
    ops.sigmoid_gate(plain_out, gate)
    ops.gemm_batched(a, k, w, fused, vd, gate=gate)
    assert torch.equal(plain_out, fused)
    want = torch.einsum("nhk,hvk->nhv", a.double().view(n, heads, k), w.double()).reshape(n, -1) * torch.sigmoid(gate.double())
    assert torch.allclose(fused.double(), want, atol=3e-2, rtol=2e-2)

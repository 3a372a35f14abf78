"""Sakusun without a GPU: configuration, plan, cache needs, the manager's kept first pages, and the oracle's own
properties (causality, windows, kept tokens, the sink, the pair table)."""
import copy

import numpy as np
import pytest
import torch

import plain_sakusun as plain
import sakusun_tiny as st
from fastllm_py_b200.cache import CacheManager
from fastllm_py_b200.cache.needs import FixedState, PagedKeysValues, PagedRows
from fastllm_py_b200.config import ConfigError, SakusunConfig
from fastllm_py_b200.config.registry import architecture_of
from fastllm_py_b200.parts import BuildContext, Decoder


def sample():
    return st.config([(st.attention(4, 2, 16, 24, window=11, keep_first=3, v_mix=True, bias_rows=6, bias_max=9), st.dense(48)),
                      (st.latent(3, 16, 8, 12, 20, 28), None),
                      (st.attention(2, 1, 16, 48, window=5, keep_first=0, v_mix=True), st.dense(20)),
                      (st.attention(2, 2, 4, 4, window=None, softcap=None, bias_max=None), None)],
                     vocab=97, width=40, taps=3)


def plan_of(raw, rows=None):
    arch = architecture_of(raw)
    cfg = arch.config_class.from_hf(raw)
    shapes = None if rows is None else st.tensor_shapes(raw, rows)
    return cfg, arch.make_plan(cfg, None if shapes is None else set(shapes), tensor_shapes=shapes)


def test_configuration_round_trip_and_summary():
    raw, _ = sample()
    cfg = SakusunConfig.from_hf(raw)
    assert SakusunConfig.from_hf(cfg.to_hf()) == cfg
    assert cfg.to_hf() == raw
    assert cfg.taps == 3 and cfg.bigram_buckets == 53 and cfg.layers[0].mixer.keep_first == 3
    assert cfg.layers[3].mixer.window is None and cfg.layers[3].mixer.softcap is None
    assert "Sakusun: 4L width=40" in cfg.summary()
    bare, _ = st.config([(st.latent(), None)], bigram=None, taps=0)
    cfg = SakusunConfig.from_hf(bare)
    assert cfg.bigram_buckets is None and cfg.taps == 0 and cfg.to_hf() == bare


@pytest.mark.parametrize("change, word", [
    (lambda r: r["layers"][0]["mixer"].update(kv_heads=3), "kv_heads"),
    (lambda r: r["layers"][1]["mixer"]["rot"].update(dims=6), "rot.dims"),
    (lambda r: r["layers"][1]["mixer"].update(rot_dim=7, rot={"base": 10.0, "dims": 7}), "even"),
    (lambda r: r["layers"][0].update(type="conv"), "not a mixer"),
    (lambda r: r["layers"][0]["mlp"].update(kind="moe"), "kind"),
    (lambda r: r["layers"][2]["mixer"].update(vdim=5), "v_mix"),
    (lambda r: r["layers"][1]["mixer"].pop("q_rank"), "q_rank"),
    (lambda r: r.pop("norm"), "norm"),
    (lambda r: r["embedding"]["bigram"].pop("buckets"), "buckets"),
    (lambda r: r.update(layers=[]), "layers"),
])
def test_configuration_refusals_name_the_key(change, word):
    raw, _ = sample()
    raw = copy.deepcopy(raw)
    change(raw)
    with pytest.raises(ConfigError) as e:
        SakusunConfig.from_hf(raw)
    assert word in str(e.value)


def test_plan_names_every_tensor_and_reads_the_bias_rows_from_the_shapes():
    raw, rows = sample()
    cfg, plan = plan_of(raw, rows)
    shapes = st.tensor_shapes(raw, rows)
    dec = Decoder(plan, BuildContext(torch.device("cpu"), torch.bfloat16, 16, 64))
    expected = dec.expected_tensors()
    unused = {"l0.mix.vmix"}                                         # the blend's source stores a number nobody reads
    assert set(expected) == set(shapes) - unused
    assert all(tuple(expected[k]) == tuple(shapes[k]) for k in expected)
    assert set(plan.ignorable) >= unused
    assert set(plan.tensor_names()) == set(expected)
    assert plan.layers[0].mixer.params["bias_rows"] == 6 and plan.layers[2].mixer.params["bias_rows"] == 8
    assert [layer.mixer.params.get("v_mix") for layer in plan.layers] == ["source", None, "blend", None]
    assert plan.layers[1].mixer.params["pairing"] == "interleaved" and plan.layers[1].mixer.params["q_rank"] == 28
    assert plan.layers[3].mixer.params["bias_rows"] is None and plan.layers[3].mixer.params["window"] is None


def test_cache_needs_pages_for_the_mixers_and_state_for_block_and_embedding():
    raw, rows = sample()
    _, plan = plan_of(raw, rows)
    needs = Decoder(plan, BuildContext(torch.device("cpu"), torch.bfloat16, 16, 64)).cache_needs()
    assert needs[0] == PagedKeysValues(2, 16, 24, 11, 3)
    assert needs[1] == PagedRows(20 + 8, None)
    assert needs[2] == PagedKeysValues(1, 16, 48, 5, 0)
    assert needs[3] == PagedKeysValues(2, 4, 4, None, 0)
    assert needs[("block", 0)] == FixedState((2 * 2 * 40,), "float32")      # two sublayers, taps - 1 rows each
    assert needs[("block", 1)] == FixedState((1 * 2 * 40,), "float32")      # no feed-forward: one sublayer
    assert needs[Decoder.EMBEDDING_STATE] == FixedState((1,), "int32")
    bare, rows = st.config([(st.latent(), None)], bigram=None, taps=1)
    _, plan = plan_of(bare, rows)
    needs = Decoder(plan, BuildContext(torch.device("cpu"), torch.bfloat16, 16, 64)).cache_needs()
    assert set(needs) == {0}                                         # one tap keeps no rows; no pair table, no last token


def test_pages_of_the_kept_first_tokens_never_go_back():
    """A window of 10 with 5 kept tokens in pages of 4: pages 0 and 1 stay (they hold tokens 0..4), the pages between
    them and the window go back as the window passes, and everything goes back at the end."""
    need = PagedKeysValues(1, 8, 8, 10, 5)
    cm = CacheManager({0: need, 1: PagedKeysValues(1, 8, 8, 10, 0)}, page_size=4, num_pages=16, max_requests=2,
                      max_pages_per_request=16)
    rc = cm.admit("a")
    for n in (3, 9, 1, 1, 20, 2, 1):
        cm.extend(rc, n)
        cm.commit(rc, n)
        cm.check()
        first_needed = rc.seq_len - 10 + 1
        kept = rc.tables[cm.group_of[0]]
        plain_window = rc.tables[cm.group_of[1]]
        for page in range(-(-rc.seq_len // 4)):
            wholly_behind = (page + 1) * 4 <= first_needed
            assert (plain_window[page] < 0) == wholly_behind
            assert (kept[page] < 0) == (wholly_behind and page >= 2)
    assert rc.seq_len == 37 and cm.groups[cm.group_of[0]].pool.held_pages == 2 + 3
    cm.release("a")
    assert all(g.pool.free_pages == 16 for g in cm.groups)


def test_random_weights_folder_reads_back(tmp_path):
    from fastllm_py_b200.weights import SafetensorsStore
    from fastllm_py_b200.weights.loader import check_store, write_model_folder

    raw, _ = sample()
    cfg = SakusunConfig.from_hf(raw)
    folder = write_model_folder(cfg, tmp_path / "m", seed=3)
    store = SafetensorsStore(folder)
    names = set(store.names())
    shapes = {n: tuple(store.describe(n)[0]) for n in names}
    arch = architecture_of(raw)
    plan = arch.make_plan(cfg, names, tensor_shapes=shapes)
    dec = Decoder(plan, BuildContext(torch.device("cpu"), torch.bfloat16, 16, 64))
    check_store(dec.expected_tensors(), store, "m", plan.ignorable)
    assert shapes["l0.norm1"] == () and shapes["final.norm"] == ()


# ------------------------------------------------------------------ the oracle's own properties

def small():
    raw, rows = st.config([(st.attention(2, 1, 8, 8, window=6, keep_first=2, v_mix=True, bias_rows=4, bias_max=7), st.dense(16)),
                           (st.latent(2, 8, 4, 8, 8, 8), None),
                           (st.attention(2, 1, 8, 8, window=9, keep_first=0, v_mix=True), None)], width=16, vocab=30)
    return raw, st.weights(raw, rows, seed=2, sharp=3.0)


def test_oracle_is_causal_and_each_mechanism_moves_it():
    raw, w = small()
    toks = np.random.default_rng(0).integers(0, 30, size=40).tolist()
    full = plain.forward(raw, w, toks)
    assert torch.allclose(plain.forward(raw, w, toks[:25]), full[:25], atol=1e-12)
    for alter in ({"window": 1}, {"keep_first": -1}, {"no_sink": True}, {"no_bias": True}, {"pairing": "halves"},
                  {"no_conv": True}, {"no_gate": True}, {"no_blend": True}, {"no_pairs": True}):
        assert float((plain.forward(raw, w, toks, alter) - full).abs().max()) > 1e-3, alter


def test_oracle_window_and_kept_tokens():
    """With one layer, changing a token outside both the window and the kept range leaves a late row alone; changing
    the last kept token or the window's first token moves it.  (The input convolution reaches taps - 1 tokens
    further back and the pair table one: the changed tokens keep clear of that.)"""
    raw, rows = st.config([(st.attention(2, 1, 8, 8, window=6, keep_first=3, bias_rows=4, bias_max=7), None)], width=16, vocab=30)
    w = st.weights(raw, rows, seed=4, sharp=3.0)
    toks = np.random.default_rng(1).integers(0, 29, size=30).tolist()
    base = plain.forward(raw, w, toks)[29]

    def moved(j):
        other = list(toks)
        other[j] = 29
        return float((plain.forward(raw, w, other)[29] - base).abs().max())

    assert moved(2) > 1e-4 and moved(24) > 1e-4                      # last kept token; first token of the window
    assert moved(3 + 3) == 0.0 and moved(24 - 4) == 0.0            # beyond the kept range's reach; before the window's


def test_oracle_sink_takes_weight_without_a_value():
    raw, rows = st.config([(st.attention(1, 1, 8, 8, window=None, bias_max=None, softcap=None), None)], width=16, vocab=30,
                          taps=0, bigram=None)
    w = st.weights(raw, rows, seed=6)
    toks = [5, 9, 11]
    h = plain.embed(raw, w, toks, {})
    with_sink = plain.sink_attention(h, w, "l0.mix.", raw["layers"][0]["mixer"], 1e-5, [None], {})
    without = plain.sink_attention(h, w, "l0.mix.", raw["layers"][0]["mixer"], 1e-5, [None], {"no_sink": True})
    # first token: one key, so without a sink its weight is 1; with the sink it is 1 / (1 + exp(sink - score))
    ratio = with_sink[0] / without[0]
    assert torch.allclose(ratio, ratio[0].expand_as(ratio), atol=1e-9) and 0.0 < float(ratio[0]) < 1.0


def test_oracle_pair_rows_and_distance_rows():
    assert plain.pair_rows([3, 4, 4], 11, 5, 3) == [11, (15 + 12) % 11, (20 + 12) % 11]
    assert [plain.distance_row(n, 8, 30) for n in (0, 3, 4, 29, 30, 500)] == [0, 3, 4, 7, 7, 7]
    assert plain.distance_row(7, 8, 30) == 4 + int(np.floor(np.log(7 / 4) / np.log(30 / 4) * 4))

"""Saberax without a GPU: configuration keys, the plan of parts, cache needs, the rotary tables, the
random-weights folder, and the plain implementation's own properties (what the GPU tests lean on)."""
import copy
import json

import numpy as np
import pytest
import torch

import plain_saberax as plain
import saberax_tiny as st
from fastllm_py_b200.architectures.saberax import make_plan
from fastllm_py_b200.cache.needs import FixedState, PagedKeysValues
from fastllm_py_b200.config import ConfigError, load_config
from fastllm_py_b200.config.saberax import SaberaxConfig
from fastllm_py_b200.parts import BuildContext, Decoder, PartSpec, build_part
from fastllm_py_b200.weights import write_model_folder

YARN = (4.0, 64, 8.0, 1.0)
BANDS = (8.0, 64, 1.0, 4.0)
RAW = st.config([(st.pair(st.normed(4, 2, 16, 24, q_temp=(0.25, 8)), st.recurrent(24, 3, 4)), st.dense(48)),
                 (st.pair(st.windowed(6, 2, 12, 20, window=11, rot=8, scaling=YARN), st.linear_attention(3, 8, 12, 8.0)),
                  st.moe(6, 2, 24, 2.5, groups=(3, 2), shared=16)),
                 (st.chunked(3, 3, 10, chunk=13, rot=10, scaling=BANDS), None),
                 0,
                 (st.chunked(2, 1, 8, chunk=None, rot=None), st.moe(4, 4, 8, 1.0, shared=None))], vocab=97, width=40)


def decoder(raw, page=8, rank=6):
    cfg = SaberaxConfig.from_hf(raw)
    plan = make_plan(cfg, None, tensor_shapes=st.tensor_shapes(raw, rank))
    return cfg, Decoder(plan, BuildContext(torch.device("cpu"), torch.float32, page, 64))


def test_config_reads_back_and_names_every_tensor():
    cfg, dec = decoder(RAW)
    assert cfg.to_hf() == RAW
    assert SaberaxConfig.from_hf(json.loads(json.dumps(cfg.to_hf()))) == cfg
    assert dec.expected_tensors() == st.tensor_shapes(RAW)
    assert "Saberax" in cfg.summary()
    assert len(dec.blocks) == 4 and [run.layer for run in dec.order] == [0, 1, 2, 0, 3]    # a layer on another's tensors
    assert dec.blocks[0].scale == 0.7
    # the decay's inner size comes from the checkpoint's shapes
    _, other = decoder(RAW, rank=11)
    assert other.expected_tensors()["l1.mix.right.a1"] == (11, 40)


def test_cache_needs_follow_the_layers():
    _, dec = decoder(RAW)
    needs = dec.cache_needs()
    assert needs[(0, "left")] == PagedKeysValues(2, 16, 24, None)           # every earlier token: nothing may go back
    assert needs[(0, "right")] == FixedState((24 * 4,), "float32")          # the state and three kept inputs per channel
    assert needs[(1, "left")] == PagedKeysValues(2, 12, 20, 11)
    assert needs[(1, "right")] == FixedState((3 * 12 * 8,), "float32")
    assert needs[2] == PagedKeysValues(3, 10, 10, 13)                       # behind a chunk's start nothing is seen again
    assert needs[(3, "left")] == needs[(0, "left")] and needs[(3, "right")] == needs[(0, "right")]   # a cache of its own
    assert needs[4] == PagedKeysValues(1, 8, 8, None)
    assert dec.blocks[3].mixer.position is None                             # no rotation: no tables
    assert set(needs) == {(0, "left"), (0, "right"), (1, "left"), (1, "right"), 2, (3, "left"), (3, "right"), 4}


@pytest.mark.parametrize("path,value,word", [
    (("layers", 0, "type"), "conv", "type"),
    (("layers", 0, "mixer", "left", "kv_heads"), 3, "kv_heads"),
    (("layers", 0, "mixer", "right", "blocks"), 5, "blocks"),
    (("layers", 0, "mixer", "left", "q_temp", "every"), 0, "every"),
    (("layers", 1, "mixer", "left", "rot", "dims"), 7, "rot.dims"),
    (("layers", 1, "mixer", "left", "rot", "dims"), 18, "rot.dims"),
    (("layers", 1, "mixer", "left", "rot", "scaling", "factor"), "big", "factor"),
    (("layers", 1, "mixer", "right", "tau"), 0, "tau"),
    (("layers", 2, "mixer", "vdim"), 12, "vdim"),
    (("layers", 2, "mixer", "rot", "scaling", "high"), 1.0, "low and high"),
    (("layers", 1, "mlp", "router", "top"), 7, "top"),
    (("layers", 1, "mlp", "router", "groups", "count"), 4, "groups"),
    (("layers", 1, "mlp", "router", "groups", "keep"), 4, "groups"),
    (("layers", 1, "mlp", "kind"), "sparse", "kind"),
    (("layers", 0, "mlp", "ff"), None, "ff"),
    (("layers", 3, "weights_of"), 3, "weights_of"),
    (("layers", 3, "weights_of"), 1, "another kind"),
    (("width",), "wide", "width"),
])
def test_wrong_values_are_refused_by_name(path, value, word):
    raw = copy.deepcopy(RAW)
    at = raw
    for key in path[:-1]:
        at = at[key]
    at[path[-1]] = value
    with pytest.raises(ConfigError, match=word):
        SaberaxConfig.from_hf(raw)


def test_a_written_folder_loads_by_its_architecture_string(tmp_path):
    cfg = SaberaxConfig.from_hf(RAW)
    folder = write_model_folder(cfg, tmp_path / "m", seed=3)
    arch, again = load_config(folder)
    assert arch.name == "Saberax" and again == cfg
    from safetensors import safe_open

    with safe_open(str(folder / "model.safetensors"), framework="pt") as f:
        assert {k: tuple(f.get_slice(k).get_shape()) for k in f.keys()} == st.tensor_shapes(RAW, rank=16)


@pytest.mark.parametrize("scaling", [None, ("yarn",) + YARN, ("yarn", 6.0, 1024, 16.0, 2.0), ("bands",) + BANDS,
                                     ("bands", 4.0, 512, 1.0, 4.0)])
def test_rotary_tables_follow_the_scaling(scaling):
    """The position part's tables against the oracle's frequencies (written apart from it)."""
    base = 700.0 if scaling is None or scaling[0] == "yarn" else 250000.0
    spec = PartSpec("rotary", dict(rot_dim=12, theta=base, scaling=scaling, exact=True))
    part = build_part("position", spec, BuildContext(torch.device("cpu"), torch.float32, 8, 300))
    cos, sin = part.tables()
    raw = None
    if scaling is not None:
        names = ("factor", "original", "fast", "slow") if scaling[0] == "yarn" else ("factor", "original", "low", "high")
        raw = dict(zip(names, scaling[1:]))
    f, gain = plain.rotary_frequencies(12, base, raw)
    ang = torch.arange(300, dtype=torch.float64)[:, None] * f[None, :]
    assert np.allclose(cos.numpy(), (torch.cos(ang) * gain).numpy(), atol=1e-6)
    assert np.allclose(sin.numpy(), (torch.sin(ang) * gain).numpy(), atol=1e-6)
    if scaling is not None:
        plain_f, _ = plain.rotary_frequencies(12, base, None)
        assert float((f / plain_f).min()) < 0.9 and float((f / plain_f).max()) == 1.0   # slow pairs stretched, fast ones kept
        if scaling[0] == "bands":                                  # all three bands occur
            ratio = (f / plain_f).tolist()
            assert any(r == 1.0 for r in ratio) and any(abs(r - 1 / scaling[1]) < 1e-12 for r in ratio)
            assert gain == 1.0


def test_plain_implementation_is_causal_and_its_masks_states_and_groups_matter():
    raw = st.config([(st.pair(st.normed(2, 1, 8, 8, q_temp=(0.5, 4)), st.recurrent(12, 2, 3)), st.moe(6, 2, 8, 2.0, groups=(3, 1))),
                     (st.pair(st.windowed(2, 1, 8, 8, window=4, rot=8, scale=1.5), st.linear_attention(2, 4, 6, 4.0)), st.dense(16)),
                     (st.chunked(2, 2, 8, chunk=5, rot=4, scale=1.5), None)], width=24, vocab=30)
    w = st.weights(raw, seed=1, slow=True)
    toks = list(range(3, 26))
    full = plain.forward(raw, w, toks)
    assert torch.allclose(plain.forward(raw, w, toks[:11]), full[:11], atol=1e-12)
    for alter, first in (("wider", 4), ("narrower", 3)):
        other = plain.forward(raw, w, toks, alter={alter})
        assert float((other - full)[6:].abs().max()) > 1e-3
        assert torch.allclose(other[:first], full[:first], atol=1e-12)                  # the first tokens see all either way
    for alter in ("no_sink", "no_gate", "no_temp", "other_pairing"):
        assert float((plain.forward(raw, w, toks, alter={alter}) - full).abs().max()) > 1e-3, alter
    moved = plain.forward(raw, w, [toks[0] + 1] + toks[1:])
    assert float((moved - full)[-1].abs().max()) > 1e-6                                 # the states reach back
    free = copy.deepcopy(raw)
    free["layers"][0]["mlp"]["router"]["groups"]["keep"] = 3
    assert float((plain.forward(free, w, toks) - full).abs().max()) > 1e-3              # the groups limit the choice
    # states handed on equal whole sequences
    h = torch.randn(17, 24, dtype=torch.float64, generator=torch.Generator().manual_seed(2))
    t = plain.sub(w, "l0.mix.right.")
    whole, _ = plain.gated_recurrence(h, t, raw["layers"][0]["mixer"]["right"])
    head, state = plain.gated_recurrence(h[:6], t, raw["layers"][0]["mixer"]["right"])
    rest, _ = plain.gated_recurrence(h[6:], t, raw["layers"][0]["mixer"]["right"], state)
    assert torch.allclose(torch.cat([head, rest]), whole, atol=1e-12)
    t = plain.sub(w, "l1.mix.right.")
    whole, _ = plain.gated_linear_attention(h, t, raw["layers"][1]["mixer"]["right"], 1e-5)
    head, state = plain.gated_linear_attention(h[:9], t, raw["layers"][1]["mixer"]["right"], 1e-5)
    rest, _ = plain.gated_linear_attention(h[9:], t, raw["layers"][1]["mixer"]["right"], 1e-5, state)
    assert torch.allclose(torch.cat([head, rest]), whole, atol=1e-12)


def test_routing_oracle_keeps_to_the_groups_with_the_best_pairs():
    h = torch.randn(50, 16, dtype=torch.float64, generator=torch.Generator().manual_seed(0))
    router = torch.randn(12, 16, dtype=torch.float64, generator=torch.Generator().manual_seed(1))
    correction = torch.randn(12, dtype=torch.float64, generator=torch.Generator().manual_seed(2)) * 0.5
    chosen, w = plain.route(h, router, correction, {"experts": 12, "top": 3, "scale": 2.5, "groups": {"count": 4, "keep": 2}})
    pick = torch.sigmoid(h @ router.T) + correction
    pairs = pick.view(50, 4, 3).sort(dim=-1).values[..., 1:].sum(dim=-1)
    differs = 0
    for t in range(50):
        kept = set(pairs[t].topk(2).indices.tolist())
        assert {e // 3 for e in chosen[t].tolist()} <= kept
        differs += kept != set(pick.view(50, 4, 3).max(dim=-1).values[t].topk(2).indices.tolist())
    assert differs > 0                                     # the sum of two is not the best one
    assert torch.allclose(w.sum(dim=-1), torch.full((50,), 2.5, dtype=torch.float64))


def test_a_layer_on_anothers_tensors_may_differ_in_its_constants():
    """The same tensors under another window: parts of its own over the same names, a run of its own."""
    raw = st.config([(st.pair(st.windowed(2, 1, 8, 8, window=4, rot=8), st.linear_attention(2, 4, 6, 4.0)), st.dense(16)), 0],
                    width=24, vocab=30)
    raw["layers"][1]["mixer"]["left"]["mask"]["size"] = 9
    cfg, dec = decoder(raw)
    assert cfg.to_hf() == raw and len(dec.blocks) == 2 and [run.layer for run in dec.order] == [0, 1]
    assert dec.expected_tensors() == st.tensor_shapes(raw)
    assert dec.blocks[0].mixer.left.window == 4 and dec.blocks[1].mixer.left.window == 9
    w = st.weights(raw, seed=2)
    toks = list(range(2, 22))
    same = copy.deepcopy(raw)
    same["layers"][1]["mixer"]["left"]["mask"]["size"] = 4
    assert float((plain.forward(raw, w, toks) - plain.forward(same, w, toks)).abs().max()) > 1e-4

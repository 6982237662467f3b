"""Pabavik without a GPU: its config reader, model description and checkpoint names, and the engine's
step, cache, state and batching logic with the plain PyTorch statements of the kernels
(tests/kernel_refs.py) standing in for the CUDA kernels."""

import copy
import json
import os

import numpy as np
import pytest
import torch

import kernel_refs
from helpers import make_engine, mixed_schedule, model_folder, replay_cuts, replay_mixed, replay_whole, tokens_for
from plain import pabavik_plain as plain_model
from plain.pabavik_plain import PlainPabavik
from tiny_pabavik import ALL, PABA_1, PABA_3, PAGE

from freetoken_b200.engine.build import describe_model, typed_config
from freetoken_b200.engine.engine import StepEntry
from freetoken_b200.errors import ConfigError
from freetoken_b200.models.pabavik import cache_windows
from freetoken_b200.parts.gla import chunk_list
from freetoken_b200.registry import architecture_of

TOL = dict(rtol=1e-4, atol=2e-5)


@pytest.fixture
def cpu_ops(monkeypatch):
    kernel_refs.install(monkeypatch)


# --------------------------------------------------------------------------- config, description, names
def test_the_cache_outlives_the_owners_window_when_a_reader_looks_farther():
    cfg = architecture_of(PABA_1).parse_config(PABA_1)
    assert cache_windows(cfg) == {1: 20}  # the owner's window is 9, its readers' 20 and 5
    _, _, spec, _ = describe_model(PABA_1)
    assert [e.cache_from for e in spec.schedule] == [None, None, 1, None, 1]
    assert spec.layers[1].mixer["cache_window"] == 20 and spec.layers[1].mixer["window"] == 9
    assert spec.layers[2].mixer["window"] == 20 and not spec.layers[2].mixer["own_kv"]
    cfg = architecture_of(PABA_3).parse_config(PABA_3)
    assert cache_windows(cfg) == {0: 300, 3: 11}


def test_config_errors_name_the_key():
    def broken(path, value, delete=False):
        raw = copy.deepcopy(PABA_1)
        d = raw
        for k in path[:-1]:
            d = d[k]
        if delete:
            del d[path[-1]]
        else:
            d[path[-1]] = value
        return raw

    for raw, word in [
        (broken(["vocab"], None, True), "vocab"),
        (broken(["layers", 1, "mixer", "kv_heads"], 3), "kv_heads"),
        (broken(["layers", 0, "type"], "conv"), "type"),
        (broken(["layers", 1, "mlp", "router", "top"], 9), "top"),
        (broken(["layers", 0, "mlp", "kind"], "dense"), "kind"),
        (broken(["layers", 2, "mixer", "kv_from"], 0), "kv_from"),  # layer 0 is no attention layer
        (broken(["layers", 2, "mixer", "kv_from"], 2), "kv_from"),  # not an earlier layer
        (broken(["layers", 4, "mixer", "kv_from"], 2), "kv_from"),  # layer 2 has no keys of its own
        (broken(["layers", 2, "mixer", "vdim"], 16), "kv_from"),  # other sizes than the owner's
        (broken(["layers", 1, "mixer", "rot", "dims"], 7), "rot.dims"),
        (broken(["layers", 1, "mixer", "mask", "size"], 0), "mask.size"),
        (broken(["layers", 0, "mixer", "tau"], 0.0), "tau"),
        (broken(["norm"], {}), "eps"),
        (broken(["logit_softcap"], -1.0), "logit_softcap"),
    ]:
        with pytest.raises(ConfigError, match=word):
            architecture_of(raw).parse_config(raw)


def test_names_shapes_and_the_decay_rank_from_the_file(tmp_path_factory):
    folder = model_folder(tmp_path_factory.getbasetemp(), "P1", PABA_1)
    from safetensors import safe_open

    with safe_open(os.path.join(folder, "model.safetensors"), framework="pt") as f:
        names = set(f.keys())
        assert {"embed", "head", "final.norm", "l0.norm1", "l0.norm1b", "l0.norm2", "l0.norm2b", "l0.mix.q", "l0.mix.k",
                "l0.mix.v", "l0.mix.g", "l0.mix.a1", "l0.mix.a2", "l0.mix.a2.b", "l0.mix.norm", "l0.mix.o", "l1.mix.q",
                "l1.mix.k", "l1.mix.v", "l1.mix.g", "l1.mix.o", "l1.mix.q.norm", "l1.mix.k.norm", "l2.mix.q", "l2.mix.g",
                "l2.mix.q.norm", "l0.mlp.e0.gate", "l0.mlp.e4.down", "l0.mlp.router", "l0.mlp.router.b",
                "l0.mlp.shared.gate", "l0.mlp.shared.up", "l0.mlp.shared.down"} <= names
        assert not any(n.startswith(("l2.mlp", "l2.norm2", "l2.mix.k", "l2.mix.v")) for n in names)
        assert f.get_tensor("l0.mix.a1").shape == (8, 64) and f.get_tensor("l0.mix.a2").shape == (32, 8)
        assert f.get_tensor("l1.mix.v").shape == (64, 64) and f.get_tensor("l1.mix.g").shape == (128, 64)
        assert f.get_tensor("l1.mix.k.norm").shape == (16,) and f.get_tensor("l0.mix.norm").shape == (24,)
    raw = json.load(open(os.path.join(folder, "config.json")))
    for l in raw["layers"]:  # a config that does not say how wide the low-rank decay projection is: the file does
        l["mixer"].pop("decay_rank", None)
    typed = typed_config(architecture_of(raw), raw, folder)
    assert [l.mixer.decay_rank for l in typed.layers if l.type == "gla"] == [8, 4]


def test_chunk_lists():
    chunks, per_seg, single, multi = chunk_list([(1, 9), (130, 130), (64, 200), (65, 65)], 64)
    assert per_seg.tolist() == [[0, 1], [1, 3], [4, 1], [5, 2]] and single and multi
    assert chunks.tolist() == [[0, 0, 1, 0], [1, 0, 64, 0], [1, 64, 64, 1], [1, 128, 2, 2], [2, 0, 64, 0], [3, 0, 64, 0],
                               [3, 64, 1, 1]]
    assert chunk_list([(1, 5), (1, 1)], 64)[2:] == (True, False)


# --------------------------------------------------------------------------- the plain model's own mechanisms
def test_the_plain_recurrence_is_the_sum_it_stands_for():
    """o_t = sum_{s <= t} (q_t . (k_s * prod_{s < r <= t} a_r)) v_s, written out for one head."""
    torch.manual_seed(0)
    T, D, Dv, W = 7, 6, 5, 12
    h = torch.randn(T, W, dtype=torch.float64)
    m = {"heads": 1, "dim": D, "vdim": Dv, "tau": 3.0}
    w = {n: torch.randn(*s, dtype=torch.float64) * 0.5 for n, s in
         dict(q=(D, W), k=(D, W), v=(Dv, W), g=(Dv, W), a1=(2, W), a2=(D, 2), o=(W, Dv)).items()}
    w["a2.b"], w["norm"] = torch.randn(D, dtype=torch.float64), torch.ones(Dv, dtype=torch.float64)
    got = plain_model.gated_linear_attention(h, w, m, 1e-5)
    q, k, v = h @ w["q"].T * D ** -0.5, h @ w["k"].T, h @ w["v"].T
    a = torch.sigmoid((h @ w["a1"].T) @ w["a2"].T + w["a2.b"]) ** (1 / 3.0)
    o = torch.zeros(T, Dv, dtype=torch.float64)
    for t in range(T):
        for s in range(t + 1):
            o[t] += (q[t] * k[s] * a[s + 1:t + 1].prod(0)).sum() * v[s]
    o = o / torch.sqrt((o * o).mean(-1, keepdim=True) + 1e-5)
    g = h @ w["g"].T
    torch.testing.assert_close(got, (o * g * torch.sigmoid(g)) @ w["o"].T)


def test_the_plain_router_takes_the_softmax_over_the_chosen_logits_only():
    h = torch.tensor([1.0, 0.0], dtype=torch.float64)
    router = torch.tensor([[0.0, 0.0], [2.0, 0.0], [1.0, 0.0], [2.0, 0.0]], dtype=torch.float64)
    ids, ps = plain_model.route(h, router, torch.tensor([0.5, 0.0, 1.5, 0.0], dtype=torch.float64), 3)
    assert ids == [2, 1, 3]  # 2.5, then the tie of 2.0 by index
    e = torch.exp(torch.tensor([2.5, 2.0, 2.0], dtype=torch.float64))
    torch.testing.assert_close(ps, e / e.sum())


# --------------------------------------------------------------------------- the engine on the CPU
@pytest.mark.parametrize("name", ["P1", "P2", "P3", "P4", "P5", "P6"])
def test_cuts_and_batches_agree_with_the_plain_model(name, cpu_ops, tmp_path_factory):
    folder = model_folder(tmp_path_factory.getbasetemp(), name, ALL[name])
    plain = PlainPabavik(folder)
    eng = make_engine(folder, "float32", "cpu", PAGE[name], pages=40)
    toks = tokens_for(plain.vocab, 70, 11)
    ref = plain.logits(toks).float()
    assert float(ref.std()) > 0.3, "the random model's logits are meant to spread"
    torch.testing.assert_close(replay_whole(eng, "w", toks), ref, **TOL)
    torch.testing.assert_close(replay_cuts(eng, "d", toks, [38]), ref, **TOL)  # last 32 one by one
    torch.testing.assert_close(replay_cuts(eng, "c", toks, [7, 2, 13, 2, 5, 3, 2, 11, 2]), ref, **TOL)
    torch.testing.assert_close(replay_cuts(eng, "one", toks[:20], []), ref[:20], **TOL)  # from the first token on, one by one
    eng.cache.check()
    assert all(g.pool.free_count == g.pool.num_pages for g in eng.cache.paged)


@pytest.mark.parametrize("name", ["P1", "P3"])
def test_mixed_steps_with_few_pages_and_slots(name, cpu_ops, tmp_path_factory):
    folder = model_folder(tmp_path_factory.getbasetemp(), name, ALL[name])
    plain = PlainPabavik(folder)
    lengths = {"r0": 45, "r1": 60, "r2": 38, "r3": 52, "r4": 41, "r5": 47}
    seqs = {r: tokens_for(plain.vocab, n, i) for i, (r, n) in enumerate(lengths.items())}
    P = PAGE[name]
    eng = make_engine(folder, "float32", "cpu", P, pages=4 * (-(-64 // P)))
    got = replay_mixed(eng, seqs, mixed_schedule(lengths, seed=3))
    for r, toks in seqs.items():
        torch.testing.assert_close(got[r], plain.logits(toks).float(), **TOL)
    for g in eng.cache.paged:
        assert g.pool.handed_out > g.pool.num_pages, "the trace was meant to use pages again"
        assert g.pool.free_count == g.pool.num_pages
    assert eng.cache.slots.free_count == 4  # six requests went through four state slots


def test_a_state_slot_that_is_used_again_starts_from_zero(cpu_ops, tmp_path_factory):
    folder = model_folder(tmp_path_factory.getbasetemp(), "P5", ALL["P5"])
    plain = PlainPabavik(folder)
    eng = make_engine(folder, "float32", "cpu", 8, pages=16, reqs=1)  # one slot: every request gets the same one
    a, b = tokens_for(plain.vocab, 30, 1), tokens_for(plain.vocab, 12, 2)
    replay_cuts(eng, "a", a, [17])
    state = eng.cache.state[0].tensors["s"]
    assert float(state[:, 1].abs().max()) > 0  # the first request left its state behind
    torch.testing.assert_close(replay_cuts(eng, "b", b, [1, 4]), plain.logits(b).float(), **TOL)


def test_the_plain_model_notices_a_window_one_token_off_a_missing_sink_and_a_lost_state(tmp_path_factory):
    """Negative control for the tolerances above: one constant off moves the logits far beyond them."""
    folder = model_folder(tmp_path_factory.getbasetemp(), "P1", PABA_1)
    toks = tokens_for(200, 60, 5)
    ref = PlainPabavik(folder).logits(toks)
    other = PlainPabavik(folder)
    other.cfg["layers"][2]["mixer"]["mask"]["size"] = 19
    assert float((other.logits(toks) - ref).abs().max()) > 100 * TOL["atol"]
    other = PlainPabavik(folder)
    other.cfg["layers"][3]["mixer"]["tau"] = 15.0
    assert float((other.logits(toks) - ref).abs().max()) > 100 * TOL["atol"]
    other = PlainPabavik(folder)
    other.cfg["layers"][0]["mlp"]["shared"]["limit"] = 0.6
    assert float((other.logits(toks) - ref).abs().max()) > 100 * TOL["atol"]


def plain_for_the_command_line(folder):
    """The plain model as the command line's tests take one: ``cfg.vocab`` and float32 ``logits``."""
    from types import SimpleNamespace

    plain = PlainPabavik(folder)
    return SimpleNamespace(cfg=SimpleNamespace(vocab=plain.vocab), logits=lambda toks: plain.logits(toks).float())


def test_the_command_line_makes_a_model_generates_and_replays(tmp_path, capsys, cpu_ops):
    from test_cli import generate_and_replay, make_model

    folder = make_model(tmp_path, PABA_1, capsys)
    generate_and_replay(folder, "cpu", "float32", capsys, tmp_path, plain_for_the_command_line(folder))

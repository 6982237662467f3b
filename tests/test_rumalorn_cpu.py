"""Rumalorn without a GPU: its config reader, model description, checkpoint names and tables, and the
engine's step, cache and batching logic with the plain PyTorch statements of the kernels
(tests/kernel_refs.py) standing in for the CUDA kernels."""

import copy
import json
import os

import pytest
import torch

import kernel_refs
from helpers import make_engine, mixed_schedule, model_folder, replay_cuts, replay_mixed, replay_whole, tokens_for
from plain.rumalorn_plain import PlainRumalorn, distance_bucket, query_temperature
from tiny_rumalorn import ALL, RUMA_1, RUMA_3, RUMA_4

from freetoken_b200.engine.build import describe_model, typed_config
from freetoken_b200.errors import ConfigError
from freetoken_b200.models.rumalorn import layer_passes
from freetoken_b200.parts import BuildEnv, Workspace
from freetoken_b200.parts.rope import LogTemperature
from freetoken_b200.parts.tied_attention import distance_buckets
from freetoken_b200.config.spec import PartSpec
from freetoken_b200.registry import architecture_of

TOL = dict(rtol=1e-4, atol=2e-5)
PAGE = {"R1": 4, "R2": 8, "R3": 4, "R4": 16, "R6": 8, "R7": 4}


@pytest.fixture
def cpu_ops(monkeypatch):
    kernel_refs.install(monkeypatch)


# --------------------------------------------------------------------------- tables and config
@pytest.mark.parametrize("B,D", [(8, 20), (16, 240), (12, 50), (6, 7.5), (4, 12), (32, 128), (2, 3), (64, 100000)])
def test_distance_buckets_are_the_plain_formula(B, D):
    table = distance_buckets(B, D)
    assert table[-1] == B - 1 and all(b < B - 1 for b in table[:-1])
    for n, b in enumerate(table):
        assert b == distance_bucket(n, B, D), (n, b)
    for n in (len(table), len(table) + 1, 10 * len(table), 1 << 20):  # everything farther lands in the last bucket
        assert distance_bucket(n, B, D) == B - 1
    assert table[: B // 2] == list(range(B // 2))
    assert all(x <= y for x, y in zip(table, table[1:]))


@pytest.mark.parametrize("coef,every", [(0.4, 4), (0.15, 1), (1.0, 16), (0.05, 100)])
def test_temperature_table(coef, every):
    cpu = torch.device("cpu")
    env = BuildEnv(dtype=torch.float32, device=cpu, max_seq_len=300, max_step_tokens=1, workspace=Workspace(cpu))
    t = LogTemperature(PartSpec("log_temperature", dict(coef=coef, every=every)), env).scale_table()
    assert t.shape == (300,) and t.dtype == torch.float32
    want = torch.tensor([query_temperature(p, coef, every) for p in range(300)], dtype=torch.float64)
    torch.testing.assert_close(t.double(), want, rtol=1e-7, atol=0)
    assert float(t[0]) == (1.0 if every > 1 else float(torch.tensor(1 + coef * 0.6931471805599453).float()))


def test_the_order_of_layers():
    order = lambda raw: [(l, e, v) for l, e, v in layer_passes(architecture_of(raw).parse_config(raw))]  # noqa: E731
    assert order(RUMA_1) == [(0, False, None), (1, False, 0), (2, False, None), (1, True, 1), (2, False, None),
                             (1, True, 2), (2, False, None), (3, False, None)]
    assert order(RUMA_3) == [(0, False, 0), (1, False, None), (0, True, 1), (1, False, None)]
    assert order(RUMA_4) == [(0, False, None), (1, False, 0), (2, False, None)]
    raw = copy.deepcopy(RUMA_1)
    del raw["loop"]
    assert order(raw) == [(l, False, None) for l in range(4)]
    _, _, spec, expected = describe_model(raw)
    assert spec.pass_vectors is None and not any(n.startswith("loop") for n in expected)
    _, _, spec, expected = describe_model(RUMA_1)
    assert expected["loop.step"].shape == (3, 64)
    assert [e.cache_from for e in spec.schedule] == [None] * 8  # every pass owns a cache


def test_config_errors_name_the_key():
    def broken(path, value, delete=False):
        raw = copy.deepcopy(RUMA_1)
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
        (broken(["layers", 0, "mixer", "vdim"], 8), "vdim"),
        (broken(["layers", 0, "type"], "conv"), "type"),
        (broken(["layers", 1, "mlp", "router", "top"], 9), "top"),
        (broken(["layers", 0, "mlp", "kind"], "sparse"), "kind"),
        (broken(["loop", "stop"], 7), "loop"),
        (broken(["layers", 2, "mixer", "q_temp"], None, True), "q_temp"),
    ]:
        with pytest.raises(ConfigError, match=word):
            architecture_of(raw).parse_config(raw)


def test_names_shapes_and_table_rows_from_the_file(tmp_path_factory):
    folder = model_folder(tmp_path_factory.getbasetemp(), "R1", RUMA_1)
    from safetensors import safe_open

    with safe_open(os.path.join(folder, "model.safetensors"), framework="pt") as f:
        names = set(f.keys())
        assert {"embed", "head", "final.norm", "final.norm.b", "final.norm.alpha", "loop.step", "l0.norm1", "l0.norm1.b",
                "l0.norm1.alpha", "l0.mix.q", "l0.mix.q.b", "l0.mix.k", "l0.mix.k.b", "l0.mix.g", "l0.mix.rel", "l0.mix.o",
                "l0.mix.o.b", "l0.mlp.gate", "l0.mlp.up", "l0.mlp.down", "l1.mlp.e0.gate", "l1.mlp.e3.down", "l1.mlp.table",
                "l3.mlp.e4.up"} <= names
        assert not any(n.startswith("l2.mlp") for n in names)
        assert f.get_tensor("l0.mix.rel").shape == (8, 4) and f.get_tensor("l1.mlp.table").shape == (200, 2)
        table = f.get_tensor("l1.mlp.table")
        assert table.dtype == torch.int32 and int(table.min()) >= 0 and int(table.max()) < 4
        assert bool((table[:, 0] != table[:, 1]).all())
    # a config that does not say how many rows the bias tables have: the file's header does
    raw = json.load(open(os.path.join(folder, "config.json")))
    for l in raw["layers"]:
        del l["mixer"]["buckets"]
    arch = architecture_of(raw)
    assert typed_config(arch, raw, folder).rel_buckets == (8, 8, 8, 8)


# --------------------------------------------------------------------------- the engine on the CPU
@pytest.mark.parametrize("name", ["R1", "R2", "R3", "R4", "R6", "R7"])
def test_cuts_and_batches_agree_with_the_plain_model(name, cpu_ops, tmp_path_factory):
    folder = model_folder(tmp_path_factory.getbasetemp(), name, ALL[name])
    plain = PlainRumalorn(folder)
    eng = make_engine(folder, "float32", "cpu", PAGE[name], pages=40)
    toks = tokens_for(plain.vocab, 70, 11)
    ref = plain.logits(toks).float()
    torch.testing.assert_close(replay_whole(eng, "w", toks), ref, **TOL)
    torch.testing.assert_close(replay_cuts(eng, "d", toks, [38]), ref, **TOL)  # last 32 one by one
    torch.testing.assert_close(replay_cuts(eng, "c", toks, [7, 2, 13, 2, 5, 3, 2, 11, 2]), ref, **TOL)
    eng.cache.check()
    assert all(g.pool.free_count == g.pool.num_pages for g in eng.cache.paged)


@pytest.mark.parametrize("name", ["R1", "R3"])
def test_mixed_steps_with_few_pages(name, cpu_ops, tmp_path_factory):
    folder = model_folder(tmp_path_factory.getbasetemp(), name, ALL[name])
    plain = PlainRumalorn(folder)
    lengths = {"r0": 45, "r1": 60, "r2": 38, "r3": 52, "r4": 41, "r5": 47}
    seqs = {r: tokens_for(plain.vocab, n, i) for i, (r, n) in enumerate(lengths.items())}
    P = PAGE[name]
    eng = make_engine(folder, "float32", "cpu", P, pages=4 * (-(-64 // P)))
    got = replay_mixed(eng, seqs, mixed_schedule(lengths, seed=3))
    for r, toks in seqs.items():
        torch.testing.assert_close(got[r], plain.logits(toks).float(), **TOL)
    pool = eng.cache.paged[0].pool
    assert pool.handed_out > pool.num_pages, "the trace was meant to use pages again"
    assert pool.free_count == pool.num_pages


def test_the_plain_model_notices_a_shifted_bucket_edge_and_a_changed_temperature(tmp_path_factory):
    """Negative control for the tolerances above: one constant off moves the logits far beyond them."""
    folder = model_folder(tmp_path_factory.getbasetemp(), "R1", RUMA_1)
    toks = tokens_for(200, 60, 5)
    ref = PlainRumalorn(folder).logits(toks)
    for key, value in (("bias_max", 26), ("q_temp", {"coef": 0.4, "every": 5})):
        other = PlainRumalorn(folder)
        for l in other.cfg["layers"]:
            l["mixer"][key] = value
        assert float((other.logits(toks) - ref).abs().max()) > 100 * TOL["atol"], key


def plain_for_the_command_line(folder):
    """The plain model as the command line's tests take one: ``cfg.vocab`` and float32 ``logits``."""
    from types import SimpleNamespace

    plain = PlainRumalorn(folder)
    return SimpleNamespace(cfg=SimpleNamespace(vocab=plain.vocab), logits=lambda toks: plain.logits(toks).float())


def test_the_command_line_makes_a_model_generates_and_replays(tmp_path, capsys, cpu_ops):
    from test_cli import generate_and_replay, make_model

    folder = make_model(tmp_path, RUMA_1, capsys)
    generate_and_replay(folder, "cpu", "float32", capsys, tmp_path, plain_for_the_command_line(folder))

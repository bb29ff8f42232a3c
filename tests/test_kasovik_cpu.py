"""Kasovik without a GPU: configuration, weight names, and the engine's host side (batch layout, cache entries and
per-request state of layers that share weights, scheduler) with the CPU twins of the kernels (tests/ref_kernels.py)
against the plain implementation (tests/plain_kasovik.py)."""
from __future__ import annotations

import copy
import json

import pytest
import torch

import plain_kasovik as plain
from helpers import random_prompt
from holon_b200.config.registry import ConfigError, resolve_architecture
from holon_b200.replay import Replayer
from kasovik_tools import CONFIGS, compare, exact_logits, make_folder, read_folder, stored_config, tensor_table
from ref_kernels import RefKernels
from replay_tools import portions, run


def test_architecture_and_configuration():
    arch = resolve_architecture(CONFIGS["a"])
    cfg = arch.parse(CONFIGS["a"])
    assert arch.name == "Kasovik" and len(cfg.layers) == 4 and cfg.pairs.buckets == 97
    assert [cfg.owner(i) for i in range(4)] == [0, 1, 0, 1]
    spec = arch.recipe(cfg)
    assert [(r.layer, r.cache, r.fills) for r in spec.order] == [(0, 0, True), (1, 1, True), (0, 2, True), (1, 3, True)]
    assert spec.layers[2] is None and spec.layers[3] is None and spec.layers[1].ffn is None
    assert spec.layers[0].block.name == "parallel" and spec.layers[0].mixer.name == "side_by_side"
    later = arch.recipe(arch.parse(CONFIGS["b"]))                       # a layer may run with a later layer's weights
    assert [(r.layer, r.cache) for r in later.order] == [(0, 0), (2, 1), (2, 2)]
    for path, value, error in (
            (("layers", 2, "weights_of"), 2, ConfigError),                  # itself
            (("layers", 2, "weights_of"), 1, ConfigError),                  # a layer of another kind
            (("layers", 2, "mixer", "left", "heads"), 8, ConfigError),      # differs from the layer whose weights it uses
            (("layers", 0, "type"), "latent", NotImplementedError),
            (("layers", 0, "mlp", "kind"), "moe", NotImplementedError),
            (("layers", 1, "mixer", "rot", "dims"), 34, ConfigError),
            (("layers", 1, "mixer", "decay"), [0.9], ConfigError),
            (("layers", 0, "mixer", "left", "kv_heads"), 3, ConfigError),
            (("layers", 0, "mixer", "left", "vdim"), 16, ConfigError),      # the values are the keys
            (("embedding", "bigram", "buckets"), 0, ConfigError)):
        c = copy.deepcopy(CONFIGS["a"])
        at = c
        for key in path[:-1]:
            at = at[key]
        at[path[-1]] = value
        with pytest.raises(error):
            arch.parse(c)
    c = stored_config(CONFIGS["a"])                                      # the ranks come from the tensors' shapes
    with pytest.raises(ConfigError):
        arch.parse(c)
    done = arch.complete(c, {"l0.mix.right.a1": (8, 64), "l0.mix.right.g1": (12, 64)})
    assert arch.parse(done) == cfg and "decay_rank" not in c["layers"][0]["mixer"]["right"]


@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_tensor_names_and_shapes(name):
    from holon_b200.weights import RandomSource
    table = {stored: tuple(shape) for stored, shape, _ in RandomSource(CONFIGS[name], 0).table()}
    assert table == dict(tensor_table(CONFIGS[name]))


def test_a_missing_and_a_misshapen_tensor_are_named(tmp_path):
    from safetensors.torch import load_file, save_file
    from holon_b200.weights.loader import WeightError
    folder = make_folder(tmp_path, "a")
    tensors = load_file(str(folder / "model.safetensors"))
    del tensors["l0.mix.left.sink"]
    tensors["l0.mix.right.v.conv"] = tensors["l0.mix.right.v.conv"][:, :3].contiguous()
    tensors["l2.norm1"] = tensors["l0.norm1"].clone()                     # layer 2 runs with layer 0's weights: it has none
    save_file(tensors, str(folder / "model.safetensors"))
    with pytest.raises(WeightError) as e:
        Replayer(str(folder), "float32", 64, device="cpu", kernels=RefKernels())
    assert e.value.missing == ["l0.mix.left.sink"] and e.value.unexpected == ["l2.norm1"]
    assert [s[0] for s in e.value.shapes] == ["l0.mix.right.v.conv"]


@pytest.fixture(scope="module", params=sorted(CONFIGS))
def model(request, tmp_path_factory):
    folder = make_folder(tmp_path_factory.mktemp("models"), request.param, seed=5)
    config = CONFIGS[request.param]
    prompts = {f"r{i}": random_prompt(config["vocab"], n, 80 + i) for i, n in enumerate((23, 41, 9, 30))}
    return folder, config, prompts, {rid: exact_logits(folder, ids) for rid, ids in prompts.items()}


def test_every_run_has_a_cache_entry_and_state_of_its_own(model):
    folder, config, _, _ = model
    r = Replayer(str(folder), "float32", 64, device="cpu", kernels=RefKernels(), page_size=4)
    runs = len(config["layers"])
    windows = [i for i, layer in enumerate(config["layers"]) if layer["type"] == "parallel"]
    assert [e.entry for e in r.built.model.entries] == [-1, *range(runs)]          # (-1: the embedding's previous token)
    assert sorted(e for g in r.built.cache.groups for e in g.entries) == windows
    states = r.built.cache.slot_states
    assert states[(-1, "previous")].dtype == torch.int32
    for i, layer in enumerate(config["layers"]):
        m = layer["mixer"]
        if layer["type"] == "retention":
            assert tuple(states[(i, "state")].shape[1:]) == (m["heads"], m["vdim"], m["dim"])
        else:
            right = m["right"]
            assert tuple(states[(i, "right.state")].shape[1:]) == (right["heads"], right["vdim"], right["dim"])
            assert ((i, "right.conv") in states) == (right["conv"] > 1)
    assert r.built.cache.prefix is None                   # a state of fixed size cannot be entered in the middle of a prompt


def test_whole_tail_portions_and_mixed(model):
    folder, config, prompts, want = model
    r = Replayer(str(folder), "float32", 64, device="cpu", kernels=RefKernels(), page_size=4)
    compare(run(r, [([(rid, ids)], [rid]) for rid, ids in prompts.items()]), want, "float32")
    steps = []
    for rid, ids in prompts.items():                                       # a portion, then one by one
        steps.append(([(rid, ids[:5])], []))
        steps += [([(rid, [t])], [rid] if i == len(ids) - 6 else []) for i, t in enumerate(ids[5:])]
    compare(run(r, steps), want, "float32")
    steps = []
    for rid, ids in prompts.items():                                       # from the first token on, one by one
        steps += [([(rid, [t])], [rid] if i == len(ids) - 1 else []) for i, t in enumerate(ids)]
    compare(run(r, steps), want, "float32")
    steps = []
    for rid, ids in prompts.items():
        parts = portions(ids, [3, 2, 7, 2, 5])
        steps += [([(rid, p)], [rid] if i == len(parts) - 1 else []) for i, p in enumerate(parts)]
    compare(run(r, steps), want, "float32")
    # four requests at once in 104 tokens of pool: portions beside single tokens, pages and slots given back and used
    # again (a slot's state, carried inputs and previous token must not leak into the request that takes it next)
    r = Replayer(str(folder), "float32", 104, device="cpu", kernels=RefKernels(), page_size=4)
    at, steps, sizes = {rid: 0 for rid in prompts}, [], {"r0": [1, 1, 4], "r1": [6, 2, 1], "r2": [2], "r3": [1, 9]}
    live, waiting, turn = ["r0", "r1", "r2"], ["r3"], 0
    while live:
        entries, end = [], []
        for rid in list(live):
            n = min(sizes[rid][turn % len(sizes[rid])], len(prompts[rid]) - at[rid])
            entries.append((rid, prompts[rid][at[rid]:at[rid] + n]))
            at[rid] += n
            if at[rid] == len(prompts[rid]):
                end.append(rid)
                live.remove(rid)
                if waiting:
                    live.append(waiting.pop())
        steps.append((entries, end))
        turn += 1
    got = run(r, steps)
    assert len(got) == sum(map(len, prompts.values())) and not r.built.cache.live
    compare(got, want, "float32")
    again = run(r, steps)                                                  # the same slots once more, now used before
    compare(again, want, "float32")


def test_a_request_left_out_of_steps_goes_on_later(model):
    folder, config, prompts, want = model
    r = Replayer(str(folder), "float32", 128, device="cpu", kernels=RefKernels(), page_size=8)
    a, b = prompts["r1"], prompts["r3"]
    steps = [([("r1", a[:7])], []), ([("r3", b[:2])], []), ([("r3", b[2:19])], []), ([("r1", a[7:9]), ("r3", b[19:20])], []),
             ([("r1", a[9:])], ["r1"]), ([("r3", b[20:])], ["r3"])]
    compare(run(r, steps), want, "float32")


def test_greedy_generation_through_the_scheduler(model):
    from holon_b200.engine import Engine, EngineConfig, SamplingParams
    folder, config, prompts, _ = model
    stored, weights = read_folder(folder)
    engine = Engine(EngineConfig(model=str(folder), dtype="float32", device="cpu", page_size=4, max_seqs=3, max_model_len=64,
                                 max_step_tokens=16, state_memory=1 << 22, prefix_cache=True, cuda_graphs=False),
                    kernels=RefKernels())
    asked = [prompts["r0"], prompts["r2"], prompts["r0"][:12] + prompts["r1"][:7], prompts["r3"]]
    with torch.inference_mode():
        got = engine.generate(asked, SamplingParams(temperature=0.0, max_tokens=6, ignore_eos=True))
    for prompt, tokens in zip(asked, got):
        ids = list(prompt)
        for token in tokens:
            logits = plain.forward(weights, stored, ids)[-1]
            best = int(logits.argmax())
            second = float(logits.topk(2).values[1])
            assert token == best or float(logits[best]) - second < 1e-3, (len(ids), token, best)
            ids.append(token)


def test_the_command_line_serves_the_design(tmp_path, capsys, monkeypatch):
    """`random-model` writes a folder with every tensor of the design, `models` lists it, and `generate` produces the
    plain implementation's greedy tokens (on the CPU, with the plain kernel table in the CUDA kernels' place)."""
    import holon_b200.engine as engine_module
    from holon_b200 import cli

    class CpuEngine(engine_module.Engine):
        def __init__(self, config):
            config.device, config.state_memory = "cpu", 1 << 22
            super().__init__(config, kernels=RefKernels())
    monkeypatch.setattr(engine_module, "Engine", CpuEngine)
    config = tmp_path / "config.json"
    config.write_text(json.dumps(CONFIGS["a"]))
    assert cli.main(["random-model", str(config), str(tmp_path / "m"), "--seed", "3"]) == 0
    folder = capsys.readouterr().out.strip()
    stored, weights = read_folder(folder)
    assert set(weights) == {name for name, _ in tensor_table(CONFIGS["a"])}
    assert cli.main(["models"]) == 0
    assert "Kasovik" in capsys.readouterr().out.split()
    assert cli.main(["generate", folder, "--prompt-ids", "5,17,3,44,9", "--max-tokens", "4", "--dtype", "float32", "--max-model-len",
                     "64", "--max-seqs", "2", "--max-step-tokens", "32", "--page-size", "8", "--ignore-eos"]) == 0
    out = json.loads(capsys.readouterr().out.splitlines()[0])
    ids = [5, 17, 3, 44, 9]
    for token in out["token_ids"]:
        logits = plain.forward(weights, stored, ids)[-1]
        assert token == int(logits.argmax()) or float(logits.max() - logits[token]) < 1e-4
        ids.append(token)
    assert len(out["token_ids"]) == 4


class _Faulty(RefKernels):
    """The plain kernel table with one fault planted: the comparisons above must notice each of them."""

    def __init__(self, fault: str) -> None:
        self.fault = fault

    def paged_attention(self, out, q, kv, block_table, rows, scale, window, sinks=None):
        if self.fault == "no_sink":
            sinks = None
        if self.fault == "window_one_more" and window > 0:
            window += 1
        if self.fault == "window_one_less" and window > 1:
            window -= 1
        super().paged_attention(out, q, kv, block_table, rows, scale, window, sinks)

    def conv_carry(self, conv_state, first, channels, taps, rows):
        if self.fault != "inputs_not_carried":
            super().conv_carry(conv_state, first, channels, taps, rows)

    def embed_pair(self, out, table, scale, pair, ids, positions, rows, prev, mul_prev, mul_cur, buckets):
        keep = prev.clone()
        super().embed_pair(out, table, scale, pair, ids, positions, rows, prev, mul_prev, mul_cur, buckets)
        if self.fault == "previous_token_not_carried":
            prev.copy_(keep)

    def recurrent_scan(self, out, qk, v, decay, head_decay, beta, state, rows):
        keep = state.clone()
        super().recurrent_scan(out, qk, v, decay, head_decay, beta, state, rows)
        if self.fault == "state_not_written":
            state.copy_(keep)

    def sum_into(self, h, terms, bias=None):
        super().sum_into(h, terms, None if self.fault == "no_output_bias" else bias)


@pytest.mark.parametrize("fault", ["none", "no_sink", "window_one_more", "window_one_less", "inputs_not_carried",
                                   "previous_token_not_carried", "state_not_written", "no_output_bias"])
def test_planted_faults_are_noticed(tmp_path, fault):
    folder = make_folder(tmp_path, "a", seed=5)
    ids = random_prompt(CONFIGS["a"]["vocab"], 41, 81)
    want = {"x": exact_logits(folder, ids)}
    r = Replayer(str(folder), "float32", 64, device="cpu", kernels=_Faulty(fault), page_size=4)
    parts = portions(ids, [3, 2, 7, 1, 5])
    got = run(r, [([("x", p)], ["x"] if i == len(parts) - 1 else []) for i, p in enumerate(parts)])
    if fault == "none":
        compare(got, want, "float32")
    else:
        with pytest.raises(AssertionError):
            compare(got, want, "float32")

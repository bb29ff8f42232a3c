"""Rulorax without a GPU: configuration, weight names, and the engine's host side (batch layout, the cache entries
that layers share, scheduler) with the CPU twins of the kernels (tests/ref_kernels.py) against the plain
implementation (tests/plain_rulorax.py)."""
from __future__ import annotations

import copy

import pytest
import torch

import plain_rulorax as plain
from helpers import random_prompt
from holon_b200.config.registry import ConfigError, resolve_architecture
from holon_b200.replay import Replayer
from ref_kernels import RefKernels
from replay_tools import portions, run
from rulorax_tools import CONFIGS, compare, exact_logits, make_folder, tensor_table


def test_architecture_and_configuration():
    arch = resolve_architecture(CONFIGS["a"])
    cfg = arch.parse(CONFIGS["a"])
    assert arch.name == "Rulorax" and cfg.streams == 3 and len(cfg.layers) == 4
    assert cfg.layers[1].mixer.kv_from == 0 and cfg.layers[3].experts is None and cfg.layers[3].dense_ff is None
    spec = arch.recipe(cfg)
    assert [(r.layer, r.cache, r.fills) for r in spec.order] == [(0, 0, True), (1, 0, False), (2, 2, True), (3, 2, False)]
    assert spec.layers[3].ffn is None and spec.layers[0].block.name == "hyper"
    assert arch.recipe(arch.parse(CONFIGS["c"])).layers[0].block.name == "prenorm"
    for path, value, error in (
            (("layers", 1, "mixer", "kv_from"), 2, ConfigError),            # a later layer
            (("layers", 3, "mixer", "kv_from"), 1, ConfigError),            # a layer that has no latent of its own
            (("layers", 1, "mixer", "kv_rank"), 16, ConfigError),           # another rank than the layer it reads
            (("layers", 0, "type"), "windowed", NotImplementedError),
            (("layers", 2, "mlp", "router", "top"), 7, ConfigError),
            (("layers", 0, "mixer", "rot", "dims"), 18, ConfigError),
            (("streams",), 0, ConfigError)):
        c = copy.deepcopy(CONFIGS["a"])
        at = c
        for key in path[:-1]:
            at = at[key]
        at[path[-1]] = value
        with pytest.raises(error):
            arch.parse(c)
    c = copy.deepcopy(CONFIGS["a"])
    del c["layers"][0]["mixer"]["scale"]
    with pytest.raises(ConfigError):
        arch.parse(c)


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
    del tensors["l1.mlp.e3.down"]
    tensors["l2.hc2.mix"] = tensors["l2.hc2.mix"][:2].contiguous()
    tensors["l1.mix.dkv"] = tensors["l0.mix.dkv"].clone()                 # layer 1 reads layer 0's latent: it has none
    save_file(tensors, str(folder / "model.safetensors"))
    with pytest.raises(WeightError) as e:
        Replayer(str(folder), "float32", 64, device="cpu", kernels=RefKernels())
    assert e.value.missing == ["l1.mlp.e3.down"] and e.value.unexpected == ["l1.mix.dkv"]
    assert [s[0] for s in e.value.shapes] == ["l2.hc2.mix"]


@pytest.fixture(scope="module", params=sorted(CONFIGS))
def model(request, tmp_path_factory):
    folder = make_folder(tmp_path_factory.mktemp("models"), request.param, seed=3)
    config = CONFIGS[request.param]
    prompts = {f"r{i}": random_prompt(config["vocab"], n, 60 + i) for i, n in enumerate((23, 41, 9, 30))}
    return folder, config, prompts, {rid: exact_logits(folder, ids) for rid, ids in prompts.items()}


def test_layers_share_cache_entries(model):
    folder, config, _, _ = model
    r = Replayer(str(folder), "float32", 64, device="cpu", kernels=RefKernels(), page_size=4)
    own = [i for i, layer in enumerate(config["layers"]) if "kv_from" not in layer["mixer"]]
    assert [e.entry for e in r.built.model.entries] == own
    assert sum(len(g.entries) for g in r.built.cache.groups) == len(own)
    for g in r.built.cache.groups:
        assert tuple(g.kv.shape[2:]) == (4, g.decl.rank + g.decl.rot_dim)


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
    for rid, ids in prompts.items():
        parts = portions(ids, [3, 2, 7, 2, 5])
        steps += [([(rid, p)], [rid] if i == len(parts) - 1 else []) for i, p in enumerate(parts)]
    compare(run(r, steps), want, "float32")
    # four requests at once in 104 tokens of pool: portions beside single tokens, pages given back and used again
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


def test_greedy_generation_through_the_scheduler(model):
    from holon_b200.engine import Engine, EngineConfig, SamplingParams
    folder, config, prompts, _ = model
    _, weights = plain.read_folder(folder)
    engine = Engine(EngineConfig(model=str(folder), dtype="float32", device="cpu", page_size=4, max_seqs=3, max_model_len=64,
                                 max_step_tokens=16, state_memory=1 << 22, prefix_cache=True, cuda_graphs=False),
                    kernels=RefKernels())
    asked = [prompts["r0"], prompts["r2"], prompts["r0"][:12] + prompts["r1"][:7], prompts["r3"]]
    with torch.inference_mode():
        got = engine.generate(asked, SamplingParams(temperature=0.0, max_tokens=6, ignore_eos=True))
    for prompt, tokens in zip(asked, got):
        ids = list(prompt)
        for token in tokens:
            logits = plain.forward(config, weights, ids)[-1]
            best = int(logits.argmax())
            second = float(logits.topk(2).values[1])
            assert token == best or float(logits[best]) - second < 1e-3, (len(ids), token, best)
            ids.append(token)


def test_the_command_line_serves_the_design(tmp_path, capsys, monkeypatch):
    """`random-model` writes a folder with every tensor of the design (hyper-connection coefficients near neutral, in
    the engine as 32-bit), `models` lists it, and `generate` produces the plain implementation's greedy tokens (on the
    CPU, with the plain kernel table in the CUDA kernels' place)."""
    import json

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
    stored, weights = plain.read_folder(folder)
    assert set(weights) == {name for name, _ in tensor_table(CONFIGS["a"])}
    assert float((weights["l0.hc1.mix"] - torch.eye(3, dtype=torch.float64)).abs().max()) < 0.3
    assert cli.main(["models"]) == 0
    assert "Rulorax" in capsys.readouterr().out.split()
    assert cli.main(["generate", folder, "--prompt-ids", "5,17,3,44,9", "--max-tokens", "4", "--dtype", "float32", "--max-model-len",
                     "64", "--max-seqs", "2", "--max-step-tokens", "32", "--page-size", "8", "--ignore-eos"]) == 0
    out = json.loads(capsys.readouterr().out.splitlines()[0])
    ids = [5, 17, 3, 44, 9]
    for token in out["token_ids"]:
        logits = plain.forward(stored, weights, ids)[-1]
        assert token == int(logits.argmax()) or float(logits.max() - logits[token]) < 1e-4
        ids.append(token)
    assert len(out["token_ids"]) == 4

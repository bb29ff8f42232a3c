"""Tiny Kasovik configurations, model folders with weights that make faults show, and the comparison with the plain
implementation (tests/plain_kasovik.py) that the CPU and GPU tests of this design share."""
from __future__ import annotations

import json

import torch
from safetensors.torch import load_file, save_file

import plain_kasovik as plain


def _window(heads, kv_heads, dim, size, sharpen):
    return {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": dim, "mask": {"size": size},
            "scale": sharpen / dim ** 0.5}


def _delta(heads, kv_heads, dim, vdim, conv, decay_rank, gate_rank):
    return {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": conv, "decay_rank": decay_rank,
            "gate_rank": gate_rank}


def _parallel(left, right, left_scale, right_scale, mlp, weights_of=None):
    out = {"type": "parallel", "mixer": {"left": left, "right": right, "left_scale": left_scale,
                                         "right_scale": right_scale}, "mlp": mlp}
    if weights_of is not None:
        out["weights_of"] = weights_of
    return out


def _retention(heads, dim, vdim, decay, base, dims, mlp, weights_of=None):
    out = {"type": "retention", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "decay": decay,
                                          "rot": {"base": base, "dims": dims}}, "mlp": mlp}
    if weights_of is not None:
        out["weights_of"] = weights_of
    return out


def _mlp(ff, limit):
    return {"kind": "dense", "ff": ff, "limit": limit}


def _model(width, vocab, eps, scale, bigram, layers):
    c = {"architecture": "Kasovik", "width": width, "vocab": vocab, "norm": {"eps": eps},
         "embedding": {"scale": scale, "bigram": {"buckets": bigram[0], "mul_prev": bigram[1], "mul_cur": bigram[2]}},
         "layers": layers}
    return json.loads(json.dumps(c))                  # (layers that share a dict above become dicts of their own)


_LA = _parallel(_window(4, 2, 32, 9, 4.0), _delta(4, 2, 16, 32, 4, 8, 12), 0.7, 1.3, _mlp(96, 2.0))
_RA = _retention(2, 32, 48, [0.9, 0.97], 10000.0, 16, None)
# A: a parallel layer, a retention layer without feed-forward, and both once more under other layers' weights. Head
# sizes that are multiples of 16 (the tensor-core attention's domain), a window of 9 (shorter than a page of 64, longer
# than a page of 4), two key heads for four query heads on both sides, four taps, partial rotation.
KA = _model(64, 211, 1e-5, 2.5, (97, 13, 5), [_LA, _RA, dict(_LA, weights_of=0), dict(_RA, weights_of=1)])
# B: sizes that are multiples of nothing (head sizes 20 and 12, width 72, an odd vocabulary), as many key heads as
# query heads on the left and a third of them on the right, two taps, a window of 5, the retention layer first, a layer
# that runs with a later layer's weights, a pair table of one bucket.
_LB = _parallel(_window(3, 3, 20, 5, 3.0), _delta(6, 2, 12, 20, 2, 5, 7), 1.2, 0.6, _mlp(100, 0.75))
_RB = _retention(3, 24, 40, [0.5, 0.95, 0.999], 500.0, 8, _mlp(56, 1.5))
KB = _model(72, 157, 1e-6, 0.8, (1, 3, 2), [_RB, dict(_LB, weights_of=2), _LB])
# C: larger heads, so that a thread of the scan holds 16 and 32 key channels (key sizes 96 and 160), a window of 70
# (over a page border of 64), one tap (no carried inputs), one query head per key head, value sizes other than key sizes.
_LC = _parallel(_window(2, 1, 64, 70, 5.0), _delta(2, 2, 96, 80, 1, 16, 16), 1.0, 1.0, None)
_RC = _retention(2, 160, 64, [0.98, 0.995], 1000000.0, 160, _mlp(64, 1.0))
KC = _model(128, 300, 1e-5, 1.0, (211, 31, 7), [_LC, _RC])
# One mechanism alone.
K_RET = _model(48, 97, 1e-5, 1.5, (31, 7, 3), [_retention(3, 16, 16, [0.8, 0.9, 0.99], 100.0, 16, None)])
K_PAR = _model(48, 97, 1e-5, 1.5, (31, 7, 3), [_parallel(_window(2, 1, 16, 6, 3.0), _delta(2, 1, 16, 24, 3, 4, 4), 0.9, 1.1, None)])
# D (GPU tests only): attention heads of 128 (the tcgen05 prompt kernel, with window and sink), key sizes 128, 256 and 512 in
# the scan (8 and 16 key channels a thread), a layer on shared weights.
_LD = _parallel(_window(4, 2, 128, 100, 5.0), _delta(4, 2, 128, 128, 4, 16, 16), 0.9, 1.2, _mlp(384, 1.0))
KD = _model(256, 700, 1e-5, 2.0, (509, 29, 5), [_LD, _retention(2, 256, 64, [0.98, 0.999], 1e6, 64, _mlp(384, 1.0)),
                                                dict(_LD, weights_of=0), _retention(1, 512, 32, [0.995], 1e4, 512, None)])
CONFIGS = {"a": KA, "b": KB, "c": KC, "ret": K_RET, "par": K_PAR}


def tensor_table(config):
    """(stored name, shape) of every tensor of a model folder, from the configuration alone."""
    w = config["width"]
    b = config["embedding"]["bigram"]
    out = [("embed", (config["vocab"], w)), ("bigram", (b["buckets"] + 1, w)), ("final.norm", (w,))]
    for i, layer in enumerate(config["layers"]):
        if "weights_of" in layer:
            continue
        m, mlp, p = layer["mixer"], layer.get("mlp"), f"l{i}."
        out.append((p + "norm1", (w,)))
        if layer["type"] == "retention":
            out += [(p + "mix.q", (m["heads"] * m["dim"], w)), (p + "mix.k", (m["heads"] * m["dim"], w)),
                    (p + "mix.v", (m["heads"] * m["vdim"], w)), (p + "mix.g", (m["heads"] * m["vdim"], w)),
                    (p + "mix.o", (w, m["heads"] * m["vdim"]))]
        else:
            le, r = m["left"], m["right"]
            nq, nv = r["kv_heads"] * r["dim"], r["heads"] * r["vdim"]
            out += [(p + "mix.left.q", (le["heads"] * le["dim"], w)), (p + "mix.left.k", (le["kv_heads"] * le["dim"], w)),
                    (p + "mix.left.sink", (le["heads"],)), (p + "mix.left.o", (w, le["heads"] * le["dim"])),
                    (p + "mix.right.q", (nq, w)), (p + "mix.right.q.conv", (nq, r["conv"])),
                    (p + "mix.right.k", (nq, w)), (p + "mix.right.k.conv", (nq, r["conv"])),
                    (p + "mix.right.v", (nv, w)), (p + "mix.right.v.conv", (nv, r["conv"])),
                    (p + "mix.right.b", (r["heads"], w)), (p + "mix.right.A_log", (r["heads"],)),
                    (p + "mix.right.norm", (r["vdim"],)), (p + "mix.right.a1", (r["decay_rank"], w)),
                    (p + "mix.right.a2", (r["heads"] * r["dim"], r["decay_rank"])),
                    (p + "mix.right.dt_bias", (r["heads"] * r["dim"],)), (p + "mix.right.g1", (r["gate_rank"], w)),
                    (p + "mix.right.g2", (nv, r["gate_rank"])), (p + "mix.right.o", (w, nv))]
        if mlp is not None:
            out += [(p + "mlp.gate", (mlp["ff"], w)), (p + "mlp.gate.b", (mlp["ff"],)), (p + "mlp.up", (mlp["ff"], w)),
                    (p + "mlp.up.b", (mlp["ff"],)), (p + "mlp.down", (w, mlp["ff"])), (p + "mlp.down.b", (w,))]
    return out


def make_weights(config, seed: int):
    """Random weights, rounded to bfloat16 (so that both sides read the same numbers). Products' weights are N(0, 1/in),
    so activations keep unit size; with the configurations' score scales the attention's scores spread over several
    units, so single keys stand out and a wrong key, page or window edge moves the logits. Sinks are N(0, 1): they take
    a visible share of the denominator. Decay rates are spread so that some channels forget within a few tokens and
    others keep what the first tokens wrote."""
    g = torch.Generator().manual_seed(seed)
    out = {}
    for name, shape in tensor_table(config):
        x = torch.randn(shape, generator=g, dtype=torch.float32)
        if name.endswith(".conv"):
            x = 0.6 * x
        elif name.endswith("A_log"):
            x = -1.0 + 1.5 * x
        elif name.endswith(("dt_bias", ".sink", ".b")) and len(shape) == 1:
            pass
        elif len(shape) == 1:
            x = 1.0 + 0.1 * x
        elif name in ("embed", "bigram"):
            pass
        else:
            x = x / shape[1] ** 0.5
        out[name] = x.to(torch.bfloat16).contiguous()
    return out


def stored_config(config):
    """The configuration as a stored model has it: without the two ranks that only tensor shapes give."""
    c = json.loads(json.dumps(config))
    for layer in c["layers"]:
        if layer["type"] == "parallel":
            layer["mixer"]["right"].pop("decay_rank")
            layer["mixer"]["right"].pop("gate_rank")
    return c


def make_folder(tmp_path, name: str, seed: int = 0, config=None):
    config = config or CONFIGS[name]
    folder = tmp_path / f"kasovik_{name}"
    folder.mkdir(parents=True, exist_ok=True)
    (folder / "config.json").write_text(json.dumps(stored_config(config)))
    save_file(make_weights(config, seed), str(folder / "model.safetensors"))
    return folder


def read_folder(folder):
    import pathlib
    folder = pathlib.Path(folder)
    return json.loads((folder / "config.json").read_text()), load_file(str(folder / "model.safetensors"))


def exact_logits(folder, ids):
    config, weights = read_folder(folder)
    return plain.forward(weights, config, list(ids)).float()


# The measure, per row: the distance from the plain implementation's 64-bit logits (mean taken off, root mean square
# over the vocabulary) relative to the row's own spread. float32: every row within 2e-4 and every arg max the same
# unless the two best logits are closer than that. bfloat16: rounding alone leaves rows of these models 0.005 to 0.03
# away; every row within 0.08 and the median within 0.03. A wrong key, window edge, state or slot moves the rows it
# touches by a good part of their spread.
LIMITS = {"float32": 2e-4, "bfloat16": 0.08}


def row_error(got, want):
    d = got.double() - want.double()
    d = d - d.mean()
    spread = (want.double() - want.double().mean()).pow(2).mean().sqrt()
    return float(d.pow(2).mean().sqrt() / spread)


def compare(got, want, dtype):
    """`got`: {(request, position): logits row}; `want`: {request: exact logits [tokens, vocab]}."""
    assert got, "nothing to compare"
    errors = sorted((row_error(row, want[rid][pos]), rid, pos) for (rid, pos), row in got.items())
    worst = errors[-1]
    assert worst[0] <= LIMITS[dtype], f"request {worst[1]} position {worst[2]}: error {worst[0]:.3g} of the row's spread"
    if dtype == "bfloat16":
        assert errors[len(errors) // 2][0] <= 0.03, f"the median row is {errors[len(errors) // 2][0]:.3g} of its spread off"

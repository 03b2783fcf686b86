"""Host side of the Ratasun hybrid family (no GPU): the configuration reader accepts what the family allows and refuses the rest with a
client error, the model registry keys on config.json's "architecture", and the float64 oracle the GPU tests lean on is itself causal."""
import ctypes as C
import json
import os

import numpy as np
import pytest

import hybrid_oracle as O
from opsagent_b200 import _lib


def model_info(folder, **extra):
    L = _lib.load()
    buf = C.create_string_buffer(4096)
    rc = L.oa_host_model_info(json.dumps(dict({"model_dir": str(folder)}, **extra)).encode(), buf, 4096)
    return rc, (json.loads(buf.value.decode()) if rc == 0 else None)


def write_cfg(folder, cfg):
    os.makedirs(folder, exist_ok=True)
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(cfg, f)


def good_cfg():
    return O.make_config([O.attention_layer(mlp=O.moe()), O.delta_layer(), O.mamba_layer(mlp=O.moe())], width=40, vocab=77, loop={"start": 1, "stop": 3, "times": 2})


def test_config_reader_accepts_the_family(tmp_path):
    write_cfg(tmp_path, good_cfg())
    rc, info = model_info(tmp_path)
    assert rc == 0 and info["hidden"] == 40 and info["vocab"] == 77 and info["n_layers"] == 5     # 1 + 2 x 2 executions
    rc, _ = model_info(tmp_path, dtype="float32")
    assert rc == 0
    rc, _ = model_info(tmp_path, dtype="float16")
    assert rc == 400


def mutate(path, value):
    def f(cfg):
        node = cfg
        for k in path[:-1]:
            node = node[k]
        node[path[-1]] = value
    return f


@pytest.mark.parametrize("change", [
    mutate(["architecture"], "SomethingElse"),
    mutate(["layers", 0, "type"], "sliding_attention"),
    mutate(["layers", 0, "mixer", "rot", "dims"], 10),                 # more rotated channels than rot_dim
    mutate(["layers", 1, "mixer", "kv_heads"], 3),                     # does not divide heads
    mutate(["layers", 2, "mixer", "groups"], 3),
    mutate(["layers", 2, "mixer", "norm_groups"], 5),
    mutate(["layers", 0, "mlp", "router", "top"], 5),                  # more choices than the kept groups hold
    mutate(["layers", 0, "mlp", "router", "groups", "keep"], 4),
    mutate(["layers", 0, "mlp", "kind"], "dense"),
    mutate(["loop", "stop"], 7),
    mutate(["loop", "times"], 0),
    mutate(["width"], 0),
], ids=lambda f: "")
def test_config_reader_refuses(tmp_path, change):
    cfg = good_cfg()
    change(cfg)
    write_cfg(tmp_path, cfg)
    rc, _ = model_info(tmp_path)
    assert rc == 400


def test_missing_folder_is_a_client_error(tmp_path):
    rc, _ = model_info(tmp_path / "nowhere")
    assert rc == 400


def test_checkpoint_writer_and_oracle_are_consistent(tmp_path):
    cfg = good_cfg()
    W = O.random_weights(cfg, 1)
    O.write_checkpoint(str(tmp_path), cfg, W)
    raw = open(tmp_path / "model.safetensors", "rb").read()
    n = int.from_bytes(raw[:8], "little")
    hdr = json.loads(raw[8:8 + n])
    assert set(hdr) == set(W) and all(v["dtype"] == "BF16" for v in hdr.values())
    a, b = hdr["l1.mix.a2"]["data_offsets"]
    got = (np.frombuffer(raw[8 + n + a:8 + n + b], dtype=np.uint16).astype(np.uint32) << 16).view(np.float32).reshape(hdr["l1.mix.a2"]["shape"])
    assert np.array_equal(got.astype(np.float64), W["l1.mix.a2"])      # weights are bf16-representable, so the file holds them exactly
    toks = np.random.default_rng(0).integers(0, cfg["vocab"], 40).tolist()
    full = O.forward(cfg, W, toks)
    assert np.abs(O.forward(cfg, W, toks[:17]) - full[:17]).max() < 1e-9          # causal: a prefix sees nothing of what follows
    assert np.abs(O.forward(cfg, W, toks[1:])[5:] - full[6:]).max() > 1e-3         # and the past matters (positions, states, cache)


def test_router_oracle_keeps_only_the_best_groups():
    m = O.moe(experts=8, top=3, groups=4, keep=2, ff=8)
    rng = np.random.default_rng(3)
    W = {"r.router": rng.standard_normal((8, 16)), "r.correction": rng.standard_normal(8)}
    idx, wgt = O.route(rng.standard_normal((50, 16)), W, "r.", m)
    assert np.allclose(wgt.sum(1), m["router"]["scale"])
    for row in idx:
        assert len(set(row)) == 3 and len({e // 2 for e in row}) <= 2

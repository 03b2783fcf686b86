"""Host side of the Zurevik design (no GPU): the configuration reader accepts what the design allows and refuses the rest with a client
error, and the float64 oracle the GPU tests lean on has the masks it claims."""
import ctypes as C
import json
import os

import numpy as np
import pytest

import zurevik_oracle as Z
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
    return Z.make_config([Z.diff_layer(mlp=Z.moe()), Z.sink_layer(), Z.sink_layer(kv_from=1, mlp=Z.moe(experts=4, top=4))], width=40, vocab=77)


def test_config_reader_accepts_the_design(tmp_path):
    write_cfg(tmp_path, good_cfg())
    rc, info = model_info(tmp_path)
    assert rc == 0 and info["hidden"] == 40 and info["vocab"] == 77 and info["n_layers"] == 3
    assert model_info(tmp_path, dtype="float32")[0] == 0
    cfg = good_cfg()                                       # optional keys: no kept tokens, no soft cap, a layer without feed-forward
    del cfg["layers"][0]["mixer"]["mask"]["keep_first"], cfg["logit_softcap"]
    cfg["layers"][0]["mlp"] = None
    write_cfg(tmp_path / "b", cfg)
    assert model_info(tmp_path / "b")[0] == 0


def mutate(path, value):
    def f(cfg):
        node = cfg
        for k in path[:-1]:
            node = node[k]
        node[path[-1]] = value
    return f


@pytest.mark.parametrize("change", [
    mutate(["layers", 0, "type"], "attention_3"),
    mutate(["layers", 0, "mixer", "kv_heads"], 3),                     # does not divide heads
    mutate(["layers", 0, "mixer", "mask", "size"], 0),
    mutate(["layers", 0, "mixer", "vdim"], 300),                       # beyond what the kernels hold
    mutate(["layers", 2, "mixer", "kv_from"], 2),                      # itself
    mutate(["layers", 2, "mixer", "kv_from"], 0),                      # a layer of another kind
    mutate(["layers", 2, "mixer", "dim"], 8),                          # not the size of the keys it reads
    mutate(["layers", 1, "mixer", "kv_from"], 2),                      # a later layer
    mutate(["layers", 0, "mlp", "router", "top"], 7),                  # more choices than experts
    mutate(["layers", 0, "mlp", "kind"], "dense"),
    mutate(["vocab"], 0),
], ids=lambda f: "")
def test_config_reader_refuses(tmp_path, change):
    cfg = good_cfg()
    change(cfg)
    write_cfg(tmp_path, cfg)
    assert model_info(tmp_path)[0] == 400


def test_oracle_masks_and_causality():
    vis = Z.visible(12, 4, 2)
    assert vis[9].tolist() == [True, True, False, False, False, False, True, True, True, True, False, False]
    assert vis[2].tolist() == [True, True, True] + [False] * 9 and Z.visible(5, 1)[3].tolist() == [False, False, False, True, False]
    p = Z.masked_softmax(np.zeros((1, 3)), np.array([[True, True, False]]), sink=0.0)
    assert np.allclose(p, [[1 / 3, 1 / 3, 0.0]])                       # the sink counts once in the denominator and has no value
    cfg = good_cfg()
    W = Z.random_weights(cfg, 1)
    toks = np.random.default_rng(0).integers(0, cfg["vocab"], 60).tolist()
    full = Z.forward(cfg, W, toks)
    assert np.abs(Z.forward(cfg, W, toks[:17]) - full[:17]).max() < 1e-9          # causal: a prefix sees nothing of what follows
    idx, wgt = Z.route(np.random.default_rng(1).standard_normal((20, 40)), W, "l0.mlp.", cfg["layers"][0]["mlp"])
    assert np.allclose(wgt.sum(1), 1.0) and (np.diff(wgt, axis=1) <= 0).all() and all(len(set(r)) == 2 for r in idx)

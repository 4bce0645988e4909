"""Rifizen without a GPU: its configuration, the run order a loop gives, what its mixers ask of the cache, and the
plain implementation's recurrence against the same sums written as one double loop."""
import copy
import json

import pytest
import torch

from helpers import RIFIZEN_CONFIGS, config_dict, random_tokens
from plain import rifizen_plain as P


def parsed(cfg):
    from rocmforge_b200.config import architecture_for
    arch = architecture_for("Rifizen")
    return arch, arch.config_cls.from_dict(config_dict(cfg))


def test_the_design_is_chosen_by_its_name(tmp_path):
    from rocmforge_b200.config import load_config, UnknownArchitecture
    (tmp_path / "config.json").write_text(json.dumps(config_dict(RIFIZEN_CONFIGS["RA"])))
    arch, cfg = load_config(str(tmp_path))
    assert arch.name == "Rifizen" and cfg.width == 64 and cfg.layers[1].mlp.kind == "moe" and cfg.layers[2].mlp is None
    assert cfg.to_dict() == config_dict(RIFIZEN_CONFIGS["RA"])
    bad = dict(config_dict(RIFIZEN_CONFIGS["RA"]), architecture="Rifizzen")
    (tmp_path / "config.json").write_text(json.dumps(bad))
    with pytest.raises(UnknownArchitecture):
        load_config(str(tmp_path))


@pytest.mark.parametrize("path,value,error", [
    ("width", None, "MissingKey"), ("norm.eps", None, "MissingKey"), ("vocab", 0, "InvalidValue"),
    ("layers.0.mixer.left.kv_heads", 3, "InvalidValue"), ("layers.0.mixer.left.mask.size", 0, "InvalidValue"),
    ("layers.0.mixer.left.scale", None, "MissingKey"), ("layers.1.mixer.right.decay", [0.5], "InvalidValue"),
    ("layers.1.mixer.right.rot.dims", 7, "InvalidValue"), ("layers.1.mlp.router.top", 6, "InvalidValue"),
    ("layers.1.mlp.kind", "sparse", "InvalidValue"), ("layers.2.type", "serial", "InvalidValue"),
    ("loop.stop", 9, "InvalidValue"), ("loop.times", 0, "InvalidValue"),
])
def test_faults_of_a_configuration_name_their_key(path, value, error):
    from rocmforge_b200.config import errors
    raw = copy.deepcopy(config_dict(RIFIZEN_CONFIGS["RA"]))
    cur = raw
    parts = path.split(".")
    for p in parts[:-1]:
        cur = cur[int(p)] if p.isdigit() else cur[p]
    if value is None:
        del cur[parts[-1]]
    else:
        cur[parts[-1]] = value
    from rocmforge_b200.config import architecture_for
    with pytest.raises(getattr(errors, error)) as e:
        architecture_for("Rifizen").config_cls.from_dict(raw)
    assert parts[-1] in str(e.value)


def test_optional_keys():
    raw = copy.deepcopy(config_dict(RIFIZEN_CONFIGS["RB"]))
    del raw["layers"][0]["mixer"]["left"]["softcap"]            # no cap
    _, cfg = parsed(raw)
    assert cfg.layers[0].left.softcap is None and not cfg.has_loop


@pytest.mark.parametrize("name,order", [
    ("RA", [(0, 0), (1, None), (0, 1), (1, None), (2, None)]),
    ("RB", [(0, None), (1, None)]),
    ("RC", [(0, None), (1, 0), (1, 1), (1, 2), (2, None)]),
])
def test_run_order_of_looped_layers(name, order):
    """Layers start .. stop-1 run ``times`` times in a row; the first layer of every pass carries the pass number; every
    execution owns a cache of its own.  The plain implementation's order is the same."""
    arch, cfg = parsed(RIFIZEN_CONFIGS[name])
    spec = arch.build(cfg)
    assert [(e.layer, e.pass_index) for e in spec.schedule] == order
    assert P.layer_order(config_dict(RIFIZEN_CONFIGS[name])) == order
    assert sorted(spec.cache_requests()) == list(range(len(order)))
    assert (spec.pass_offsets is not None) == cfg.has_loop


def test_tensor_names_and_shapes():
    arch, cfg = parsed(RIFIZEN_CONFIGS["RA"])
    specs = arch.build(cfg).param_specs()
    want = {"embed": (96, 64), "head": (96, 64), "final.norm": (64,), "loop.step": (2, 64), "l0.norm1b": (64,),
            "l0.mix.left.q": (64, 64), "l0.mix.left.k": (32, 64), "l0.mix.left.v": (48, 64), "l0.mix.left.o": (64, 96),
            "l0.mix.right.g": (24, 64), "l0.mix.right.o": (64, 24), "l0.mix.left.out": (64,), "l0.mix.right.out": (64,),
            "l0.mlp.up": (40, 64), "l1.mlp.router": (5, 64), "l1.mlp.router.b": (5,), "l1.mlp.e4.down": (64, 20),
            "l2.mix.right.q": (40, 64)}
    for name, shape in want.items():
        assert tuple(specs[name].shape) == shape, name
    # a layer without feed-forward: no mlp tensors; its second pair of norms may be in a folder, and is not used
    assert not any(n.startswith("l2.mlp") for n in specs) and specs["l2.norm2"].optional and specs["l2.norm2b"].optional
    assert len([n for n, s in specs.items() if not s.optional]) == 4 + 3 * 13 + (2 + 2) + (2 + 2 + 3 * 5)


def test_cache_of_side_by_side_mixers():
    """The attention half asks for a window of keys (values of another size in a tensor of their own), the retention half
    for a 32-bit state; every execution of a looped layer has both; a slot's state is zero when it is handed out."""
    from rocmforge_b200.cache import SequenceCache
    arch, cfg = parsed(RIFIZEN_CONFIGS["RA"])
    spec = arch.build(cfg)
    cache = SequenceCache(spec.cache_requests(), max_tokens=256, max_slots=3, dtype=torch.float32, device="cpu")
    view = cache.view(0)
    assert set(view) == {"left", "right"}
    assert view["left"].k_pages.shape[1:] == (2, 64, 16) and view["left"].v_pages.shape[1:] == (2, 64, 24)
    assert view["left"].window == 7 and cache.view(1)["left"].window == 3
    assert view["right"]["S"].shape == (3, 2, 12, 24) and view["right"]["S"].dtype == torch.float32
    assert cache.view(2)["right"]["S"].data_ptr() != view["right"]["S"].data_ptr()            # pass 2 of layer 0
    s = cache.alloc_slot()
    view["right"]["S"][s] = 5.0
    cache.prepare([s], [100]); cache.commit([s], [100])
    held = [len(g.held_pages(s)) for g in cache.groups]
    assert max(held) <= 2                                                                     # windows of 7, 3 and 1: old pages go back
    cache.free_slot(s)
    assert cache.alloc_slot() == s and float(view["right"]["S"][s].abs().max()) == 0.0
    assert all(g.pool.n_free == g.n_pages for g in cache.groups)


def test_plain_retention_is_the_decayed_sum():
    """S_t = d S_(t-1) + k_t v_t^T, o_t = S_t^T q_t  ==  o_t = sum_(s<=t) d^(t-s) (q_t . k_s) v_s, and carrying the state
    over a cut changes nothing."""
    torch.manual_seed(0)
    T, width = 30, 16
    m = {"heads": 2, "dim": 6, "vdim": 4, "decay": [0.9, 1.0], "rot": {"dims": 4, "base": 10.0}}
    W = {"r." + n: torch.randn(s, width, dtype=torch.float64) for n, s in (("q", 12), ("k", 12), ("v", 8), ("g", 8))}
    W["r.o"] = torch.eye(8, dtype=torch.float64)                                      # the gated heads themselves
    h = torch.randn(T, width, dtype=torch.float64)
    out, S = P.retention(h, W, "r.", m, 1e-6)
    pos = torch.arange(T)
    q = P.rotate_half_layout((h @ W["r.q"].T).reshape(T, 2, 6), pos, 4, 10.0)
    k = P.rotate_half_layout((h @ W["r.k"].T).reshape(T, 2, 6), pos, 4, 10.0) * 6 ** -0.5
    v = (h @ W["r.v"].T).reshape(T, 2, 4)
    o = torch.zeros(T, 2, 4, dtype=torch.float64)
    for t in range(T):
        for s in range(t + 1):
            for hh, d in enumerate(m["decay"]):
                o[t, hh] += d ** (t - s) * (q[t, hh] @ k[s, hh]) * v[s, hh]
    want = (P.unit_rms(o, 1e-6) * P.silu(h @ W["r.g"].T).reshape(T, 2, 4)).reshape(T, 8)
    assert (out - want).abs().max() < 1e-10
    a, Sa = P.retention(h[:11], W, "r.", m, 1e-6)
    b, Sb = P.retention(h[11:], W, "r.", m, 1e-6, positions=pos[11:], state=Sa)
    assert (torch.cat([a, b]) - out).abs().max() < 1e-12 and (Sb - S).abs().max() < 1e-12


def test_plain_window_and_routing_edges():
    """A query sees itself and window-1 tokens before it; of the experts only the ``top`` best count."""
    torch.manual_seed(1)
    T, width = 12, 8
    m = {"heads": 2, "kv_heads": 1, "dim": 4, "vdim": 4, "scale": 0.5, "softcap": 10.0, "mask": {"size": 3}}
    W = {"a." + n: torch.randn(s, width, dtype=torch.float64) for n, s in (("q", 8), ("k", 4), ("v", 4))}
    W["a.o"] = torch.eye(8, dtype=torch.float64)
    h = torch.randn(T, width, dtype=torch.float64)
    base = P.capped_window_attention(h, W, "a.", m, 1e-6)
    h2 = h.clone(); h2[5] += 1.0
    moved = (P.capped_window_attention(h2, W, "a.", m, 1e-6) - base).abs().sum(dim=1) > 1e-12
    assert moved.tolist() == [i in (5, 6, 7) for i in range(T)]
    Wm = {"m.router": torch.zeros(4, width, dtype=torch.float64), "m.router.b": torch.tensor([0.0, 3.0, 1.0, 2.0], dtype=torch.float64)}
    for e in range(4):
        Wm[f"m.e{e}.gate"] = torch.full((2, width), 0.1 * (e + 1), dtype=torch.float64)
        Wm[f"m.e{e}.up"] = torch.ones(2, width, dtype=torch.float64)
        Wm[f"m.e{e}.down"] = torch.ones(width, 2, dtype=torch.float64)
    out = P.routed_ff(h[:1], Wm, "m.", 4, 2)
    w = torch.softmax(torch.tensor([3.0, 2.0], dtype=torch.float64), dim=0)
    def expert(e):
        return (P.silu(h[0] @ Wm[f"m.e{e}.gate"].T) * (h[0] @ Wm[f"m.e{e}.up"].T)) @ Wm[f"m.e{e}.down"].T
    assert (out[0] - (w[0] * expert(1) + w[1] * expert(3))).abs().max() < 1e-12


def test_command_line_writes_a_random_model_folder(tmp_path):
    """rocmforge --random-config CONFIG --write-random DIR for this design: config.json comes back as it went in, the
    tensors are those the builder names, and the same seed gives the same bits."""
    import subprocess
    import sys
    from helpers import ROOT
    from safetensors.torch import load_file
    cfg_path = tmp_path / "cfg.json"
    cfg_path.write_text(json.dumps(config_dict(RIFIZEN_CONFIGS["RA"])))
    outs = []
    for name in ("a", "b"):
        out = tmp_path / name
        r = subprocess.run([sys.executable, f"{ROOT}/bin/rocmforge", "--random-config", str(cfg_path), "--write-random", str(out),
                            "--random-seed", "5", "--dtype", "float32"], capture_output=True, text=True)
        assert r.returncode == 0, r.stderr
        outs.append(load_file(str(out / "model.safetensors")))
    written = json.load(open(tmp_path / "a" / "config.json"))
    assert {k: v for k, v in written.items() if k != "torch_dtype"} == config_dict(RIFIZEN_CONFIGS["RA"])
    arch, cfg = parsed(RIFIZEN_CONFIGS["RA"])
    assert set(outs[0]) == {n for n, s in arch.build(cfg).param_specs().items() if not s.optional}
    assert all(torch.equal(outs[0][k], outs[1][k]) for k in outs[0])
    assert float(outs[0]["l1.mlp.router.b"].abs().max()) > 0 and torch.equal(outs[0]["l0.norm1"], torch.ones(64))


def test_a_folder_may_hold_the_unused_norms_and_an_unused_pass_table(tmp_path):
    """A layer without feed-forward whose second pair of norms is stored all the same, and a loop over an empty stretch of
    layers whose table of pass vectors is stored: both folders load; a tensor nobody knows is still a fault."""
    from rocmforge_b200 import WeightError, write_model_folder
    from rocmforge_b200.weights import load_folder
    from rocmforge_b200.weights.safetensors_io import write_safetensors
    from safetensors.torch import load_file
    raw = copy.deepcopy(config_dict(RIFIZEN_CONFIGS["RA"]))
    raw["loop"] = {"start": 1, "stop": 1, "times": 2}
    arch, cfg = parsed(raw)
    spec = arch.build(cfg)
    assert [(e.layer, e.pass_index) for e in spec.schedule] == [(0, None), (1, None), (2, None)]
    folder = str(tmp_path / "m")
    write_model_folder(folder, raw, spec.param_specs(), 3, torch.float32)
    tensors = load_file(folder + "/model.safetensors")
    assert "loop.step" in tensors and "l2.norm2" not in tensors
    tensors["l2.norm2"] = torch.ones(64)
    tensors["l2.norm2b"] = torch.ones(64)
    write_safetensors(folder + "/model.safetensors", tensors.items())
    loaded = load_folder(folder, spec.param_specs(), torch.float32, "cpu")
    assert "l2.norm2" in loaded and "l0.mix.left.q" in loaded
    tensors["l2.norm3"] = torch.ones(64)
    write_safetensors(folder + "/model.safetensors", tensors.items())
    with pytest.raises(WeightError) as e:
        load_folder(folder, spec.param_specs(), torch.float32, "cpu")
    assert e.value.unexpected == ["l2.norm3"]

"""Vilulorn without a GPU: its configuration (keys, faults, sizes that are a tensor's shape), the parts its builder picks,
which executions lend and borrow keys, what the cache keeps and hands back for chunked attention, the stretched rotary
frequencies, and the plain implementation's mechanisms against the same sums written another way."""
import copy
import json
import math

import pytest
import torch

from helpers import VILULORN_CONFIGS, random_tokens, vilulorn_config, write_vilulorn
from plain import vilulorn_plain as P


def test_the_design_is_chosen_by_its_name_and_ranks_come_from_the_tensors(tmp_path):
    from rocmforge_b200.config import load_config
    write_vilulorn(VILULORN_CONFIGS["VA"], str(tmp_path))
    arch, cfg = load_config(str(tmp_path))
    assert arch.name == "Vilulorn" and cfg.width == 64 and cfg.max_positions == 400
    assert [L.type for L in cfg.layers] == ["attention", "gla", "attention", "gla"]
    assert [L.mixer.rank for L in cfg.layers if L.type == "gla"] == [5, 8]          # rows of l<i>.mix.a1 in the folder
    assert cfg.layers[1].mlp is None and cfg.layers[2].mixer.kv_from == 0 and cfg.layers[0].mixer.rot_scaling is None
    assert cfg.layers[0].mlp.limit == 0.5 and cfg.layers[0].mlp.top == 2
    raw = json.load(open(tmp_path / "config.json"))
    assert cfg.to_dict() == raw and "ranks" not in raw
    assert vilulorn_config(VILULORN_CONFIGS["VB"])[0].layers[1].mixer.rot_scaling == dict(factor=8.0, low=1.0, high=4.0, original=64.0)


@pytest.mark.parametrize("path,value,error", [
    ("width", None, "MissingKey"), ("norm.eps", None, "MissingKey"), ("vocab", 0, "InvalidValue"), ("max_positions", None, "MissingKey"),
    ("layers.0.mixer.kv_heads", 3, "InvalidValue"), ("layers.0.mixer.mask.size", 0, "InvalidValue"),
    ("layers.0.mixer.scale", None, "MissingKey"), ("layers.0.mixer.rot.dims", 7, "InvalidValue"),
    ("layers.0.mixer.rot.dims", 18, "InvalidValue"), ("layers.1.mixer.tau", 0.0, "InvalidValue"), ("layers.1.mixer.vdim", None, "MissingKey"),
    ("layers.0.mlp.router.top", 6, "InvalidValue"), ("layers.0.mlp.expert.limit", None, "MissingKey"),
    ("layers.0.mlp.kind", "dense", "InvalidValue"), ("layers.3.type", "retention", "InvalidValue"),
    ("layers.2.mixer.kv_from", 1, "InvalidValue"), ("layers.2.mixer.kv_from", 2, "InvalidValue"), ("layers.2.mixer.dim", 32, "InvalidValue"),
])
def test_faults_of_a_configuration_name_their_key(path, value, error):
    from rocmforge_b200.config import architecture_for, errors
    raw = copy.deepcopy(vilulorn_config(VILULORN_CONFIGS["VA"])[1])
    cur = raw
    parts = path.split(".")
    for p in parts[:-1]:
        cur = cur[int(p)] if p.isdigit() else cur[p]
    if value is None:
        del cur[parts[-1]]
    else:
        cur[parts[-1]] = value
    with pytest.raises(getattr(errors, error)) as e:
        architecture_for("Vilulorn").config_cls.from_dict(raw)
    assert parts[-1] in str(e.value) or "kv_from" in str(e.value)


def test_the_builder_picks_parts_and_names_by_the_configuration():
    from rocmforge_b200.config import architecture_for
    for name, c in VILULORN_CONFIGS.items():
        cfg, _ = vilulorn_config(c)
        spec = architecture_for("Vilulorn").build(cfg)
        specs = spec.param_specs()
        W = c["width"]
        assert specs["embed"].shape == (c["vocab"], W) and specs["pos"].shape == (c["max_positions"], W)
        for i, L in enumerate(c["layers"]):
            m = L["mixer"]
            assert specs[f"l{i}.norm1"].shape == (W,)
            assert (f"l{i}.mlp.router" in specs) == (L["mlp"] is not None)
            assert specs.get(f"l{i}.norm2") is not None
            assert specs[f"l{i}.norm2"].optional == (L["mlp"] is None)
            if L["type"] == "gla":
                assert specs[f"l{i}.mix.a1"].shape == (c["ranks"][i], W)
                assert specs[f"l{i}.mix.a2"].shape == (m["heads"] * m["dim"], c["ranks"][i])
                assert specs[f"l{i}.mix.a2.b"].shape == (m["heads"] * m["dim"],) and specs[f"l{i}.mix.norm"].shape == (m["vdim"],)
                assert specs[f"l{i}.mix.g"].shape == (m["heads"] * m["vdim"], W)
            else:
                borrowed = "kv_from" in m
                assert (f"l{i}.mix.k" in specs) == (not borrowed) and (f"l{i}.mix.v" in specs) == (not borrowed)
                assert (f"l{i}.mix.k.norm" in specs) == (not borrowed) and specs[f"l{i}.mix.q.norm"].shape == (m["dim"],)
                assert specs[f"l{i}.mix.g"].shape == (m["heads"] * m["vdim"], W) and specs[f"l{i}.mix.o"].shape == (W, m["heads"] * m["vdim"])
                assert spec.schedule[i].kv_from == m.get("kv_from")
        requests = spec.cache_requests()
        for i, L in enumerate(c["layers"]):
            if L["type"] == "attention" and "kv_from" in L["mixer"]:
                assert i not in requests
        assert spec.max_position == c["max_positions"]


def test_a_lender_with_borrowers_of_another_chunk_size_keeps_all_its_keys():
    from rocmforge_b200.config import architecture_for
    spec = architecture_for("Vilulorn").build(vilulorn_config(VILULORN_CONFIGS["VA"])[0])
    req = spec.cache_requests()
    assert req[0].chunk is None and req[0].window is None           # chunks of 7, read by a layer with chunks of 64
    spec = architecture_for("Vilulorn").build(vilulorn_config(VILULORN_CONFIGS["VC"])[0])
    req = spec.cache_requests()
    assert req[1].chunk == 130 and req[3].chunk == 33               # the borrower shares the lender's chunk size


def test_the_cache_hands_back_the_pages_of_finished_chunks():
    from rocmforge_b200.cache import SequenceCache
    from rocmforge_b200.cache.requests import KVRequest
    cache = SequenceCache({0: KVRequest(2, 8, None, None, 100), 1: KVRequest(2, 8)}, max_tokens=64 * 8, max_slots=2,
                          dtype=torch.float32, device="cpu")
    chunked, full = (cache._group_of[0], cache._group_of[1])
    s = cache.alloc_slot()
    cache.prepare([s], [99]); cache.commit([s], [99])
    assert chunked.held_pages(s) == full.held_pages(s) and len(full.held_pages(s)) == 2        # position 99 still sees 0..98
    cache.prepare([s], [1]); cache.commit([s], [1])               # length 100: the next query (100) starts a new chunk
    assert len(full.held_pages(s)) == 2 and chunked.table[s, 0] < 0 and chunked.table[s, 1] >= 0     # page 0 (0..63) is free, page 1 holds 100
    cache.prepare([s], [150]); cache.commit([s], [150])           # length 250: the chunk 200..299 lies in pages 3 and 4
    assert [int(p) for p in (chunked.table[s] >= 0).nonzero()[0]] == [3]
    assert len(full.held_pages(s)) == 4
    # a prompt that starts inside a chunk needs that chunk's earlier pages to be there, not the ones before
    assert chunked.pages_missing(s, 250, 330) == 2                # pages 4 and 5; page 3 is held
    cache.free_slot(s)
    assert chunked.pool.n_free == chunked.n_pages and full.pool.n_free == full.n_pages
    with pytest.raises(ValueError):
        KVRequest(2, 8, 5, None, 7)


def test_stretched_frequencies():
    from rocmforge_b200.parts.rope import NeoxRope
    for dims, base, sc in [(32, 1e6, dict(factor=4.0, low=1.0, high=4.0, original=512)), (40, 1e4, dict(factor=8.0, low=1.0, high=4.0, original=64)),
                           (8, 100.0, None), (64, 5e5, dict(factor=32.0, low=1.0, high=4.0, original=8192))]:
        rope = NeoxRope(dims + 8, base, rotary_dim=dims, interleaved=True, scaling=sc)
        want = P.scaled_frequencies(dims, base, sc)
        assert torch.allclose(rope.inv_freq_host.double(), want, rtol=1e-6, atol=0)
        plain = base ** (-2.0 * torch.arange(dims // 2, dtype=torch.float64) / dims)
        if sc is not None:
            wave = 2 * math.pi / plain
            short, long_ = wave < sc["original"] / sc["high"], wave > sc["original"] / sc["low"]
            assert torch.equal(want[short], plain[short]) and torch.allclose(want[long_], plain[long_] / sc["factor"])
            between = ~short & ~long_
            assert ((want[between] < plain[between]) & (want[between] > plain[between] / sc["factor"])).all()
    with pytest.raises(ValueError):
        NeoxRope(16, 100.0, scaling=dict(factor=2.0, low=4.0, high=4.0, original=64))


def test_plain_recurrence_against_its_closed_form():
    """o_t = sum_(s<=t) (q_t * prod_(s<r<=t) alpha_r) . k_s  v_s, written as a double loop over (t, s)."""
    torch.manual_seed(0)
    T, H, D, DV, W = 9, 2, 4, 3, 16
    Wt = {"m.q": torch.randn(H * D, W), "m.k": torch.randn(H * D, W), "m.v": torch.randn(H * DV, W), "m.g": torch.randn(H * DV, W),
          "m.o": torch.randn(W, H * DV), "m.a1": torch.randn(2, W), "m.a2": torch.randn(H * D, 2), "m.a2.b": torch.randn(H * D),
          "m.norm": torch.rand(DV) + 0.5}
    Wt = {k: v.double() for k, v in Wt.items()}
    h = torch.randn(T, W, dtype=torch.float64)
    m = dict(heads=H, dim=D, vdim=DV, tau=2.0)
    got = P.gated_linear_attention(h, Wt, "m.", m, 1e-6)
    q = (h @ Wt["m.q"].T).reshape(T, H, D) * D ** -0.5
    k = (h @ Wt["m.k"].T).reshape(T, H, D)
    v = (h @ Wt["m.v"].T).reshape(T, H, DV)
    a = torch.sigmoid((h @ Wt["m.a1"].T) @ Wt["m.a2"].T + Wt["m.a2.b"]).pow(0.5).reshape(T, H, D)
    o = torch.zeros(T, H, DV, dtype=torch.float64)
    for t in range(T):
        for s in range(t + 1):
            decay = torch.ones(H, D, dtype=torch.float64)
            for r in range(s + 1, t + 1):
                decay = decay * a[r]
            o[t] += ((q[t] * decay * k[s]).sum(-1))[:, None] * v[s]
    want = (P.rms_norm(o, Wt["m.norm"], 1e-6).reshape(T, H * DV) * P.silu(h @ Wt["m.g"].T)) @ Wt["m.o"].T
    assert torch.allclose(got, want, rtol=1e-9, atol=1e-12)


def test_plain_model_chunks_and_borrowed_keys():
    """In the plain model a token never feels a token of an earlier chunk through attention: with the recurrent layers'
    outputs and the experts silenced, changing a token changes later logits only inside the chunk of every layer."""
    from safetensors.torch import load_file
    import tempfile
    c = copy.deepcopy(VILULORN_CONFIGS["VC"])
    c["layers"] = [c["layers"][1], c["layers"][4]]                # an attention layer and its borrower, chunks of 130
    c["layers"][1]["mixer"]["kv_from"] = 0
    c["ranks"] = {}
    with tempfile.TemporaryDirectory() as d:
        write_vilulorn(c, d)
        model = P.PlainVilulorn(json.load(open(d + "/config.json")), load_file(d + "/model.safetensors"))
    toks = random_tokens(c["vocab"], 140, 4)
    other = list(toks)
    other[100] = (other[100] + 1) % c["vocab"]
    a, b = model.logits(toks), model.logits(other)
    assert torch.equal(a[:100], b[:100])
    assert (a[100:130] - b[100:130]).abs().max() > 1e-6           # inside the chunk the change is felt
    assert (a[130:] - b[130:]).abs().max() == 0                   # beyond the chunk's end it is not

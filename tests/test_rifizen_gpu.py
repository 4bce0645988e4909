"""The Rifizen decoder in the engine against the plain implementation (needs a GPU): whole prompts, token-by-token
decoding, portions, ragged batches, slots and pages used again, generation through the public entry point, and the
replay program; then each new kernel alone against the arithmetic written out in torch."""
import json
import os

import numpy as np
import pytest
import torch

from helpers import RIFIZEN_CONFIGS, TraceRun, assert_logits_close, random_tokens
from plain import rifizen_plain as P

pytestmark = pytest.mark.gpu

TORCH = {"float32": torch.float32, "bfloat16": torch.bfloat16}
_models, _plains, _refs = {}, {}, {}


def engine(folders, name, dtype):
    import rocmforge_b200 as rf
    if (name, dtype) not in _models:
        _models[(name, dtype)] = rf.Model.from_folder(folders(name, dtype), dtype=TORCH[dtype])
    return _models[(name, dtype)]


def plain_logits(folders, name, dtype, tokens):
    """Logits of the plain model on the folder's stored (rounded) weights, every position."""
    from safetensors.torch import load_file
    if (name, dtype) not in _plains:
        folder = folders(name, dtype)
        _plains[(name, dtype)] = (json.load(open(os.path.join(folder, "config.json"))),
                                  load_file(os.path.join(folder, "model.safetensors")))
    key = (name, dtype, tuple(tokens))
    if key not in _refs:
        cfg, W = _plains[(name, dtype)]
        _refs[key] = P.forward(cfg, W, list(tokens))
    return _refs[key]


def close(got, ref, dtype, what):
    """float32: element by element, at the tolerance of the other models' tests.  bfloat16: this design norms every
    sub-layer's output again, which carries the rounding of one layer run at full size into the next, and with random
    weights a token's choice of experts now and then hangs on the last bits of the router's bfloat16 input (one
    expert swapped changes that row visibly).  So rows are judged by the root mean square of their difference against
    that of the logits: under 4.5 % on average (rounding alone gives 2 to 3 %) and nine rows in ten under 6 % (a row whose
    token took another expert may be off by its whole size).  What a fault changes by less than that, the float32 runs show."""
    if dtype == "float32":
        return assert_logits_close(got, ref, dtype, what)
    got = torch.as_tensor(np.asarray(got), dtype=torch.float64)
    ref = torch.as_tensor(np.asarray(ref), dtype=torch.float64)
    assert got.shape == ref.shape and torch.isfinite(got).all(), what
    d = got - ref
    d = d - d.mean(dim=-1, keepdim=True)
    err = d.pow(2).mean(dim=-1).sqrt() / (ref - ref.mean(dim=-1, keepdim=True)).pow(2).mean().sqrt()
    ok = float(err.mean()) < 0.045 and float((err < 0.06).double().mean()) >= 0.9
    assert ok or err.numel() < 10 and float(err.max()) < 0.40, \
        f"{what}: row errors up to {float(err.max()):.3f}, mean {float(err.mean()):.3f}, {int((err >= 0.06).sum())} of {err.numel()} over 6 %"



def vocab(name):
    return RIFIZEN_CONFIGS[name]["vocab"]


def poison_free_pages(cache):
    for g in cache.groups:
        free = [p for p in range(g.n_pages) if not g.pool.is_held(p)]
        if free:
            idx = torch.tensor(free, device=g.storage.device)
            g.storage[:, :, idx] = float("nan")
            if g.value_storage is not None:
                g.value_storage[:, :, idx] = float("nan")


# --------------------------------------------------------------------------- the model in the engine

@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["RA", "RB", "RC"])
def test_whole_prompt(folders, name, dtype):
    """Every position of a prompt that crosses three page borders and every window of the configuration."""
    from rocmforge_b200 import StepRequest
    m = engine(folders, name, dtype)
    toks = random_tokens(vocab(name), 210, 3)
    cache = m.new_cache(max_tokens=512, max_slots=2)
    poison_free_pages(cache)
    s = cache.alloc_slot()
    got = m.step(cache, [StepRequest(s, toks, range(len(toks)))]).cpu()
    close(got, plain_logits(folders, name, dtype, toks), dtype, f"{name} {dtype} whole prompt")


@pytest.mark.parametrize("name", ["RA", "RB"])
def test_token_by_token_from_the_first_token(folders, name):
    """One token a step from an empty cache and a zero state: the first tokens, every window's first full turn, a
    page border; and the same logits as the prompt in one step."""
    from rocmforge_b200 import StepRequest
    m = engine(folders, name, "float32")
    toks = random_tokens(vocab(name), 150, 5)
    ref = plain_logits(folders, name, "float32", toks)
    cache = m.new_cache(max_tokens=512, max_slots=2)
    s = cache.alloc_slot()
    got = torch.cat([m.step(cache, [StepRequest(s, [t], [0])]).cpu() for t in toks])
    close(got, ref, "float32", f"{name} token by token")
    s2 = cache.alloc_slot()
    whole = m.step(cache, [StepRequest(s2, toks, range(len(toks)))]).cpu()
    assert (got - whole).abs().max() < 2e-5


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["RA", "RB", "RC"])
def test_portions_of_many_sizes(folders, name, dtype):
    """A prompt cut into portions of 2 to 70 tokens (the state and the window's keys are carried from step to step)."""
    from rocmforge_b200 import StepRequest
    m = engine(folders, name, dtype)
    sizes = [2, 3, 64, 1, 5, 17, 2, 70, 33, 2, 1, 8]
    toks = random_tokens(vocab(name), sum(sizes), 7)
    ref = plain_logits(folders, name, dtype, toks)
    cache = m.new_cache(max_tokens=512, max_slots=2)
    poison_free_pages(cache)
    s = cache.alloc_slot()
    got, at = [], 0
    for n in sizes:
        got.append(m.step(cache, [StepRequest(s, toks[at:at + n], range(n))]).cpu())
        at += n
    close(torch.cat(got), ref, dtype, f"{name} {dtype} portions")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["RA", "RC"])
def test_ragged_batch_then_decoding_with_slots_used_again(folders, name, dtype):
    """Unequal prompts in one step, decoded together; requests end at different steps, their slots (state!) and pages go
    to new requests that join with prompts of their own; every request must equal itself alone."""
    from rocmforge_b200 import StepRequest
    m = engine(folders, name, dtype)
    V = vocab(name)
    lens = [(1, 30), (70, 12), (131, 25), (33, 6)]
    seqs = [random_tokens(V, a + b, 20 + i) for i, (a, b) in enumerate(lens)]
    refs = [plain_logits(folders, name, dtype, t) for t in seqs]
    cache = m.new_cache(max_tokens=64 * 8, max_slots=4)
    poison_free_pages(cache)
    slots = [cache.alloc_slot() for _ in lens]
    got = m.step(cache, [StepRequest(sl, t[:a], [0, a - 1]) for sl, t, (a, _) in zip(slots, seqs, lens)]).cpu()
    want = torch.stack([r[i] for r, (a, _) in zip(refs, lens) for i in (0, a - 1)])
    close(got, want, dtype, f"{name} {dtype} ragged prompts")
    live = list(range(len(lens)))
    for step in range(30):
        for i in [i for i in live if lens[i][1] <= step]:
            cache.free_slot(slots[i]); live.remove(i)
        poison_free_pages(cache)
        got = m.step(cache, [StepRequest(slots[i], [seqs[i][lens[i][0] + step]], [0]) for i in live]).cpu()
        close(got, torch.stack([refs[i][lens[i][0] + step] for i in live]), dtype,
                            f"{name} {dtype} batch decode step {step}")
    for i in live:
        cache.free_slot(slots[i])
    # the freed slots again: a state that was not zeroed or a page that kept old keys would show here
    again = [random_tokens(V, n, 40 + n) for n in (45, 9)]
    slots = [cache.alloc_slot() for _ in again]
    got = m.step(cache, [StepRequest(sl, t, range(len(t))) for sl, t in zip(slots, again)]).cpu()
    close(got, torch.cat([plain_logits(folders, name, dtype, t) for t in again]), dtype, f"{name} {dtype} reused slots")


def test_long_decoding(folders):
    """Three hundred single-token steps after a short prompt: the windows of 70 and 130 pass over decoded tokens, pages
    that left a window are handed back, the state decays by factors from 0.8 to 0.9999."""
    from rocmforge_b200 import StepRequest
    m = engine(folders, "RB", "float32")
    toks = random_tokens(vocab("RB"), 330, 9)
    ref = plain_logits(folders, "RB", "float32", toks)
    cache = m.new_cache(max_tokens=64 * 6, max_slots=1)            # the windows' pages only: fewer than the sequence needs
    s = cache.alloc_slot()
    got = [m.step(cache, [StepRequest(s, toks[:30], [29])]).cpu()]
    for t in toks[30:]:
        poison_free_pages(cache)
        got.append(m.step(cache, [StepRequest(s, [t], [0])]).cpu())
    close(torch.cat(got), ref[29:], "float32", "RB long decoding")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_greedy_generation_through_the_public_entry_point(folders, dtype):
    """LLM.generate: the scheduler admits unequal prompts, decode steps replay from graphs (the warm-up run before a
    capture must leave the state as it was), requests end at different lengths."""
    import rocmforge_b200 as rf
    name = "RC"
    llm = rf.LLM(folders(name, dtype), dtype=dtype)
    prompts = [random_tokens(vocab(name), n, 60 + n) for n in (3, 40, 11)]
    out = llm.generate(prompts, max_tokens=12, temperature=0.0, stop_token_ids=[])
    for p, r in zip(prompts, out):
        assert len(r.tokens) == 12
        seq = list(p)
        for k, tok in enumerate(r.tokens):
            row = plain_logits(folders, name, dtype, seq)[-1]
            best = int(torch.argmax(row))
            if dtype == "float32":
                assert tok == best, f"request of {len(p)} tokens, generated token {k}: {tok}, plain {best}"
            else:                                        # bfloat16: the chosen token must be (nearly) the plain model's best
                assert float(row[best] - row[tok]) <= 6e-2 * float(row.abs().max())
            seq.append(tok)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_replay_program(folders, tmp_path, dtype):
    """bin/trace_run on a Rifizen folder: whole prompts, a prompt and its last tokens one by one, and a batch."""
    name = "RA"
    V = vocab(name)
    a, b, c = random_tokens(V, 80, 71), random_tokens(V, 37, 72), random_tokens(V, 5, 73)
    ra, rb, rc = (plain_logits(folders, name, dtype, t) for t in (a, b, c))
    tr = TraceRun(folders(name, dtype), dtype, str(tmp_path / "out"), max_tokens=256)
    got = tr.step([("a", a, [0, 6, 7, 79])], end=["a"])
    close(got, ra[[0, 6, 7, 79]], dtype, "replay: whole")
    got = tr.step([("b", b[:30], [29])])
    close(got, rb[[29]], dtype, "replay: prompt")
    for i in range(30, 37):
        got = tr.step([("b", [b[i]], [0])], end=["b"] if i == 36 else [])
        close(got, rb[[i]], dtype, f"replay: decoded {i}")
    got = tr.step([("x", a[:60], [59]), ("y", c[:3], []), ("z", b[:20], [0, 19])])
    close(got, torch.stack([ra[59], rb[0], rb[19]]), dtype, "replay: batch")
    got = tr.step([("x", [a[60]], [0]), ("y", [c[3]], [0]), ("z", [b[20]], [0])], end=["y"])
    close(got, torch.stack([ra[60], rc[3], rb[20]]), dtype, "replay: batch decoded")
    assert tr.step([("x", [a[61]], []), ("z", [b[21]], [])], end=["x", "z"]) is None
    assert tr.close() == 0


# --------------------------------------------------------------------------- the kernels alone

def _paged(k, v, n_pages_extra=2):
    """One sequence's keys [T, nkv, d] and values [T, nkv, dv] as pages in a shuffled order, with its block table."""
    T, nkv, d = k.shape
    dv = v.shape[2]
    n = (T + 63) // 64
    order = torch.randperm(n + n_pages_extra)[:n]
    kp = torch.full((n + n_pages_extra, nkv, 64, d), float("nan"), device=k.device, dtype=k.dtype)
    vp = torch.full((n + n_pages_extra, nkv, 64, dv), float("nan"), device=k.device, dtype=k.dtype)
    for p in range(n):
        rows = slice(64 * p, min(T, 64 * p + 64))
        kp[order[p], :, : rows.stop - rows.start] = k[rows].transpose(0, 1)
        vp[order[p], :, : rows.stop - rows.start] = v[rows].transpose(0, 1)
    return kp, vp, order.to(torch.int32).to(k.device).reshape(1, n)


@pytest.mark.parametrize("window", [1, 5, 64, 65, 200])
def test_attention_sees_exactly_its_window(window):
    """One key stands out just inside the window and one just outside (their scores are the largest by far): the output
    is the inside key's value, and not a trace of the outside key's.  Queries in a prompt and alone, heads of 24 with
    values of 40."""
    from rocmforge_b200 import kernels
    torch.manual_seed(window)
    dev, T, nh, nkv, d, dv = "cuda", 300, 4, 2, 24, 40
    q = torch.randn(T, nh, d, device=dev) * 0.1
    k = torch.randn(T, nkv, d, device=dev) * 0.1
    v = torch.randn(T, nkv, dv, device=dev)
    i = T - 1
    inside, outside = i - window + 1, i - window
    q[i] = 0.0
    q[i, :, 0] = 30.0
    k[inside, :, 0] = 1.0
    k[outside, :, 0] = 2.0                       # would win if it were seen
    v[outside] = 1000.0
    kp, vp, bt = _paged(k, v)
    zero = torch.zeros(1, dtype=torch.int32, device=dev)
    for rows in (range(T), [i]):                 # the whole prompt, and the last query as a step of its own
        pos = torch.tensor(list(rows), dtype=torch.int32, device=dev)
        seq = torch.zeros(len(pos), dtype=torch.int32, device=dev)
        out = kernels.attention_generic(q[list(rows)].reshape(len(pos), nh * d).contiguous(), nh, nkv, d, kp, vp, seq, pos,
                                        zero, bt, 1.0, window, v_head_dim=dv).reshape(len(pos), nh, dv)
        want = v[inside][[0, 0, 1, 1]] if window > 1 else v[i][[0, 0, 1, 1]]
        assert (out[-1] - want).abs().max() < 1e-3, f"window {window}: the query sees the wrong keys"


def test_attention_cap_and_distance_bias_against_torch():
    from rocmforge_b200 import kernels
    torch.manual_seed(0)
    dev, T, nh, nkv, d, dv, window, cap, scale = "cuda", 150, 6, 3, 20, 12, 70, 3.0, 0.7
    q, k, v = torch.randn(T, nh, d, device=dev), torch.randn(T, nkv, d, device=dev), torch.randn(T, nkv, dv, device=dev)
    slopes = torch.tensor(P.distance_slopes(nh), dtype=torch.float32, device=dev)
    kp, vp, bt = _paged(k, v)
    pos = torch.arange(T, dtype=torch.int32, device=dev)
    zeros = torch.zeros(T, dtype=torch.int32, device=dev)
    out = kernels.attention_generic(q.reshape(T, -1).contiguous(), nh, nkv, d, kp, vp, zeros, pos, zeros[:1], bt, scale, window,
                                    v_head_dim=dv, softcap=cap, slopes=slopes).reshape(T, nh, dv)
    qd, kd, vd = q.double().cpu(), k.double().cpu(), v.double().cpu()
    for h in range(nh):
        s = (qd[:, h] @ kd[:, h // 2].T) * scale
        s = cap * torch.tanh(s / cap)
        ii, jj = torch.arange(T)[:, None], torch.arange(T)[None, :]
        s = s - slopes[h].item() * (ii - jj)
        s = s.masked_fill((jj > ii) | (ii - jj >= window), float("-inf"))
        want = torch.softmax(s, dim=1) @ vd[:, h // 2]
        assert (out[:, h].double().cpu() - want).abs().max() < 1e-4


@pytest.mark.parametrize("dim,vdim,heads", [(24, 12, 2), (64, 32, 3), (130, 9, 1), (256, 16, 1)])
def test_retention_scan_against_the_recurrence_and_across_cuts(dim, vdim, heads):
    """The recurrence over 700 tokens of two sequences, once in one step and once cut into steps of many sizes (down to
    one token): the same bits, and the plain recurrence's numbers.  A token 650 places back, made large, still shows."""
    from rocmforge_b200 import kernels
    torch.manual_seed(dim)
    dev, T = "cuda", 700
    decay = torch.tensor(([1.0, 0.5, 0.999] * 3)[:heads], dtype=torch.float32, device=dev)
    state = torch.zeros(3, heads, vdim, dim, device=dev)           # kept transposed: a value dimension's column is contiguous
    qk = torch.randn(2, 2 * T, heads * dim, device=dev) * dim ** -0.5
    v = torch.randn(2 * T, heads * vdim, device=dev)
    v[20] *= 50.0
    cu = torch.tensor([0, T, 2 * T], dtype=torch.int32, device=dev)
    slots = torch.tensor([2, 0], dtype=torch.int32, device=dev)
    whole = kernels.retention_scan(qk, v, state, decay, cu, slots, heads, dim, vdim)
    end_state = state.clone()
    # plain recurrence for the first sequence, in double
    S = torch.zeros(heads, dim, vdim, dtype=torch.float64)
    q64, k64, v64 = qk[0, :T].double().cpu().reshape(T, heads, dim), qk[1, :T].double().cpu().reshape(T, heads, dim), v[:T].double().cpu().reshape(T, heads, vdim)
    d64 = decay.double().cpu()[:, None, None]
    want = torch.zeros(T, heads, vdim, dtype=torch.float64)
    for t in range(T):
        S = d64 * S + k64[t][:, :, None] * v64[t][:, None, :]
        want[t] = torch.einsum("hdv,hd->hv", S, q64[t])
    got = whole[:T].double().cpu().reshape(T, heads, vdim)
    assert (got - want).abs().max() <= 1e-4 * want.abs().max()
    assert (end_state[2].double().cpu().transpose(-1, -2) - S).abs().max() <= 1e-4 * S.abs().max()
    assert (state[1] == 0).all()                                  # a slot that no sequence of the step holds
    # the same in portions
    state.zero_()
    sizes = [1, 2, 16, 17, 1, 63, 300, 5]
    sizes.append(T - sum(sizes))
    parts, at = [], 0
    for n in sizes:
        rows = torch.cat([torch.arange(at, at + n), torch.arange(T + at, T + at + n)]).to(dev)
        cu_n = torch.tensor([0, n, 2 * n], dtype=torch.int32, device=dev)
        parts.append(kernels.retention_scan(qk[:, rows].contiguous(), v[rows], state, decay, cu_n, slots, heads, dim, vdim))
        at += n
    cut = torch.cat([p[: p.shape[0] // 2] for p in parts] + [p[p.shape[0] // 2:] for p in parts])
    assert torch.equal(cut, whole), "the recurrence depends on how the prompt was cut"
    assert torch.equal(state, end_state)


def test_retention_rotation_and_gate_against_torch():
    from rocmforge_b200 import kernels
    torch.manual_seed(1)
    dev, T, heads, dim, vdim, rot = "cuda", 40, 3, 24, 10, 8
    width = 2 * heads * dim + 2 * heads * vdim
    for dt in (torch.float32, torch.bfloat16):
        proj = torch.randn(T, width, device=dev).to(dt)
        pos = torch.randint(0, 5000, (T,), dtype=torch.int32, device=dev)
        inv_freq = (1.0 / torch.pow(torch.tensor(100.0, dtype=torch.float64), 2.0 * torch.arange(rot // 2, dtype=torch.float64) / rot)).float().to(dev)
        qk = kernels.retention_prepare(proj, 0, heads * dim, heads, dim, rot, inv_freq, pos, 0.25)
        x = proj.float().cpu()
        for which, scale in ((0, 1.0), (1, 0.25)):
            src = x[:, which * heads * dim:(which + 1) * heads * dim].reshape(T, heads, dim).double()
            want = P.rotate_half_layout(src, pos.cpu(), rot, 100.0) * scale
            assert (qk[which].cpu().reshape(T, heads, dim).double() - want).abs().max() < 2e-5
        o = torch.randn(T, heads * vdim, device=dev)
        gate = proj[:, 2 * heads * dim + heads * vdim:]
        got = kernels.retention_gate(o, gate, heads, vdim, 1e-5).float().cpu().reshape(T, heads, vdim)
        want = P.unit_rms(o.cpu().double().reshape(T, heads, vdim), 1e-5) * P.silu(gate.float().cpu().double().reshape(T, heads, vdim))
        assert (got - want).abs().max() < (1e-5 if dt == torch.float32 else 1e-2 * float(want.abs().max()))


@pytest.mark.parametrize("H", [64, 200, 4096])
def test_branch_norm_add_against_torch(H):
    from rocmforge_b200 import kernels
    torch.manual_seed(H)
    dev, T, eps = "cuda", 37, 1e-5
    for wdt in (torch.float32, torch.bfloat16):
        h = torch.randn(T, H, device=dev)
        a, b = torch.randn(T, H, device=dev) * 3, torch.randn(T, H, device=dev) * 0.01
        wa, wb, wp, wn, ex = (torch.randn(H, device=dev).to(wdt) for _ in range(5))
        f = lambda t: t.double().cpu()
        # two branches, an extra row and the next norm
        h2 = h.clone()
        y = kernels.branch_norm_add(h2, [(a, wa), (b, wb)], wp, eps, torch.float32, extra=ex, next_weight=wn)
        m = 0.5 * (P.rms_norm(f(a), f(wa), eps) + P.rms_norm(f(b), f(wb), eps))
        want_h = f(h) + P.rms_norm(m, f(wp), eps) + f(ex)
        assert (f(h2) - want_h).abs().max() < 1e-4
        assert (f(y) - P.rms_norm(want_h, f(wn), eps)).abs().max() < 1e-4
        # a branch as a stack of partial sums
        h4 = h.clone()
        parts = torch.stack([a * 0.5, a * 0.25, a * 0.25])
        kernels.branch_norm_add(h4, [(parts, wa), (b, wb)], wp, eps, torch.float32, extra=ex)
        assert (f(h4) - want_h).abs().max() < 1e-4
        # one branch, nothing else
        h3 = h.clone()
        assert kernels.branch_norm_add(h3, [(a, None)], wp, eps, torch.float32) is None
        assert (f(h3) - (f(h) + P.rms_norm(f(a), f(wp), eps))).abs().max() < 1e-4


@pytest.mark.parametrize("T,E,top", [(1, 5, 2), (50, 8, 1), (300, 6, 3), (33, 40, 16)])
def test_routing_and_grouped_products_against_torch(T, E, top):
    """Routing, the sort by expert, both grouped products and the weighted sum, against a loop over tokens."""
    from rocmforge_b200 import kernels
    torch.manual_seed(T)
    dev, H, F = "cuda", 48, 20
    y = torch.randn(T, H, device=dev)
    z = torch.randn(T, E, device=dev)
    gate_up = torch.randn(E, 2 * F, H, device=dev) * 0.2
    down = torch.randn(E, H, F, device=dev) * 0.2
    idx, w = kernels.moe_route(z, top)
    vals, ref_idx = torch.topk(z, top, dim=1)
    assert torch.equal(idx.long(), ref_idx)
    assert (w - torch.softmax(vals, dim=1)).abs().max() < 1e-6
    for rows in (kernels.MOE_TILE_SMALL, kernels.MOE_TILE_LARGE):
        perm, inv, tiles, max_tiles = kernels.moe_sort(idx, E, rows)
        flat = idx.reshape(-1)
        assert torch.equal(torch.sort(perm.long()).values, torch.arange(T * top, device=dev))
        assert (flat[perm.long()][1:] >= flat[perm.long()][:-1]).all()            # sorted by expert
        assert torch.equal(perm[inv.long()].long(), torch.arange(T * top, device=dev))
        gu = kernels.gemm_simt_grouped(y, gate_up, tiles, max_tiles, rows, T * top, row_map=perm, row_div=top)
        a = kernels.swiglu(gu)
        d = kernels.gemm_simt_grouped(a, down, tiles, max_tiles, rows, T * top, out_f32=True)
        out = kernels.moe_combine(d, inv, w)
        want = torch.zeros(T, H, dtype=torch.float64)
        for t in range(T):
            for kk in range(top):
                e = int(idx[t, kk])
                g = gate_up[e].double().cpu() @ y[t].double().cpu()
                act = P.silu(g[0::2]) * g[1::2]
                want[t] += float(w[t, kk]) * (down[e].double().cpu() @ act)
        assert (out.double().cpu() - want).abs().max() < 1e-4


def test_head_norm_and_cache_write_against_torch():
    """Query and key heads divided by their root mean square (values not), then into the cache's pages; from one
    tensor and from a stack of partial sums."""
    from rocmforge_b200 import kernels
    torch.manual_seed(2)
    dev, T, nh, nkv, d, dv, eps = "cuda", 70, 4, 2, 24, 40, 1e-3
    width = (nh + nkv) * d + nkv * dv
    parts = torch.randn(3, T, width, device=dev)
    qkv = parts.sum(0)
    pos = torch.arange(T, dtype=torch.int32, device=dev)
    zeros = torch.zeros(T, dtype=torch.int32, device=dev)
    bt = torch.tensor([[3, 1]], dtype=torch.int32, device=dev)
    for src in (qkv, parts):
        kp = torch.zeros(4, nkv, 64, d, device=dev)
        vp = torch.zeros(4, nkv, 64, dv, device=dev)
        q = kernels.head_norm_kv_write(src, nh, nkv, d, dv, None, zeros, pos, zeros[:1], bt, kp, vp,
                                       compute_dtype=torch.float32, unit_norm_eps=eps)
        x = qkv.double().cpu()
        want_q = P.unit_rms(x[:, :nh * d].reshape(T, nh, d), eps)
        want_k = P.unit_rms(x[:, nh * d:(nh + nkv) * d].reshape(T, nkv, d), eps)
        want_v = x[:, (nh + nkv) * d:].reshape(T, nkv, dv)
        assert (q.double().cpu().reshape(T, nh, d) - want_q).abs().max() < 1e-5
        got_k = torch.cat([kp[3], kp[1]], dim=1)[:, :T].transpose(0, 1).double().cpu()
        got_v = torch.cat([vp[3], vp[1]], dim=1)[:, :T].transpose(0, 1).double().cpu()
        assert (got_k - want_k).abs().max() < 1e-5 and (got_v - want_v).abs().max() < 1e-5


@pytest.mark.parametrize("T,E,top,H,F", [(1, 5, 2, 64, 32), (300, 6, 3, 128, 72), (700, 4, 1, 256, 160)])
def test_grouped_tensor_core_products_against_the_cuda_core_ones(T, E, top, H, F):
    """bfloat16: tiles of 128 sorted rows against their expert's matrices on the tensor cores (the gated activation in the
    first product's epilogue), against the same routing through the CUDA-core grouped products."""
    from rocmforge_b200 import kernels
    tc = kernels.tensor_core
    torch.manual_seed(T)
    dev = "cuda"
    y = torch.randn(T, H, device=dev).to(torch.bfloat16)
    idx, w = kernels.moe_route(torch.randn(T, E, device=dev), top)
    gate_up = (torch.randn(E, 2 * F, H, device=dev) * 0.2).to(torch.bfloat16)
    down = (torch.randn(E, H, F, device=dev) * 0.2).to(torch.bfloat16)
    perm, inv, tiles, max_tiles = kernels.moe_sort(idx, E, kernels.MOE_TILE_TC)
    a = tc.gemm_tc_grouped(kernels.moe_gather(y, perm, top), gate_up, tiles, max_tiles, mode=tc.SWIGLU)
    got = kernels.moe_combine(tc.gemm_tc_grouped(a, down, tiles, max_tiles, mode=tc.F32), inv, w)
    perm2, inv2, tiles2, max2 = kernels.moe_sort(idx, E, kernels.MOE_TILE_LARGE)
    a2 = kernels.swiglu(kernels.gemm_simt_grouped(y, gate_up, tiles2, max2, kernels.MOE_TILE_LARGE, T * top, row_map=perm2, row_div=top))
    want = kernels.moe_combine(kernels.gemm_simt_grouped(a2, down, tiles2, max2, kernels.MOE_TILE_LARGE, T * top, out_f32=True), inv2, w)
    assert (got - want).abs().max() <= 2e-2 * want.abs().max()
    tc.check_status(dev)


@pytest.mark.parametrize("window", [1, 7, 40, 100, 1000])
@pytest.mark.parametrize("hd", [64, 128])
def test_tensor_core_prompt_attention_with_cap_and_slopes(hd, window):
    """bfloat16 prompts of two sequences (one continuing a cached context) with capped scores, distance slopes and windows
    from one key to more than the prompt: the tcgen05 kernel against the generic one."""
    from rocmforge_b200 import kernels
    torch.manual_seed(hd)
    dev, nh, nkv, cap, scale = "cuda", 4, 2, 6.0, 0.4
    lens, starts = [300, 150], [0, 70]
    T = sum(lens)
    total = [s + n for s, n in zip(starts, lens)]
    k = [torch.randn(t, nkv, hd, device=dev).to(torch.bfloat16) for t in total]
    v = [torch.randn(t, nkv, hd, device=dev).to(torch.bfloat16) for t in total]
    n_pages = [(t + 63) // 64 for t in total]
    kp = torch.zeros(sum(n_pages) + 1, nkv, 64, hd, device=dev, dtype=torch.bfloat16)
    vp = torch.zeros_like(kp)
    bt = torch.zeros(2, max(n_pages), dtype=torch.int32, device=dev)
    page = 1
    for b in range(2):
        for p in range(n_pages[b]):
            rows = slice(64 * p, min(total[b], 64 * p + 64))
            kp[page, :, : rows.stop - rows.start] = k[b][rows].transpose(0, 1)
            vp[page, :, : rows.stop - rows.start] = v[b][rows].transpose(0, 1)
            bt[b, p] = page
            page += 1
    q = (torch.randn(T, nh * hd, device=dev) * 0.5).to(torch.bfloat16)
    i32 = lambda x: torch.tensor(x, dtype=torch.int32, device=dev)
    tok_seq = i32([0] * lens[0] + [1] * lens[1])
    tok_pos = i32(list(range(starts[0], total[0])) + list(range(starts[1], total[1])))
    slopes = torch.tensor(P.distance_slopes(nh), dtype=torch.float32, device=dev) * 4
    want = kernels.attention_generic(q, nh, nkv, hd, kp, vp, tok_seq, tok_pos, i32([0, 1]), bt, scale, window, softcap=cap, slopes=slopes)
    tiles = sorted([(b, q0) for b in range(2) for q0 in range(0, lens[b], 128)], key=lambda t: starts[t[0]] + t[1])
    got = kernels.attention_prefill_tc(q, nh, nkv, hd, kp, vp, i32([x for t in tiles for x in t]), i32([0, 1]), i32(starts), i32(lens),
                                       i32([0, lens[0], T]), bt, scale, window, softcap=cap, slopes=slopes)
    assert (got.float() - want.float()).abs().max() < 3e-2
    kernels.tensor_core.check_status(dev)


@pytest.mark.parametrize("dim,vdim,heads", [(24, 12, 2), (128, 128, 2), (200, 70, 1)])
def test_chunked_retention_against_the_token_by_token_kernel(dim, vdim, heads):
    """Prompts of 1 to 300 new tokens in one step (chunks of 64 side by side, states carried between them, a state that an
    earlier step left) against the scan; the two differ by rounding alone."""
    from rocmforge_b200 import kernels
    torch.manual_seed(dim)
    dev = "cuda"
    lens = [300, 1, 64, 65, 130]
    T, B = sum(lens), len(lens)
    decay = torch.tensor(([1.0, 0.6, 0.999] * 3)[:heads], dtype=torch.float32, device=dev)
    state0 = torch.randn(B + 2, heads, vdim, dim, device=dev)
    qk = torch.randn(2, T, heads * dim, device=dev) * dim ** -0.5
    v = torch.randn(T, heads * vdim, device=dev)
    cu = torch.tensor([0] + list(np.cumsum(lens)), dtype=torch.int32, device=dev)
    slots = torch.tensor([3, 0, 6, 1, 4], dtype=torch.int32, device=dev)
    s_scan, s_chunk = state0.clone(), state0.clone()
    want = kernels.retention_scan(qk, v, s_scan, decay, cu, slots, heads, dim, vdim)
    counts = [(n + 63) // 64 for n in lens]
    table = list(np.concatenate([[0], np.cumsum(counts)])) + [x for b, n in enumerate(lens) for q0 in range(0, n, 64) for x in (b, q0)]
    got = kernels.retention_chunked(qk, v, s_chunk, decay, torch.tensor(table, dtype=torch.int32, device=dev), cu, slots, heads, dim, vdim)
    assert (got - want).abs().max() <= 2e-5 * want.abs().max()
    assert (s_chunk - s_scan).abs().max() <= 2e-5 * s_scan.abs().max()
    assert torch.equal(s_chunk[2], state0[2]) and torch.equal(s_chunk[5], state0[5])        # slots of no sequence of the step


@pytest.mark.parametrize("window", [1, 40, 300])
@pytest.mark.parametrize("hd,nh,nkv", [(64, 8, 2), (128, 4, 4), (128, 6, 1)])
def test_clustered_decode_attention_with_cap_and_slopes(hd, nh, nkv, window):
    """bfloat16, one new token per sequence at contexts of 1 to 700 with windows of 1, 40 and 300, capped scores and
    distance slopes: the clustered kernel (1, 2 and 4 CTAs a pair) against the generic one."""
    from rocmforge_b200 import kernels
    torch.manual_seed(hd + nh)
    dev, cap, scale = "cuda", 6.0, 0.4
    ctx_len = [1, 63, 64, 65, 299, 300, 301, 700]
    B = len(ctx_len)
    n_pages = [(t + 63) // 64 for t in ctx_len]
    kp = (torch.randn(sum(n_pages) + 1, nkv, 64, hd, device=dev)).to(torch.bfloat16)
    vp = (torch.randn(sum(n_pages) + 1, nkv, 64, hd, device=dev)).to(torch.bfloat16)
    bt = torch.zeros(B, max(n_pages), dtype=torch.int32, device=dev)
    page = 1
    for b in range(B):
        for p in range(n_pages[b]):
            bt[b, p] = page
            page += 1
    q = (torch.randn(B, nh * hd, device=dev) * 0.5).to(torch.bfloat16)
    i32 = lambda x: torch.tensor(x, dtype=torch.int32, device=dev)
    tok_seq, tok_pos, slot = i32(list(range(B))), i32([t - 1 for t in ctx_len]), i32(list(range(B)))
    slopes = torch.tensor(P.distance_slopes(nh), dtype=torch.float32, device=dev) * 4
    want = kernels.attention_generic(q, nh, nkv, hd, kp, vp, tok_seq, tok_pos, slot, bt, scale, window, softcap=cap, slopes=slopes)
    for splits in (1, 2, 4):
        got = kernels.attention_decode_warps(q, nh, nkv, hd, kp, vp, tok_seq, tok_pos, slot, bt, scale, window, splits=splits,
                                             softcap=cap, slopes=slopes)
        assert (got.float() - want.float()).abs().max() < 3e-2, f"{splits} CTAs a pair"
    kernels.tensor_core.check_status(dev)


def test_command_line_generates_with_this_design(folders):
    """bin/rocmforge on a Rifizen folder: greedy tokens as the plain model picks them, sampled tokens with top-p, and the
    statistics; the same flags as for any other model."""
    import subprocess
    import sys
    from helpers import ROOT
    name = "RA"
    prompt = random_tokens(vocab(name), 9, 81)
    exe = [sys.executable, os.path.join(ROOT, "bin", "rocmforge"), "--model", folders(name, "float32"), "--dtype", "float32"]
    out = subprocess.run(exe + ["--prompt-ids", ",".join(map(str, prompt)), "--max-tokens", "6", "--temperature", "0",
                                "--stop-ids", "", "--debug"], capture_output=True, text=True)
    assert out.returncode == 0, out.stderr
    got = [int(l.split("token_id=")[1]) for l in out.stderr.splitlines() if l.startswith("[Generated]")]
    seq = list(prompt)
    for tok in got:
        assert tok == int(torch.argmax(plain_logits(folders, name, "float32", seq)[-1]))
        seq.append(tok)
    assert len(got) == 6 and "ended by max_tokens" in out.stderr
    js = subprocess.run(exe + ["--prompt-len", "70", "--prompt-len", "3", "--max-tokens", "5", "--temperature", "0.8", "--top-p", "0.9",
                               "--stop-ids", "", "--stats-json", "-"], capture_output=True, text=True)
    assert js.returncode == 0, js.stderr
    stats = json.loads(js.stdout.strip().splitlines()[-1])
    assert stats["prompt_tokens"] == 73 and stats["generated_tokens"] == 10

"""The Vilulorn decoder in the engine against the plain implementation (needs a GPU): whole prompts, token-by-token
decoding, portions, ragged batches, slots and pages used again, long decoding over chunk edges, generation through the
public entry point and the command line, the replay program; then each mechanism's kernels alone against the plain
functions, with inputs made so that a key one place off, a lost state or a missing gate shows."""
import json
import os
import subprocess

import numpy as np
import pytest
import torch

from helpers import ROOT, VILULORN_CONFIGS, TraceRun, random_tokens
from plain import vilulorn_plain as P

pytestmark = pytest.mark.gpu

TORCH = {"float32": torch.float32, "bfloat16": torch.bfloat16}
_models, _plains, _refs = {}, {}, {}


def engine(folders, name, dtype):
    import rocmforge_b200 as rf
    if (name, dtype) not in _models:
        _models[(name, dtype)] = rf.Model.from_folder(folders(name, dtype), dtype=TORCH[dtype])
    return _models[(name, dtype)]


def plain_model(folders, name, dtype):
    from safetensors.torch import load_file
    if (name, dtype) not in _plains:
        folder = folders(name, dtype)
        _plains[(name, dtype)] = P.PlainVilulorn(json.load(open(os.path.join(folder, "config.json"))),
                                                 load_file(os.path.join(folder, "model.safetensors")))
    return _plains[(name, dtype)]


def plain_logits(folders, name, dtype, tokens):
    """Logits of the plain model on the folder's stored (rounded) weights, every position."""
    key = (name, dtype, tuple(tokens))
    if key not in _refs:
        _refs[key] = plain_model(folders, name, dtype).logits(list(tokens))
    return _refs[key]


def row_errors(got, ref):
    """Per row: root mean square of the difference (mean taken off) over the root mean square of the reference logits."""
    got = torch.as_tensor(np.asarray(got), dtype=torch.float64)
    ref = torch.as_tensor(np.asarray(ref), dtype=torch.float64)
    assert got.shape == ref.shape and torch.isfinite(got).all()
    d = got - ref
    d = d - d.mean(dim=-1, keepdim=True)
    return d.pow(2).mean(dim=-1).sqrt() / (ref - ref.mean(dim=-1, keepdim=True)).pow(2).mean().sqrt()


def close(got, ref, dtype, what):
    """float32: element by element (6e-5 + 3e-4 |reference|).  bfloat16 (with the experts' choice agreed, see ``routed_like_the_engine``): rows
    within 2.5 % on average by the root mean square of their difference, and none beyond 15 %: every layer norms its
    sub-layers' outputs to unit size, which carries one layer's rounding at full size into the next, and blows the
    rounding of a sub-layer's output up where that output happens to be small."""
    if dtype == "float32":
        # three times the other models' bound: an out-norm divides a sub-layer's output by its size, and where that output
        # is small (experts whose clamped halves nearly cancel) the 32-bit rounding of its sums is divided with it
        g = torch.as_tensor(np.asarray(got), dtype=torch.float64)
        r = torch.as_tensor(np.asarray(ref), dtype=torch.float64)
        assert g.shape == r.shape and torch.isfinite(g).all(), what
        bad = (g - r).abs() > 6e-5 + 3e-4 * r.abs()
        assert not bad.any(), f"{what}: {int(bad.sum())} of {bad.numel()} logits differ, max diff {float((g - r).abs().max()):.3g}"
        return
    err = row_errors(got, ref)
    assert float(err.mean()) < 0.025 and float(err.max()) < 0.15, \
        f"{what}: row errors up to {float(err.max()):.3f} (row {int(err.argmax())}), mean {float(err.mean()):.3f}"


class routed_like_the_engine:
    """With random weights a token's best experts are now and then nearly tied, and the bfloat16 engine, whose router
    sees rounded activations, takes another one than the plain model: that row is then off by its whole size, and through
    the recurrent state so are, a little, all rows after it.  So the comparison is done in two halves.  Inside this
    context every choice of the engine's router is recorded (``kernels.moe_route`` is wrapped); ``logits`` then runs the
    plain model with those choices forced on it (the scores stay its own) and checks that the engine's choices are the
    plain model's own wherever the plain model's margin (2 % of the logits' spread) is not small."""

    def __init__(self, monkeypatch):
        from rocmforge_b200 import kernels
        self.calls = []
        real = kernels.moe_route

        def recording(z, top, scoring="softmax_of_chosen"):
            idx, w = real(z, top, scoring)
            self.calls.append(idx)
            return idx, w
        monkeypatch.setattr(kernels, "moe_route", recording)

    def logits(self, plain, tokens, steps=1):
        """The plain model's logits for ``tokens`` (one sequence, run through the engine in ``steps`` steps inside this
        context), routed as the engine routed."""
        moe_layers = [i for i, L in enumerate(plain.cfg["layers"]) if L.get("mlp") is not None]
        assert len(self.calls) == steps * len(moe_layers)
        forced = {layer: torch.cat([self.calls[s * len(moe_layers) + n] for s in range(steps)]).cpu()
                  for n, layer in enumerate(moe_layers)}
        chosen = {}
        out = plain.logits(list(tokens), forced=forced, chosen=chosen)
        # where the plain model's margin is clear, the engine chose the same set
        clear = agree = 0
        for layer in moe_layers:
            for t, (own, margin) in enumerate(chosen[layer]):
                if margin > 0.02:
                    clear += 1
                    agree += set(own) == set(int(e) for e in forced[layer][t])
        assert clear == 0 or agree >= 0.995 * clear, f"the engine's router differs from the plain one on {clear - agree} of {clear} clear calls"
        self.calls.clear()
        return out


def vocab(name):
    return VILULORN_CONFIGS[name]["vocab"]


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
@pytest.mark.parametrize("name", ["VA", "VB", "VC", "VD", "VE"])
def test_whole_prompt(folders, name, dtype, monkeypatch):
    """Every position of a prompt that crosses four page borders and every chunk edge of the configuration."""
    from rocmforge_b200 import StepRequest
    m = engine(folders, name, dtype)
    toks = random_tokens(vocab(name), 270, 3)
    cache = m.new_cache(max_tokens=512, max_slots=2)
    poison_free_pages(cache)
    s = cache.alloc_slot()
    routes = routed_like_the_engine(monkeypatch)
    got = m.step(cache, [StepRequest(s, toks, range(len(toks)))]).cpu()
    ref = plain_logits(folders, name, dtype, toks) if dtype == "float32" else routes.logits(plain_model(folders, name, dtype), toks)
    close(got, ref, dtype, f"{name} {dtype} whole prompt")


@pytest.mark.parametrize("name", ["VA", "VB"])
def test_token_by_token_from_the_first_token(folders, name):
    """One token a step from an empty cache and a zero state: the first tokens, every chunk's first position, a page
    border; and the same logits as the prompt in one step."""
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
@pytest.mark.parametrize("name", ["VA", "VB", "VC", "VD", "VE"])
def test_portions_of_many_sizes(folders, name, dtype, monkeypatch):
    """A prompt cut into portions of 1 to 70 tokens: the state is carried from step to step, and chunks are counted from
    the sequence's first position, not from where a portion starts."""
    from rocmforge_b200 import StepRequest
    m = engine(folders, name, dtype)
    sizes = [2, 3, 64, 1, 5, 17, 2, 70, 33, 2, 1, 8, 40]
    toks = random_tokens(vocab(name), sum(sizes), 7)
    cache = m.new_cache(max_tokens=512, max_slots=2)
    poison_free_pages(cache)
    s = cache.alloc_slot()
    routes = routed_like_the_engine(monkeypatch)
    got, at = [], 0
    for n in sizes:
        got.append(m.step(cache, [StepRequest(s, toks[at:at + n], range(n))]).cpu())
        at += n
    ref = (plain_logits(folders, name, dtype, toks) if dtype == "float32"
           else routes.logits(plain_model(folders, name, dtype), toks, steps=len(sizes)))
    close(torch.cat(got), ref, dtype, f"{name} {dtype} portions")


def alone(m, tokens, n_prompt):
    """A request through the engine by itself: its prompt in one step, the rest token by token; logits of every position
    from the prompt's last on, and of the prompt's first."""
    from rocmforge_b200 import StepRequest
    cache = m.new_cache(max_tokens=512, max_slots=1)
    s = cache.alloc_slot()
    rows = {}
    first = m.step(cache, [StepRequest(s, tokens[:n_prompt], [0, n_prompt - 1])]).cpu()
    rows[0], rows[n_prompt - 1] = first[0], first[-1]
    for i in range(n_prompt, len(tokens)):
        rows[i] = m.step(cache, [StepRequest(s, [tokens[i]], [0])]).cpu()[0]
    return rows


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["VA", "VC", "VD", "VE"])
def test_ragged_batch_then_decoding_with_slots_used_again(folders, name, dtype):
    """Unequal prompts in one step, decoded together; requests end at different steps, their slots (state!) and pages go
    to new requests; every request must equal itself alone: the plain model's logits on the 32-bit path; on the bfloat16
    path the engine's own for the request by itself (nearly tied experts make single rows of the bfloat16 engine differ
    from the plain model, see ``routed_like_the_engine``; between two schedules of the same engine that is rare, so nine
    rows in ten must agree to 2 % and the rest may differ)."""
    from rocmforge_b200 import StepRequest
    m = engine(folders, name, dtype)
    V = vocab(name)
    lens = [(1, 30), (70, 12), (131, 25), (33, 6)]
    seqs = [random_tokens(V, a + b, 20 + i) for i, (a, b) in enumerate(lens)]
    if dtype == "float32":
        refs = [plain_logits(folders, name, dtype, t) for t in seqs]
    else:
        refs = [alone(m, t, a) for t, (a, _) in zip(seqs, lens)]
    errs = []

    def compare(got, want, what):
        if dtype == "float32":
            close(got, want, dtype, what)
        else:
            errs.extend(row_errors(got, want).tolist())
    cache = m.new_cache(max_tokens=64 * 8, max_slots=4)
    poison_free_pages(cache)
    slots = [cache.alloc_slot() for _ in lens]
    got = m.step(cache, [StepRequest(sl, t[:a], [0, a - 1]) for sl, t, (a, _) in zip(slots, seqs, lens)]).cpu()
    want = torch.stack([r[i] for r, (a, _) in zip(refs, lens) for i in (0, a - 1)])
    compare(got, want, f"{name} {dtype} ragged prompts")
    live = list(range(len(lens)))
    for step in range(30):
        for i in [i for i in live if lens[i][1] <= step]:
            cache.free_slot(slots[i]); live.remove(i)
        poison_free_pages(cache)
        got = m.step(cache, [StepRequest(slots[i], [seqs[i][lens[i][0] + step]], [0]) for i in live]).cpu()
        compare(got, torch.stack([refs[i][lens[i][0] + step] for i in live]), f"{name} {dtype} batch decode step {step}")
    for i in live:
        cache.free_slot(slots[i])
    # the freed slots again: a state that was not zeroed or a page that kept old keys would show here
    again = [random_tokens(V, n, 40 + n) for n in (45, 9)]
    slots = [cache.alloc_slot() for _ in again]
    got = m.step(cache, [StepRequest(sl, t, [0, len(t) - 1]) for sl, t in zip(slots, again)]).cpu()
    if dtype == "float32":
        want = torch.cat([plain_logits(folders, name, dtype, t)[[0, len(t) - 1]] for t in again])
    else:
        want = torch.stack([r[i] for t in again for r in [alone(m, t, len(t))] for i in (0, len(t) - 1)])
    compare(got, want, f"{name} {dtype} reused slots")
    if errs:
        errs = torch.tensor(errs)
        assert float((errs < 0.02).double().mean()) >= 0.9 and float(errs.median()) < 0.01, \
            f"{name} bfloat16: batch against alone, median row error {float(errs.median()):.4f}, {int((errs >= 0.02).sum())} of {errs.numel()} rows over 2 %"


def test_a_batch_changes_nothing_beyond_rounding(folders):
    """A request's logits in a batch of unequal requests equal its logits alone up to the order of 32-bit sums (products of
    few tokens cut K into partial sums, products of many do not), in the prompt step and in decoding."""
    from rocmforge_b200 import StepRequest
    m = engine(folders, "VB", "float32")
    V = vocab("VB")
    seqs = [random_tokens(V, n, 80 + n) for n in (150, 3, 77)]
    cache = m.new_cache(max_tokens=64 * 12, max_slots=6)
    alone = []
    for t in seqs:
        s = cache.alloc_slot()
        a = [m.step(cache, [StepRequest(s, t[:-2], [len(t) - 3])]).cpu()]
        a += [m.step(cache, [StepRequest(s, [x], [0])]).cpu() for x in t[-2:]]
        alone.append(torch.cat(a))
        cache.free_slot(s)
    slots = [cache.alloc_slot() for _ in seqs]
    tog = [m.step(cache, [StepRequest(sl, t[:-2], [len(t) - 3]) for sl, t in zip(slots, seqs)]).cpu()]
    tog += [m.step(cache, [StepRequest(sl, [t[k]], [0]) for sl, t in zip(slots, seqs)]).cpu() for k in (-2, -1)]
    for i in range(len(seqs)):
        assert (torch.stack([x[i] for x in tog]) - alone[i]).abs().max() < 2e-5, f"request {i} depends on its batch"


def test_long_decoding_over_chunk_edges(folders):
    """Three hundred single-token steps after a short prompt, two sequences side by side: chunks of 100 end and begin
    among decoded tokens, pages of finished chunks are handed back (the two sequences have twelve pages' worth of tokens,
    the cache has seven pages), the state runs on."""
    from rocmforge_b200 import StepRequest
    m = engine(folders, "VB", "float32")
    a, b = random_tokens(vocab("VB"), 330, 9), random_tokens(vocab("VB"), 330, 10)
    ra, rb = plain_logits(folders, "VB", "float32", a), plain_logits(folders, "VB", "float32", b)
    cache = m.new_cache(max_tokens=64 * 7, max_slots=2)
    sa, sb = cache.alloc_slot(), cache.alloc_slot()
    got = [m.step(cache, [StepRequest(sa, a[:30], [29]), StepRequest(sb, b[:30], [29])]).cpu()]
    for x, y in zip(a[30:], b[30:]):
        poison_free_pages(cache)
        got.append(m.step(cache, [StepRequest(sa, [x], [0]), StepRequest(sb, [y], [0])]).cpu())
    got = torch.stack(got)
    close(got[:, 0], ra[29:], "float32", "VB long decoding, first sequence")
    close(got[:, 1], rb[29:], "float32", "VB long decoding, second sequence")


def test_a_lender_keeps_what_its_borrowers_see(folders):
    """VA's first layer has chunks of 7, the layer that reads its keys chunks of 64: the lender's pages must stay while
    the borrower's chunk lasts (decoding past position 64 * k with the cache poisoned)."""
    from rocmforge_b200 import StepRequest
    m = engine(folders, "VA", "float32")
    toks = random_tokens(vocab("VA"), 200, 13)
    ref = plain_logits(folders, "VA", "float32", toks)
    cache = m.new_cache(max_tokens=64 * 5, max_slots=1)
    s = cache.alloc_slot()
    got = [m.step(cache, [StepRequest(s, toks[:100], [99])]).cpu()]
    for t in toks[100:]:
        poison_free_pages(cache)
        got.append(m.step(cache, [StepRequest(s, [t], [0])]).cpu())
    close(torch.cat(got), ref[99:], "float32", "VA lender and borrower")


def test_positions_beyond_the_table_are_refused(folders):
    from rocmforge_b200 import CacheError, StepRequest
    m = engine(folders, "VA", "float32")
    cache = m.new_cache(max_tokens=1024, max_slots=1)
    s = cache.alloc_slot()
    with pytest.raises(CacheError):
        m.step(cache, [StepRequest(s, random_tokens(vocab("VA"), VILULORN_CONFIGS["VA"]["max_positions"] + 1, 1), [0])])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_greedy_generation_through_the_public_entry_point(folders, dtype):
    """LLM.generate: the scheduler admits unequal prompts, decode steps replay from graphs (the warm-up run before a
    capture must leave the state as it was), requests end at different lengths."""
    import rocmforge_b200 as rf
    name = "VC"
    llm = rf.LLM(folders(name, dtype), dtype=dtype)
    prompts = [random_tokens(vocab(name), n, 60 + n) for n in (3, 140, 11)]
    out = llm.generate(prompts, max_tokens=12, temperature=0.0, stop_token_ids=[])
    for p, r in zip(prompts, out):
        assert len(r.tokens) == 12
        seq = list(p)
        for k, tok in enumerate(r.tokens):
            row = plain_logits(folders, name, dtype, seq)[-1]
            best = int(torch.argmax(row))
            if dtype == "float32":
                assert tok == best or float(row[best] - row[tok]) <= 1e-5, f"request of {len(p)} tokens, generated token {k}: {tok}, plain {best}"
            seq.append(tok)
            if dtype != "float32":
                break
        if dtype != "float32":
            # bfloat16: against the engine's own step function, token by token without graphs (the plain model may take
            # another expert on a nearly tied token): the generated token is the best one there, or next to it
            from rocmforge_b200 import StepRequest
            cache = llm.model.new_cache(max_tokens=512, max_slots=1)
            s = cache.alloc_slot()
            row = llm.model.step(cache, [StepRequest(s, list(p), [len(p) - 1])]).cpu()[0]
            for tok in r.tokens:
                assert float(row.max() - row[tok]) <= 2e-2 * float(row.abs().max())
                row = llm.model.step(cache, [StepRequest(s, [tok], [0])]).cpu()[0]


def test_command_line(folders):
    """bin/rocmforge on a Vilulorn folder: greedy tokens equal the plain model's."""
    folder = folders("VA", "float32")
    prompt = random_tokens(vocab("VA"), 9, 91)
    out = subprocess.run([os.path.join(ROOT, "bin", "rocmforge"), "--model", folder, "--dtype", "float32", "--prompt-ids",
                          ",".join(map(str, prompt)), "--max-tokens", "5", "--temperature", "0", "--stop-ids", "", "--debug"],
                         capture_output=True, text=True, timeout=600)
    assert out.returncode == 0, out.stderr[-2000:]
    ids = [int(l.split("token_id=")[1]) for l in out.stderr.splitlines() if l.startswith("[Generated]")]
    seq = list(prompt)
    for tok in ids:
        row = plain_logits(folders, "VA", "float32", seq)[-1]
        assert tok == int(torch.argmax(row)) or float(row.max() - row[tok]) <= 1e-5
        seq.append(tok)
    assert len(ids) == 5


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_replay_program(folders, tmp_path, dtype):
    """bin/trace_run on a Vilulorn folder: whole prompts, a prompt and its last tokens one by one, and a batch."""
    name = "VA"
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


def _chunk_case(chunk, T, i, dev, dtype, nh, nkv, d, dv):
    """Queries, keys and values in which, for the query at position i, the first key of i's chunk and the key just before
    it stand out (the outside one more): the output is the inside key's value, and not a trace of the outside key's."""
    torch.manual_seed(chunk * 1000 + i)
    q = torch.randn(T, nh, d, device=dev) * 0.05
    k = torch.randn(T, nkv, d, device=dev) * 0.05
    v = torch.randn(T, nkv, dv, device=dev)
    inside = i // chunk * chunk
    outside = inside - 1
    q[i] = 0.0
    q[i, :, 0] = 40.0
    k[inside, :, 0] = 1.0
    if outside >= 0:
        k[outside, :, 0] = 2.0                    # would win if it were seen
        v[outside] = 1000.0
    return q.to(dtype), k.to(dtype), v.to(dtype), inside


@pytest.mark.parametrize("chunk,i", [(1, 299), (5, 299), (64, 255), (64, 256), (65, 129), (65, 130), (120, 239), (120, 240),
                                     (200, 299), (300, 299)])
def test_attention_sees_exactly_its_chunk(chunk, i):
    """Positions just before and on a chunk's first position, chunk edges on and off page borders; the query in a prompt
    and as a step of its own; heads of 24 with values of 40 on the generic kernel (32-bit)."""
    from rocmforge_b200 import kernels
    dev, T, nh, nkv, d, dv = "cuda", 300, 4, 2, 24, 40
    q, k, v, inside = _chunk_case(chunk, T, i, dev, torch.float32, nh, nkv, d, dv)
    kp, vp, bt = _paged(k, v)
    zero = torch.zeros(1, dtype=torch.int32, device=dev)
    for rows in (range(i + 1), [i]):
        pos = torch.tensor(list(rows), dtype=torch.int32, device=dev)
        seq = torch.zeros(len(pos), dtype=torch.int32, device=dev)
        out = kernels.attention_generic(q[list(rows)].reshape(len(pos), nh * d).contiguous(), nh, nkv, d, kp, vp, seq, pos,
                                        zero, bt, 1.0, None, v_head_dim=dv, chunk=chunk).reshape(len(pos), nh, dv)
        assert (out[-1] - v[inside][[0, 0, 1, 1]]).abs().max() < 1e-3, f"chunk {chunk}, query {i}: the wrong keys are seen"


@pytest.mark.parametrize("hd", [64, 128])
@pytest.mark.parametrize("chunk,i", [(64, 447), (64, 448), (120, 359), (120, 360), (130, 389), (130, 390), (33, 395), (500, 449)])
def test_tensor_core_attention_sees_exactly_its_chunk(chunk, i, hd):
    """The same on the bfloat16 kernels: the tcgen05 prompt attention (tiles of 128 queries whose rows lie in different
    chunks) and the clustered decode attention, against the generic kernel on every row."""
    from rocmforge_b200 import kernels
    dev, T, nh, nkv = "cuda", 450, 4, 2
    q, k, v, inside = _chunk_case(chunk, T, i, dev, torch.bfloat16, nh, nkv, hd, hd)
    kp, vp, bt = _paged(k, v)
    zero = torch.zeros(1, dtype=torch.int32, device=dev)
    pos = torch.arange(T, dtype=torch.int32, device=dev)
    seq = torch.zeros(T, dtype=torch.int32, device=dev)
    q2 = q.reshape(T, nh * hd).contiguous()
    ref = kernels.attention_generic(q2, nh, nkv, hd, kp, vp, seq, pos, zero, bt, 0.3, None, chunk=chunk).float()
    tiles = torch.tensor([[0, r] for r in range(0, T, 128)], dtype=torch.int32, device=dev).flip(0).reshape(-1).contiguous()
    start, nnew = zero, torch.tensor([T], dtype=torch.int32, device=dev)
    cu = torch.tensor([0, T], dtype=torch.int32, device=dev)
    got = kernels.attention_prefill_tc(q2, nh, nkv, hd, kp, vp, tiles, zero, start, nnew, cu, bt, 0.3, None, chunk=chunk).float()
    assert (got - ref).abs().max() <= 2e-2 * ref.abs().max().clamp(min=1.0), f"prompt kernel, chunk {chunk}"
    assert (got[i].reshape(nh, hd) - v[inside][[0, 0, 1, 1]].float()).abs().max() < 0.1
    one = kernels.attention_decode_warps(q2[i:i + 1].contiguous(), nh, nkv, hd, kp, vp, zero, pos[i:i + 1].contiguous(), zero, bt,
                                         0.3, None, chunk=chunk).float()
    assert (one[0] - ref[i]).abs().max() <= 2e-2 * ref[i].abs().max().clamp(min=1.0), f"decode kernel, chunk {chunk}"
    assert (one[0].reshape(nh, hd) - v[inside][[0, 0, 1, 1]].float()).abs().max() < 0.1


def test_head_norm_weights_and_neighbour_rotation_against_the_plain_functions():
    """q | k | v | gate rows through the cache writer: weighted norms per head, neighbouring pairs of the first 12 of 20
    elements turned with stretched frequencies, q out, k and v in their pages, the gate's columns untouched."""
    from rocmforge_b200 import kernels
    from rocmforge_b200.parts.rope import NeoxRope
    torch.manual_seed(1)
    dev, T, nh, nkv, d, dv, rot, eps = "cuda", 90, 4, 2, 20, 12, 12, 1e-5
    scaling = dict(factor=8.0, low=1.0, high=4.0, original=64)
    rope = NeoxRope(d, 100.0, rotary_dim=rot, interleaved=True, scaling=scaling)
    rope.prepare(dev)
    want_f = P.scaled_frequencies(rot, 100.0, scaling)
    assert torch.allclose(rope.inv_freq_host.double(), want_f, rtol=1e-6)
    assert not torch.allclose(want_f, P.scaled_frequencies(rot, 100.0, None))            # the stretch does something here
    row = torch.randn(T, (nh + nkv) * d + nkv * dv + 7, device=dev)
    qw, kw = torch.rand(d, device=dev) + 0.5, torch.rand(d, device=dev) + 0.5
    pos = torch.arange(T, dtype=torch.int32, device=dev) + 3
    seq = torch.zeros(T, dtype=torch.int32, device=dev)
    zero = torch.zeros(1, dtype=torch.int32, device=dev)
    kp = torch.zeros(3, nkv, 64, d, device=dev)
    vp = torch.zeros(3, nkv, 64, dv, device=dev)
    bt = torch.tensor([[2, 0, 1]], dtype=torch.int32, device=dev)
    q = kernels.head_norm_kv_write(row, nh, nkv, d, dv, rope.inv_freq, seq, pos, zero, bt, kp, vp, True, rot_dim=rot,
                                   interleaved=True, unit_norm_eps=eps, q_norm_weight=qw, k_norm_weight=kw)
    r64 = row.double().cpu()
    positions = pos.cpu()
    wq = P.rotate_neighbours(P.rms_norm(r64[:, : nh * d].reshape(T, nh, d), qw.double().cpu(), eps), positions, rot, want_f)
    wk = P.rotate_neighbours(P.rms_norm(r64[:, nh * d: (nh + nkv) * d].reshape(T, nkv, d), kw.double().cpu(), eps), positions, rot, want_f)
    wv = r64[:, (nh + nkv) * d: (nh + nkv) * d + nkv * dv].reshape(T, nkv, dv)
    assert (q.double().cpu().reshape(T, nh, d) - wq).abs().max() < 2e-5
    for t in range(T):
        p = int(pos[t])
        page = int(bt[0, p // 64])
        assert (kp[page, :, p % 64].double().cpu() - wk[t]).abs().max() < 2e-5
        assert (vp[page, :, p % 64].double().cpu() - wv[t]).abs().max() < 1e-6
    # a layer that borrows its keys: only the q heads of a q | gate row are read, nothing is written
    kp2 = kp.clone()
    q2 = kernels.head_norm_kv_write(torch.cat([row[:, : nh * d], row[:, -7:]], dim=1).contiguous(), nh, nkv, d, dv, rope.inv_freq,
                                    seq, pos, zero, bt, kp, vp, False, rot_dim=rot, interleaved=True, unit_norm_eps=eps,
                                    q_norm_weight=qw)
    assert torch.equal(q2, q) and torch.equal(kp, kp2)


@pytest.mark.parametrize("dim,vdim,heads", [(24, 12, 2), (64, 32, 3), (130, 9, 1), (256, 40, 1), (48, 32, 2)])
def test_gla_scan_against_the_recurrence_and_across_cuts(dim, vdim, heads):
    """The recurrence over 700 tokens of two sequences, once in one step and once cut into steps of many sizes (down to
    one token): the same bits, and the plain recurrence's numbers.  Decays of exactly 1, near 1 and near 0 side by side; a
    token 650 places back, made large in a channel that does not decay, still shows; the same sequence among many others
    gives the same bits."""
    from rocmforge_b200 import kernels
    torch.manual_seed(dim)
    dev, T = "cuda", 700
    state = torch.zeros(3, heads, dim, vdim, device=dev)
    qka = torch.randn(3, 2 * T, heads * dim, device=dev) * dim ** -0.5
    alpha = torch.sigmoid(torch.randn(2 * T, heads * dim, device=dev) * 3 + 2) ** 0.25
    alpha[:, 0] = 1.0                                  # a channel that never forgets
    alpha[:, 1] = 1e-3                                 # and one that forgets at once
    qka[2] = alpha
    v = torch.randn(2 * T, heads * vdim, device=dev)
    v[20] *= 50.0
    qka[1, 20, 0] = 3.0
    cu = torch.tensor([0, T, 2 * T], dtype=torch.int32, device=dev)
    slots = torch.tensor([2, 0], dtype=torch.int32, device=dev)
    whole = kernels.gla_scan(qka, v, state, cu, slots, heads, dim, vdim)
    end_state = state.clone()
    S = torch.zeros(heads, dim, vdim, dtype=torch.float64)
    q64, k64, a64 = (qka[n, :T].double().cpu().reshape(T, heads, dim) for n in range(3))
    v64 = v[:T].double().cpu().reshape(T, heads, vdim)
    want = torch.zeros(T, heads, vdim, dtype=torch.float64)
    for t in range(T):
        S = a64[t][:, :, None] * S + k64[t][:, :, None] * v64[t][:, None, :]
        want[t] = torch.einsum("hdv,hd->hv", S, q64[t])
    got = whole[:T].double().cpu().reshape(T, heads, vdim)
    assert (got - want).abs().max() <= 1e-4 * want.abs().max()
    assert (end_state[2].double().cpu() - S).abs().max() <= 1e-4 * S.abs().max()
    assert (state[1] == 0).all()                                  # a slot that no sequence of the step holds
    assert S[0, 0].abs().max() > 50.0                             # the old token is still there, where nothing decays
    # the same in portions
    state.zero_()
    sizes = [1, 2, 16, 17, 1, 63, 300, 5]
    sizes.append(T - sum(sizes))
    parts, at = [], 0
    for n in sizes:
        rows = torch.cat([torch.arange(at, at + n), torch.arange(T + at, T + at + n)]).to(dev)
        cu_n = torch.tensor([0, n, 2 * n], dtype=torch.int32, device=dev)
        parts.append(kernels.gla_scan(qka[:, rows].contiguous(), v[rows], state, cu_n, slots, heads, dim, vdim))
        at += n
    cut = torch.cat([p[: p.shape[0] // 2] for p in parts] + [p[p.shape[0] // 2:] for p in parts])
    assert torch.equal(cut, whole), "the recurrence depends on how the prompt was cut"
    assert torch.equal(state, end_state)
    # among 400 one-token sequences: the first sequence's first token unchanged
    many = 400
    big_state = torch.zeros(many, heads, dim, vdim, device=dev)
    rows = torch.arange(many, device=dev)
    for one_token in (False, True):                   # the general kernel, and the one for steps of one token a sequence
        big_state.zero_()
        o = kernels.gla_scan(qka[:, rows].contiguous(), v[rows], big_state, torch.arange(many + 1, dtype=torch.int32, device=dev),
                             torch.arange(many, dtype=torch.int32, device=dev), heads, dim, vdim, one_token=one_token)
        assert torch.equal(o[0], whole[0])
    # decoding on from the prompt's state with the one-token kernel: the same bits as the prompt in one step
    state.zero_()
    cu_n = torch.tensor([0, 600, 1200], dtype=torch.int32, device=dev)
    rows = torch.cat([torch.arange(0, 600), torch.arange(T, T + 600)]).to(dev)
    kernels.gla_scan(qka[:, rows].contiguous(), v[rows], state, cu_n, slots, heads, dim, vdim)
    one = torch.tensor([0, 1, 2], dtype=torch.int32, device=dev)
    for t in range(600, T):
        rows = torch.tensor([t, T + t], device=dev)
        step = kernels.gla_scan(qka[:, rows].contiguous(), v[rows], state, one, slots, heads, dim, vdim, one_token=True)
        assert torch.equal(step[0], whole[t]) and torch.equal(step[1], whole[T + t])
    assert torch.equal(state, end_state)


def test_gla_prepare_against_the_plain_decay():
    """alpha = sigmoid(z)^(1/tau) for z from -60 to 60 and tau of 1, 16 and 0.5, q scaled, k passed through."""
    from rocmforge_b200 import kernels
    dev, heads, dim = "cuda", 2, 24
    T = 50
    torch.manual_seed(3)
    proj = torch.randn(T, 2 * heads * dim + 5, device=dev)
    z = torch.linspace(-60, 60, T * heads * dim, device=dev).reshape(T, heads * dim).contiguous()
    for tau in (1.0, 16.0, 0.5):
        qka = kernels.gla_prepare(proj, 0, heads * dim, z, heads, dim, 0.125, tau)
        want = torch.exp(torch.nn.functional.logsigmoid(z.double()) / tau)
        assert (qka[2].double() - want).abs().max() < 2e-6
        assert torch.isfinite(qka).all()
        assert torch.equal(qka[0], proj[:, : heads * dim] * 0.125) and torch.equal(qka[1], proj[:, heads * dim: 2 * heads * dim])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_gla_mixer_against_the_plain_function(dtype):
    """The whole mixer as a part (projections, decay of rank 5, recurrence, weighted head norm, gate, output product) on
    random weights with a norm weight that is not 1, in one step and in two."""
    import rocmforge_b200 as rf
    from rocmforge_b200.parts import MIXERS
    torch.manual_seed(5)
    dev, W, H, D, DV, tau, eps, r = "cuda", 64, 2, 24, 20, 3.0, 1e-5, 5
    dt = TORCH[dtype]
    names = {"q": "q", "k": "k", "v": "v", "g": "g", "o": "o", "a1": "a1", "a2": "a2", "a2_bias": "a2.b", "norm": "norm"}
    mixer = MIXERS.build("gla", hidden=W, n_heads=H, dim=D, vdim=DV, tau=tau, eps=eps, decay_rank=r, names=names)
    Wt = {n: (torch.randn(s.shape) * (0.3 if len(s.shape) == 2 else 1.0)).to(dt) for n, s in mixer.param_specs().items()}
    Wt["norm"] = (torch.rand(DV) + 0.5).to(dt)
    x = torch.randn(40, W).to(dt)
    want = P.gated_linear_attention(x.double(), {"m." + n: t.double() for n, t in Wt.items()}, "m.", dict(heads=H, dim=D, vdim=DV, tau=tau), eps)
    got = _run_mixer(mixer, Wt, x, dt, cuts=[(0, 40)])
    got2 = _run_mixer(mixer, Wt, x, dt, cuts=[(0, 13), (13, 40)])
    tol = 1e-4 if dtype == "float32" else 4e-2
    assert (got.double().cpu() - want).abs().max() <= tol * want.abs().max()
    assert (got2.double().cpu() - want).abs().max() <= tol * want.abs().max()


def _run_mixer(mixer, Wt, x, dt, cuts):
    """A one-layer model around ``mixer`` would need names; here the mixer runs through a minimal step context."""
    import rocmforge_b200 as rf
    from rocmforge_b200.cache import SequenceCache
    from rocmforge_b200.csrc import build
    from rocmforge_b200.engine.batch import DeviceDescriptor, StepBatch, StepRequest
    from rocmforge_b200.engine.context import Options, StepContext
    dev = "cuda"
    build.ensure_built(mixer.cuda_modules(dt) + ["gemm_simt", "gemm_tcgen05"])
    mixer.bind({n: t.to(dev) for n, t in Wt.items()}, dt)

    class Holder:
        options, compute_dtype, device = Options(), dt, torch.device(dev)

        def scratch(self, name, n, dtype):
            return torch.zeros((max(n, 1),), dtype=dtype, device=dev)
    cache = SequenceCache({0: mixer.cache_request()}, max_tokens=256, max_slots=2, dtype=dt, device=dev)
    slot = cache.alloc_slot()
    desc = DeviceDescriptor(dev)
    outs = []
    for a, b in cuts:
        batch = StepBatch([StepRequest(slot, [0] * (b - a), [])], [cache.length(slot)], 10)
        cache.prepare([slot], [b - a])
        desc.upload(batch.pack())
        ctx = StepContext(Holder(), desc.views(batch.T, batch.B, batch.R, batch.extras), T=batch.T, B=batch.B, R=batch.R,
                          is_decode=batch.is_decode, max_new=batch.max_new, max_end=batch.max_end, host=batch)
        o = mixer.output(ctx, x[a:b].to(dev).contiguous(), cache.view(0))
        outs.append(o.sum(dim=0) if o.dim() == 3 else o)
        cache.commit([slot], [b - a])
    return torch.cat(outs)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("experts,top,T", [(5, 2, 37), (3, 3, 200), (16, 1, 9), (1, 1, 5)])
def test_scored_experts_against_the_plain_function(dtype, experts, top, T):
    """Sigmoid scores on the experts' inputs, limits that bite on both sides, one expert and all experts per token."""
    from rocmforge_b200.parts import FEED_FORWARDS
    torch.manual_seed(experts * 10 + top)
    dev, W, F, limit = "cuda", 64, 40, 0.7
    dt = TORCH[dtype]
    ffn = FEED_FORWARDS.build("routed_experts", hidden=W, intermediate=F, n_experts=experts, top=top, router_bias=False,
                              scoring="sigmoid", weight_on="input", activation="clamped_glu", limit=limit, glu_alpha=1.702)
    Wt = {n: (torch.randn(s.shape) * (1.0 if n == "router" else 0.25)).to(dt) for n, s in ffn.param_specs().items()}
    x = torch.randn(T, W).to(dt)
    mlp = {"router": {"experts": experts, "top": top}, "expert": {"limit": limit}}
    want = P.scored_experts(x.double(), {"f." + n: t.double() for n, t in Wt.items()}, "f.", mlp)
    g = x.double() @ Wt["e0.gate"].double().T
    assert (g > limit).any() and (g < -limit).any()              # the clamps are exercised
    from rocmforge_b200.csrc import build
    build.ensure_built(ffn.cuda_modules(dt) + ["gemm_simt", "gemm_tcgen05"])
    ffn.bind({n: t.to(dev) for n, t in Wt.items()}, dt)
    from rocmforge_b200.engine.context import Options

    class Ctx:
        options, compute_dtype, device = Options(), dt, torch.device(dev)

        def matmul(self, a, w, bias=None, *, out_f32=False):
            from rocmforge_b200 import kernels
            return kernels.gemm_simt(a, w, bias, out_f32=out_f32)
    got = ffn.output(Ctx(), x.to(dev)).double().cpu()
    if dtype == "float32":
        assert (got - want).abs().max() <= 1e-4 * want.abs().max()
    else:
        err = (got - want).pow(2).mean(dim=1).sqrt() / want.pow(2).mean().sqrt()
        assert float(err.mean()) < 0.03 and float((err < 0.06).double().mean()) >= 0.9


def test_clamped_activation_and_gates_against_torch():
    from rocmforge_b200 import kernels
    torch.manual_seed(9)
    dev = "cuda"
    gu = torch.randn(33, 2 * 17, device=dev) * 3
    sc = torch.rand(33, device=dev)
    for scale in (None, sc):
        a = kernels.clamped_glu(gu, 2.0, 1.702, row_scale=scale)
        x = gu.double() * (scale.double()[:, None] if scale is not None else 1.0)
        g, u = x[:, 0::2].clamp(max=2.0), x[:, 1::2].clamp(-2.0, 2.0)
        assert (a.double() - g * torch.sigmoid(1.702 * g) * (u + 1)).abs().max() < 1e-5
    o, gate = torch.randn(20, 48, device=dev), torch.randn(20, 100, device=dev)
    got = kernels.sigmoid_gate(o, gate[:, 30:78])
    assert (got.double() - o.double() * torch.sigmoid(gate[:, 30:78].double())).abs().max() < 1e-6
    z = torch.randn(50, 7, device=dev) * 4
    idx, w = kernels.moe_route(z, 3, "sigmoid")
    top = torch.topk(z, 3, dim=1)
    assert torch.equal(idx.long(), top.indices) and (w - torch.sigmoid(top.values)).abs().max() < 1e-6


def test_embedding_with_positions_and_the_stream_read_as_it_is():
    from rocmforge_b200 import kernels
    torch.manual_seed(2)
    dev = "cuda"
    for dt in (torch.float32, torch.bfloat16):
        table, ptab = torch.randn(50, 36, device=dev).to(dt), torch.randn(20, 36, device=dev).to(dt)
        ids = torch.randint(0, 50, (30,), dtype=torch.int32, device=dev)
        pos = torch.randint(0, 20, (30,), dtype=torch.int32, device=dev)
        h, y = kernels.embed_positions(table, ids, ptab, pos, rounded=True)
        want = table.float()[ids.long()] + ptab.float()[pos.long()]
        assert torch.equal(h, want) and torch.equal(y, want.to(dt))
        h2, y2 = kernels.embed_positions(table, ids, None, None)
        assert torch.equal(h2, table.float()[ids.long()]) and y2 is None
    # an update whose next reader takes the stream itself
    h = torch.randn(9, 64, device=dev)
    a = torch.randn(3, 9, 64, device=dev)
    w = torch.rand(64, device=dev) + 0.5
    before = h.clone()
    y = kernels.branch_norm_add(h, [(a, None)], w, 1e-5, torch.bfloat16, next_rounded=True)
    m = a.double().sum(0)
    want = before.double() + m / torch.sqrt((m * m).mean(dim=1, keepdim=True) + 1e-5) * w.double()
    assert (h.double() - want).abs().max() < 1e-5 and torch.equal(y, h.to(torch.bfloat16))
    assert torch.equal(kernels.round_rows(h, torch.bfloat16), h.to(torch.bfloat16))
